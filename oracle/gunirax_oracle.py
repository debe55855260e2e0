"""Plain, slow CPU oracle of the Gunirax design, one function per mechanism, written from the design's equations.

It shares no code with the engine: dense loops over tokens and heads in float64, the whole sequence at once or token by
token (``Oracle.step`` carries the caches a token-by-token run needs).  ``cfg`` is the dictionary of ``config.json``,
``w`` maps tensor names to float64 tensors.

Notation.  A layer is  x <- x + mixer(n1(x)),  x <- x + ff(n2(x))  with the Dynamic-Tanh norm
n(x) = tanh(alpha x) * weight + shift.  A span of layers may run several times with the same weights; every pass after
the first starts by adding the embedding output to the stream.  Mixers:
  * "parallel": two branches on the same input, each projected back to the width, RMS-normed there, then averaged --
      - sigmoid attention: grouped-query heads with biased q/k projections, the values being the key projection itself;
        interleaved rotary pairs on the leading coordinates with frequencies stretched band by band; a weightless RMS
        division of q and k per head; weight(i, j) = sigmoid(q_i.k_j * scale + bias_h) for j <= i in i's chunk of the
        positions; the heads' weight maps are mixed by a matrix before they meet the values; one output gate per head;
      - lightning attention: silu'd q, k, v, one constant decay per head, S <- decay S + k v^T, o = S^T q; RMS norm over
        all heads together, sigmoid gate per channel;
  * "hgrn2": q = silu(.), forget gate f = low + (1 - low) sigmoid(.), S <- diag(f) S + (1 - f) v^T, o = S^T q, RMS norm
    per head.
Feed-forwards: down(silu(gate) * up), or a routed mixture of down(relu(up)^2) experts (sigmoid scores, a correction
added for the choice only, groups ranked by their two best choice scores, normalised weights times a scale) plus one
shared expert of the same form.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def dyt(x: torch.Tensor, w: Dict[str, torch.Tensor], name: str) -> torch.Tensor:
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def rotary_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i/dims), stretched band by band: long wavelengths are divided by `factor`, short ones kept, the band
    between blended linearly in original/wavelength."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F)
    sc = rot.get("scaling")
    if not sc:
        return f
    factor, low, high, orig = sc["factor"], sc["low"], sc["high"], sc["original"]
    out = f.clone()
    for i in range(dims // 2):
        wl = 2.0 * math.pi / float(f[i])
        if wl < orig / high:
            continue
        if wl > orig / low:
            out[i] = f[i] / factor
        else:
            s = (orig / wl - low) / (high - low)
            out[i] = (1.0 - s) * f[i] / factor + s * f[i]
    return out


def rotate(x: torch.Tensor, pos: torch.Tensor, freq: torch.Tensor) -> torch.Tensor:
    """x [n, heads, d]; pairs (2i, 2i+1), i < len(freq), turn by pos * freq_i; the other coordinates pass."""
    out = x.clone()
    ang = pos.to(F)[:, None, None] * freq[None, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    r = 2 * freq.numel()
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    out[..., 0:r:2] = u * c - v * s
    out[..., 1:r:2] = v * c + u * s
    return out


def sigmoid_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, past: Optional[dict] = None) -> torch.Tensor:
    """h [n, width] -> [n, width].  ``past``: {"k": [pos0, G, d] rotated and normed, "v": [pos0, G, d]}, extended in place."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    assert dv == d, "the values are the key projection"
    n = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(n, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(n, G, d)
    v = k.clone()
    pos0 = past["k"].shape[0] if past is not None and "k" in past else 0
    pos = torch.arange(pos0, pos0 + n)
    freq = rotary_frequencies(m["rot"])
    q = rms(rotate(q, pos, freq), eps)
    k = rms(rotate(k, pos, freq), eps)
    if past is not None:
        if "k" in past:
            k = torch.cat([past["k"], k], 0)
            v = torch.cat([past["v"], v], 0)
        past["k"], past["v"] = k, v
    chunk = m["mask"]["size"]
    talk, pb = w[p + "talk"], w[p + "pb"]
    gate = torch.sigmoid(h @ w[p + "g"].T)                      # [n, H]
    out = torch.zeros(n, H, dv, dtype=F)
    for t in range(n):
        i = pos0 + t
        lo = (i // chunk) * chunk
        wt = torch.zeros(H, i + 1 - lo, dtype=F)
        for hh in range(H):
            g = hh // (H // G)
            wt[hh] = torch.sigmoid((k[lo:i + 1, g] @ q[t, hh]) * m["scale"] + pb[hh])
        mixed = talk @ wt                                       # [H, keys]
        for hh in range(H):
            g = hh // (H // G)
            out[t, hh] = (mixed[hh] @ v[lo:i + 1, g]) * gate[t, hh]
    return out.reshape(n, H * dv) @ w[p + "o"].T


def lightning_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, past: Optional[dict] = None) -> torch.Tensor:
    """h [n, width] -> [n, width].  ``past``: {"S": [heads, d, dv]}, updated in place."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = silu(h @ w[p + "q"].T).view(n, H, d)
    k = silu(h @ w[p + "k"].T).view(n, H, d)
    v = silu(h @ w[p + "v"].T).view(n, H, dv)
    S = past["S"] if past is not None and "S" in past else torch.zeros(H, d, dv, dtype=F)
    S = S.clone()
    o = torch.zeros(n, H, dv, dtype=F)
    for t in range(n):
        for hh in range(H):
            S[hh] = m["decay"][hh] * S[hh] + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    if past is not None:
        past["S"] = S
    y = rms(o.reshape(n, H * dv), eps) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps, past=None):
    pl = past.setdefault("left", {}) if past is not None else None
    pr = past.setdefault("right", {}) if past is not None else None
    a = sigmoid_attention(h, w, p + "left.", m["left"], eps, pl)
    b = lightning_attention(h, w, p + "right.", m["right"], eps, pr)
    return 0.5 * (rms(a, eps) * w[p + "left.out"] + rms(b, eps) * w[p + "right.out"])


def hgrn2(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, past: Optional[dict] = None) -> torch.Tensor:
    """h [n, width] -> [n, width].  ``past``: {"S": [heads, d, dv]}, updated in place."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    n = h.shape[0]
    q = silu(h @ w[p + "q"].T).view(n, H, d)
    v = (h @ w[p + "v"].T).view(n, H, dv)
    low = w[p + "lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w[p + "f"].T + w[p + "f.b"])).view(n, H, d)
    S = past["S"] if past is not None and "S" in past else torch.zeros(H, d, dv, dtype=F)
    S = S.clone()
    o = torch.zeros(n, H, dv, dtype=F)
    for t in range(n):
        for hh in range(H):
            S[hh] = f[t, hh][:, None] * S[hh] + torch.outer(1.0 - f[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    if past is not None:
        past["S"] = S
    y = rms(o, eps) * w[p + "norm"]
    return y.reshape(n, H * dv) @ w[p + "o"].T


def gated_unit(h, w_gate, w_up, w_down):
    return (silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def squared_relu_unit(h, w_up, w_down):
    return torch.relu(h @ w_up.T).pow(2) @ w_down.T


def route(h: torch.Tensor, w_router: torch.Tensor, correction: torch.Tensor, r: dict):
    """-> (chosen experts [n, top], weights [n, top])."""
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.sigmoid(h @ w_router.T)
    choice = s + correction
    size = E // groups["count"]
    ids, wts = [], []
    for t in range(h.shape[0]):
        c = choice[t].clone()
        gs = [float(torch.sort(c[g * size:(g + 1) * size], descending=True).values[:2].sum()) for g in range(groups["count"])]
        order = sorted(range(groups["count"]), key=lambda g: (-gs[g], g))
        for g in order[groups["keep"]:]:
            c[g * size:(g + 1) * size] = -math.inf
        pick = sorted(range(E), key=lambda e: (-float(c[e]), e))[:top]
        sc = s[t, pick]
        ids.append(pick)
        wts.append(sc / (sc.sum() + 1e-20) * r["scale"])
    return ids, torch.stack(wts)


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return gated_unit(h, w[p + "gate"], w[p + "up"], w[p + "down"])
    ids, wts = route(h, w[p + "router"], w[p + "correction"], mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for k, e in enumerate(ids[t]):
            out[t] += wts[t, k] * squared_relu_unit(h[t:t + 1], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + squared_relu_unit(h, w[p + "shared.up"], w[p + "shared.down"])
    return out


def layer_runs(cfg: dict) -> List[tuple]:
    """(layer index, whether the embedding output is added before it) of every layer run, in execution order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    if times <= 1 or b <= a:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(a)]
    for rep in range(times):
        runs += [(i, rep > 0 and i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


class Oracle:
    def __init__(self, cfg: dict, weights: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.w = {k: v.to(F) for k, v in weights.items()}
        self.runs = layer_runs(cfg)
        self.reset()

    def reset(self) -> None:
        self.past = [dict() for _ in self.runs]

    def _run(self, tokens, past, layers_out=None) -> torch.Tensor:
        cfg, w, eps = self.cfg, self.w, self.cfg["norm"]["eps"]
        x0 = w["embed"][torch.tensor(list(tokens), dtype=torch.long)] * cfg["embedding"]["scale"]
        x = x0.clone()
        for n, (i, add) in enumerate(self.runs):
            L, p = cfg["layers"][i], f"l{i}."
            if add:
                x = x + x0
            h = dyt(x, w, p + "norm1")
            ps = past[n] if past is not None else None
            if L["type"] == "parallel":
                x = x + parallel_mixer(h, w, p + "mix.", L["mixer"], eps, ps)
            elif L["type"] == "hgrn2":
                x = x + hgrn2(h, w, p + "mix.", L["mixer"], eps, ps)
            else:
                raise ValueError(L["type"])
            if L.get("mlp"):
                x = x + feed_forward(dyt(x, w, p + "norm2"), w, p + "mlp.", L["mlp"])
            if layers_out is not None:
                layers_out.append(x.clone())
        return dyt(x, w, "final.norm") @ w["head"].T

    def forward(self, tokens, layers_out=None) -> torch.Tensor:
        """Logits [n, vocab] of a whole sequence from position 0 (no state is kept)."""
        return self._run(tokens, None, layers_out)

    def step(self, tokens) -> torch.Tensor:
        """Logits of the next tokens of the sequence this oracle has seen so far (``reset`` starts a new one)."""
        return self._run(tokens, self.past)


def random_weights(cfg: dict, seed: int = 0, scale: float = 1.0) -> Dict[str, torch.Tensor]:
    """Random bf16-representable weights for ``cfg`` (names and shapes of a checkpoint)."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    out: Dict[str, torch.Tensor] = {}

    def mat(name, o, i, s=1.0):
        out[name] = torch.randn(o, i, generator=g) * (s * scale / math.sqrt(i))

    def vec(name, n, mean=0.0, s=0.1):
        out[name] = mean + torch.randn(n, generator=g) * s

    def norm(name):
        vec(name, D, 1.0)
        vec(name + ".b", D, 0.0, 0.05)
        out[name + ".alpha"] = torch.tensor(0.4) + 0.1 * torch.rand((), generator=g)

    out["embed"] = torch.randn(V, D, generator=g) / cfg["embedding"]["scale"]
    mat("head", V, D)
    norm("final.norm")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        norm(p + "norm1")
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            q = p + "mix.left."
            mat(q + "q", a["heads"] * a["dim"], D, 2.0); vec(q + "q.b", a["heads"] * a["dim"], 0.0, 0.3)
            mat(q + "k", a["kv_heads"] * a["dim"], D, 2.0); vec(q + "k.b", a["kv_heads"] * a["dim"], 0.0, 0.3)
            out[q + "talk"] = torch.eye(a["heads"]) * 0.7 + torch.randn(a["heads"], a["heads"], generator=g) * 0.3
            vec(q + "pb", a["heads"], -1.0, 0.5)
            mat(q + "g", a["heads"], D, 2.0)
            mat(q + "o", D, a["heads"] * a["vdim"])
            q = p + "mix.right."
            for nm in ("q", "k"):
                mat(q + nm, r["heads"] * r["dim"], D, 2.0)
            for nm in ("v", "g"):
                mat(q + nm, r["heads"] * r["vdim"], D, 2.0)
            mat(q + "o", D, r["heads"] * r["vdim"])
            vec(q + "norm", r["heads"] * r["vdim"], 1.0)
            vec(p + "mix.left.out", D, 1.0); vec(p + "mix.right.out", D, 1.0)
        else:
            q = p + "mix."
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            mat(q + "q", hd, D, 2.0); mat(q + "f", hd, D, 2.0); vec(q + "f.b", hd, 1.0, 1.0)
            out[q + "lower"] = torch.rand(hd, generator=g) * 0.9
            mat(q + "v", hv, D, 2.0)
            mat(q + "o", D, hv)
            vec(q + "norm", m["vdim"], 1.0)
        mlp = L.get("mlp")
        if mlp:
            norm(p + "norm2")
            if mlp["kind"] == "dense":
                mat(p + "mlp.gate", mlp["ff"], D, 2.0); mat(p + "mlp.up", mlp["ff"], D, 2.0); mat(p + "mlp.down", D, mlp["ff"])
            else:
                ff = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    mat(f"{p}mlp.e{e}.up", ff, D, 2.0); mat(f"{p}mlp.e{e}.down", D, ff)
                mat(p + "mlp.router", mlp["router"]["experts"], D, 3.0)
                vec(p + "mlp.correction", mlp["router"]["experts"], 0.0, 0.2)
                if mlp.get("shared"):
                    mat(p + "mlp.shared.up", mlp["shared"]["ff"], D, 2.0); mat(p + "mlp.shared.down", D, mlp["shared"]["ff"])
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in out.items()}
