"""Plain, slow CPU oracle of the Sunutar design, one function per mechanism, written from the design's equations.

It shares no code with the engine: dense loops over tokens and heads in float64, the whole sequence at once or token by
token (``Oracle.step`` carries the caches a token-by-token run needs).  ``cfg`` is the dictionary of ``config.json``,
``w`` maps tensor names to float64 tensors.

Notation: a layer is  x <- x + m * norm_b(sublayer(norm_a(x)))  for the mixer and then the feed-forward, with plain
RMS-norm weights.  The mixer runs two branches on the same input and adds them with two scales:
  * windowed attention: grouped-query heads, biases, RMS norm over the whole query / key projection, score
    c * tanh(q.k * scale / c) - slope_h * (i - j), keys 0 <= i - j < window, softmax whose denominator holds an extra 1;
  * a state-space branch (scalar decay per head): causal convolution + silu on (x | B | C), dt = softplus(dt + bias),
    S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, gate silu(z) before a grouped RMS norm.
Feed-forwards: g = min(gate, L), u = clamp(up, -L, L), y = g * sigmoid(1.702 g) * (u + 1), either dense or routed
(sigmoid scores, the `top` best, the score multiplies the expert's INPUT, no renormalisation).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * weight


def head_slopes(heads: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)], dtype=F)


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, past: Optional[dict] = None) -> torch.Tensor:
    """h [n, width] -> [n, width].  ``past``: {"k": [pos0, G*d], "v": [pos0, G*dv]} of earlier positions, extended in place."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    window, cap, scale = m["mask"]["size"], m["softcap"], m["scale"]
    q = h @ w[p + "q"].T + w[p + "q.b"]
    k = h @ w[p + "k"].T + w[p + "k.b"]
    v = h @ w[p + "v"].T + w[p + "v.b"]
    q = rms_norm(q, w[p + "q.norm"], eps)
    k = rms_norm(k, w[p + "k.norm"], eps)
    pos0 = 0
    if past is not None:
        if "k" in past:
            pos0 = past["k"].shape[0]
            k = torch.cat([past["k"], k], 0)
            v = torch.cat([past["v"], v], 0)
        past["k"], past["v"] = k, v
    n = h.shape[0]
    slopes = head_slopes(H)
    out = torch.zeros(n, H * dv, dtype=F)
    for t in range(n):
        i = pos0 + t
        lo = max(0, i - window + 1)
        for hh in range(H):
            g = hh // (H // G)
            qv = q[t, hh * d:(hh + 1) * d]
            ks = k[lo:i + 1, g * d:(g + 1) * d]
            vs = v[lo:i + 1, g * dv:(g + 1) * dv]
            s = (ks @ qv) * scale
            s = cap * torch.tanh(s / cap)
            s = s - slopes[hh] * (i - torch.arange(lo, i + 1, dtype=F))
            e = torch.exp(s)
            pr = e / (1.0 + e.sum())
            out[t, hh * dv:(hh + 1) * dv] = pr @ vs
    return out @ w[p + "o"].T + w[p + "o.b"]


def state_space(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float, past: Optional[dict] = None) -> torch.Tensor:
    """h [n, width] -> [n, width].  ``past``: {"S": [heads, N, vdim], "conv": [taps - 1, channels]}, updated in place."""
    H, dv, N, G, taps, parts = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner = H * dv
    n = h.shape[0]
    proj = h @ w[p + "in"].T
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    dt = proj[:, 2 * inner + 2 * G * N:]
    channels = xbc.shape[1]
    before = past["conv"] if past is not None and "conv" in past else torch.zeros(taps - 1, channels, dtype=F)
    padded = torch.cat([before, xbc], 0)                      # row r + taps - 1 is token r
    cw, cb = w[p + "conv"], w[p + "conv.b"]
    conv = torch.zeros(n, channels, dtype=F)
    for t in range(n):
        acc = cb.clone()
        for j in range(taps):                                 # the last column multiplies the current token
            acc = acc + cw[:, j] * padded[t + j]
        conv[t] = acc
    conv = conv * torch.sigmoid(conv)
    if past is not None:
        past["conv"] = padded[padded.shape[0] - (taps - 1):].clone()
    x = conv[:, :inner]
    B = conv[:, inner:inner + G * N]
    C = conv[:, inner + G * N:]
    dt = torch.nn.functional.softplus(dt + w[p + "dt_bias"])
    A = torch.exp(w[p + "A_log"])
    S = past["S"] if past is not None and "S" in past else torch.zeros(H, N, dv, dtype=F)
    y = torch.zeros(n, inner, dtype=F)
    for t in range(n):
        for hh in range(H):
            g = hh // (H // G)
            xt = x[t, hh * dv:(hh + 1) * dv]
            Bt = B[t, g * N:(g + 1) * N]
            Ct = C[t, g * N:(g + 1) * N]
            S[hh] = torch.exp(-A[hh] * dt[t, hh]) * S[hh] + dt[t, hh] * torch.outer(Bt, xt)
            y[t, hh * dv:(hh + 1) * dv] = S[hh].T @ Ct + w[p + "D"][hh] * xt
    if past is not None:
        past["S"] = S
    y = y * (z * torch.sigmoid(z))
    y = rms(y.view(n, parts, inner // parts), eps).reshape(n, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps, past=None):
    left = window_attention(h, w, p + "left.", m["left"], eps, None if past is None else past.setdefault("left", {}))
    right = state_space(h, w, p + "right.", m["right"], eps, None if past is None else past.setdefault("right", {}))
    return m["left_scale"] * left + m["right_scale"] * right


def clamped_glu(h: torch.Tensor, w_gate, w_up, w_down, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ w_gate.T, max=limit)
    u = torch.clamp(h @ w_up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w_down.T


def route(h: torch.Tensor, w_router: torch.Tensor, top: int):
    """-> chosen experts [n, top] and their sigmoid scores."""
    s = torch.sigmoid(h @ w_router.T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return clamped_glu(h, w[p + "gate"], w[p + "up"], w[p + "down"], mlp["limit"])
    idx, val = route(h, w[p + "router"], mlp["router"]["top"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), val[t]):
            q = f"{p}e{e}."
            out[t] += clamped_glu((s * h[t])[None], w[q + "gate"], w[q + "up"], w[q + "down"], mlp["expert"]["limit"])[0]
    return out


class Oracle:
    """The whole model.  ``forward(tokens)`` runs a sequence from its start; ``step(tokens)`` continues from what earlier
    ``step`` calls left (caches of every layer)."""

    def __init__(self, cfg: dict, weights: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.w = {k: v.to(F) for k, v in weights.items()}
        self.past: List[dict] = [{} for _ in cfg["layers"]]

    def reset(self) -> None:
        self.past = [{} for _ in self.cfg["layers"]]

    def _run(self, tokens, past, layers_out=None) -> torch.Tensor:
        cfg, w = self.cfg, self.w
        eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
        x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
        for i, L in enumerate(cfg["layers"]):
            p = f"l{i}."
            if L["type"] != "parallel":
                raise ValueError(f"unknown layer type {L['type']!r}")
            y = parallel_mixer(rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps, None if past is None else past[i])
            x = x + mult * rms_norm(y, w[p + "norm1b"], eps)
            if L.get("mlp"):
                y = feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", L["mlp"])
                x = x + mult * rms_norm(y, w[p + "norm2b"], eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        return rms_norm(x, w["final.norm"], eps) @ w["embed"].T

    def forward(self, tokens, layers_out=None) -> torch.Tensor:
        return self._run(tokens, None, layers_out)

    def step(self, tokens) -> torch.Tensor:
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

    out["embed"] = torch.randn(V, D, generator=g)
    vec("final.norm", D, 1.0)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        for nm in ("norm1", "norm1b"):
            vec(p + nm, D, 1.0)
        a, r = L["mixer"]["left"], L["mixer"]["right"]
        q = p + "mix.left."
        mat(q + "q", a["heads"] * a["dim"], D, 2.0); vec(q + "q.b", a["heads"] * a["dim"])
        mat(q + "k", a["kv_heads"] * a["dim"], D, 2.0); vec(q + "k.b", a["kv_heads"] * a["dim"])
        mat(q + "v", a["kv_heads"] * a["vdim"], D); vec(q + "v.b", a["kv_heads"] * a["vdim"])
        vec(q + "q.norm", a["heads"] * a["dim"], 1.0); vec(q + "k.norm", a["kv_heads"] * a["dim"], 1.0)
        mat(q + "o", D, a["heads"] * a["vdim"]); vec(q + "o.b", D)
        q = p + "mix.right."
        inner, gn = r["heads"] * r["vdim"], r["groups"] * r["state"]
        mat(q + "in", 2 * inner + 2 * gn + r["heads"], D)
        out[q + "conv"] = torch.randn(inner + 2 * gn, r["conv"], generator=g) * 0.5
        vec(q + "conv.b", inner + 2 * gn)
        vec(q + "dt_bias", r["heads"], -1.0, 1.0)
        out[q + "A_log"] = torch.log(torch.rand(r["heads"], generator=g) * 1.5 + 0.05)
        vec(q + "D", r["heads"], 1.0, 0.3)
        vec(q + "norm", inner, 1.0)
        mat(q + "o", D, inner)
        mlp = L.get("mlp")
        if mlp:
            for nm in ("norm2", "norm2b"):
                vec(p + nm, D, 1.0)
            if mlp["kind"] == "dense":
                mat(p + "mlp.gate", mlp["ff"], D, 2.0); mat(p + "mlp.up", mlp["ff"], D, 2.0); mat(p + "mlp.down", D, mlp["ff"])
            else:
                ff = mlp["expert"]["ff"]
                for e in range(mlp["router"]["experts"]):
                    mat(f"{p}mlp.e{e}.gate", ff, D, 2.0); mat(f"{p}mlp.e{e}.up", ff, D, 2.0); mat(f"{p}mlp.e{e}.down", D, ff)
                mat(p + "mlp.router", mlp["router"]["experts"], D, 3.0)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in out.items()}
