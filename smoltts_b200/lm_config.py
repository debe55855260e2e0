"""Configuration of the hybrid language models (``config.json`` with an ``"architecture"`` key).

A model is a list of layers; each layer names its token mixer (``type``) with the mixer's sizes and its feed-forward
(``mlp`` or null).  ``loop`` repeats a span of layers with shared weights; every repetition ("layer run") owns its own
key/value cache or recurrent state.  Every size and every constant that can differ between models is read from the
file; what the design fixes is a class constant of the mixer's spec.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional

# values of SMOL_LM_MIX_* (include/smoltts_b200_lm.h)
MIXER_KINDS = {"attention": 0, "general_delta": 1, "latent_attention": 2, "gla": 3, "state_space": 4, "sigmoid_attention": 5,
               "lightning": 6, "hgrn2": 7}
MLP_KINDS = {None: 0, "dense": 1}                        # SMOL_LM_MLP_* of Pamasun: "dense" = up, PolyNorm, down
# SMOL_LM_MLP_* of Maferax: "dense" = gated (tanh-form gelu), "moe" = routed mixture of gated (silu) experts
MAFERAX_MLP_KINDS = {None: 0, "dense": 2, "moe": 3}
ACT_GELU_TANH, ACT_SILU, ACT_CLAMPED, ACT_RELU_SQUARED = 0, 1, 2, 3      # SMOL_LM_ACT_*
ROUTE_SOFTMAX, ROUTE_SIGMOID = 0, 1                      # SMOL_LM_ROUTE_*
BLOCK_SANDWICH, BLOCK_POSTNORM, BLOCK_PRENORM = 0, 1, 2   # SMOL_LM_BLOCK_*
NORM_RMS, NORM_DYT = 0, 1                                # SMOL_LM_NORM_*


@dataclass
class MixerSpec:
    kind: str
    heads: int
    dim: int
    kv_heads: int = 0           # attention only
    vdim: int = 0               # attention only
    scale: float = 1.0          # attention only: multiplies q.k
    # constants of the generalized delta rule (fixed by the design, parameters of the kernels)
    decay_coef: float = math.exp(-0.5)
    unit_eps: float = 1e-6

    @classmethod
    def from_dict(cls, kind: str, d: Dict[str, Any]) -> "MixerSpec":
        if kind not in ("attention", "general_delta"):
            raise ValueError(f"unknown mixer type {kind!r}; have ['attention', 'general_delta']")
        if kind == "attention":
            # kv_heads and vdim default to heads and dim (plain multi-head attention with square heads)
            return cls(kind, int(d["heads"]), int(d["dim"]), int(d.get("kv_heads", d["heads"])), int(d.get("vdim", d["dim"])), float(d["scale"]))
        return cls(kind, int(d["heads"]), int(d["dim"]), int(d["heads"]), int(d["dim"]))

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "attention":
            return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        return {"heads": self.heads, "dim": self.dim}


@dataclass
class LayerSpec:
    mixer: MixerSpec
    mlp_kind: Optional[str] = None
    ff: int = 0

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LayerSpec":
        mlp = d.get("mlp")
        kind = mlp["kind"] if mlp else None
        if kind not in MLP_KINDS:
            raise ValueError(f"unknown feed-forward kind {kind!r}")
        return cls(MixerSpec.from_dict(d["type"], d["mixer"]), kind, int(mlp["ff"]) if mlp else 0)

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.mixer.kind, "mixer": self.mixer.to_dict(),
                "mlp": {"kind": self.mlp_kind, "ff": self.ff} if self.mlp_kind else None}


@dataclass
class PamasunConfig:
    architecture: str = "Pamasun"
    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    norm_eps: float = 1e-5
    layers: List[LayerSpec] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    extra: Dict[str, Any] = field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "PamasunConfig":
        loop = d.get("loop") or {}
        known = {"architecture", "vocab", "width", "embedding", "norm", "layers", "loop"}
        return cls(architecture=d.get("architecture", "Pamasun"), vocab=int(d["vocab"]), width=int(d["width"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   norm_eps=float((d.get("norm") or {}).get("eps", 1e-5)),
                   layers=[LayerSpec.from_dict(x) for x in d["layers"]],
                   loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)), loop_times=int(loop.get("times", 1)),
                   extra={k: v for k, v in d.items() if k not in known})

    @classmethod
    def from_pretrained(cls, pathname: str) -> "PamasunConfig":
        path = Path(pathname)
        if path.is_dir():
            path = path / "config.json"
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.extra)
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width, embedding={"scale": self.embedding_scale},
                 norm={"eps": self.norm_eps}, layers=[x.to_dict() for x in self.layers],
                 loop={"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times})
        return d

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=1, sort_keys=True)

    def layer_runs(self) -> List[int]:
        """Layer index of every layer run, in execution order."""
        n, a, b = len(self.layers), self.loop_start, self.loop_stop
        if b <= a or self.loop_times == 1:
            if self.loop_times < 1:
                raise ValueError("loop.times must be at least 1")
            return list(range(n))
        if not (0 <= a < b <= n) or self.loop_times < 1:
            raise ValueError(f"loop {a}..{b} x {self.loop_times} does not fit {n} layers")
        return list(range(a)) + list(range(a, b)) * self.loop_times + list(range(b, n))

    def tensor_shapes(self, rank_of: Optional[Dict[int, int]] = None) -> Dict[str, tuple]:
        """Checkpoint tensor names and shapes.  The decay projection's inner size is not in the configuration: it is read
        from the checkpoint (``rank_of[layer]``), 8 where unknown."""
        D, V = self.width, self.vocab
        out: Dict[str, tuple] = {"embed": (V, D), "head": (V, D), "final.norm": (D,)}
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L.mixer
            for nm in ("norm1", "norm1b", "ls1"):
                out[p + nm] = (D,)
            if m.kind == "attention":
                out.update({p + "mix.q": (m.heads * m.dim, D), p + "mix.k": (m.kv_heads * m.dim, D), p + "mix.v": (m.kv_heads * m.vdim, D),
                            p + "mix.g": (m.heads * m.vdim, D), p + "mix.o": (D, m.heads * m.vdim), p + "mix.q.norm": (m.dim,),
                            p + "mix.k.norm": (m.dim,), p + "mix.r1": (m.heads,), p + "mix.r2": (m.heads,), p + "mix.sink": (m.heads,)})
            else:
                hd, rank = m.heads * m.dim, (rank_of or {}).get(i, 8)
                for nm in ("r", "k", "v", "g", "a", "o"):
                    out[p + "mix." + nm] = (hd, D) if nm != "o" else (D, hd)
                out.update({p + "mix.a.b": (hd,), p + "mix.w1": (rank, D), p + "mix.w2": (hd, rank), p + "mix.w0": (hd,),
                            p + "mix.norm": (hd,)})
            if L.mlp_kind:
                for nm in ("norm2", "norm2b", "ls2"):
                    out[p + nm] = (D,)
                out.update({p + "mlp.up": (L.ff, D), p + "mlp.down": (D, L.ff), p + "mlp.act": (4,)})
        return out

    # ---- accounting used by the benchmark ----
    def weight_elements(self, rank: int = 8) -> int:
        """Matrix elements one token touches (looped layers once: their weights are shared)."""
        shapes = self.tensor_shapes({i: rank for i in range(len(self.layers))})
        return sum(s[0] * s[1] for k, s in shapes.items() if len(s) == 2 and k != "embed")

    def matmul_flops_per_token(self, rank: int = 8) -> int:
        shapes = self.tensor_shapes({i: rank for i in range(len(self.layers))})
        per_layer = [0] * len(self.layers)
        for k, s in shapes.items():
            if len(s) == 2 and k.startswith("l"):
                per_layer[int(k[1:k.index(".")])] += 2 * s[0] * s[1]
        return sum(per_layer[i] for i in self.layer_runs()) + 2 * self.vocab * self.width


# ---------------------------------------------------------------------------------------------------------------------
# Maferax: post-norm layers (one gain per norm) with a depth-weighted average of all earlier layer results; mixers are
# latent attention (low-rank queries and keys/values, a rotated shared key part) and a gated linear recurrence;
# feed-forwards are gated (dense) or a routed mixture of experts with grouped choice and identity outputs.


@dataclass
class LatentAttentionSpec:
    kind = "latent_attention"
    heads: int
    dim: int              # unrotated query/key coordinates per head
    rot_dim: int          # rotated coordinates per head (after the unrotated ones); the rotated key part is shared by the heads
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int         # leading coordinates of the rotated part the rotation acts on (the design: all rot_dim)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LatentAttentionSpec":
        rot = d["rot"]
        spec = cls(int(d["heads"]), int(d["dim"]), int(d["rot_dim"]), int(d["vdim"]), int(d["q_rank"]), int(d["kv_rank"]),
                   float(d["scale"]), float(rot["base"]), int(rot.get("dims", d["rot_dim"])))
        if spec.rot_dims > spec.rot_dim or spec.rot_dims % 2:
            raise ValueError("latent attention: rot.dims must be even and at most rot_dim")
        return spec

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim, "q_rank": self.q_rank,
                "kv_rank": self.kv_rank, "scale": self.scale, "rot": {"base": self.rot_base, "dims": self.rot_dims}}


@dataclass
class GatedLinearSpec:
    kind = "gla"
    heads: int
    dim: int              # key channels per head
    vdim: int
    tau: float            # decay = sigmoid(z)^(1/tau)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GatedLinearSpec":
        return cls(int(d["heads"]), int(d["dim"]), int(d["vdim"]), float(d["tau"]))

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "tau": self.tau}


@dataclass
class RouterSpec:
    experts: int
    identity: int
    top: int
    groups: int
    keep: int
    scale: float

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RouterSpec":
        g = d.get("groups") or {"count": 1, "keep": 1}
        spec = cls(int(d["experts"]), int(d.get("identity", 0)), int(d["top"]), int(g["count"]), int(g["keep"]), float(d.get("scale", 1.0)))
        total = spec.experts + spec.identity
        if total % spec.groups or not 1 <= spec.keep <= spec.groups or spec.top > spec.keep * (total // spec.groups):
            raise ValueError(f"router: {total} outputs do not form {spec.groups} equal groups of which {spec.keep} can hold {spec.top} choices")
        return spec

    def to_dict(self) -> Dict[str, Any]:
        return {"experts": self.experts, "identity": self.identity, "top": self.top, "groups": {"count": self.groups, "keep": self.keep},
                "scale": self.scale}


@dataclass
class MaferaxLayer:
    mixer: Any                               # LatentAttentionSpec | GatedLinearSpec
    mlp_kind: Optional[str] = None           # None | "dense" | "moe"
    ff: int = 0                              # dense: feed-forward size; moe: size of one expert
    router: Optional[RouterSpec] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MaferaxLayer":
        kinds = {"latent_attention": LatentAttentionSpec, "gla": GatedLinearSpec}
        if d["type"] not in kinds:
            raise ValueError(f"unknown mixer type {d['type']!r}; have {sorted(kinds)}")
        mixer = kinds[d["type"]].from_dict(d["mixer"])
        mlp = d.get("mlp")
        if not mlp:
            return cls(mixer)
        if mlp["kind"] == "dense":
            return cls(mixer, "dense", int(mlp["ff"]))
        if mlp["kind"] == "moe":
            return cls(mixer, "moe", int(mlp["expert"]["ff"]), RouterSpec.from_dict(mlp["router"]))
        raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")

    def to_dict(self) -> Dict[str, Any]:
        mlp = None
        if self.mlp_kind == "dense":
            mlp = {"kind": "dense", "ff": self.ff}
        elif self.mlp_kind == "moe":
            mlp = {"kind": "moe", "expert": {"ff": self.ff}, "router": self.router.to_dict()}
        return {"type": self.mixer.kind, "mixer": self.mixer.to_dict(), "mlp": mlp}


@dataclass
class MaferaxConfig:
    architecture: str = "Maferax"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    postln_alpha: float = 1.0
    logit_scale: float = 1.0
    layers: List[MaferaxLayer] = field(default_factory=list)
    extra: Dict[str, Any] = field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MaferaxConfig":
        known = {"architecture", "vocab", "width", "norm", "postln_alpha", "logit_scale", "layers"}
        return cls(architecture=d.get("architecture", "Maferax"), vocab=int(d["vocab"]), width=int(d["width"]),
                   norm_eps=float(d["norm"]["eps"]), postln_alpha=float(d["postln_alpha"]), logit_scale=float(d.get("logit_scale", 1.0)),
                   layers=[MaferaxLayer.from_dict(x) for x in d["layers"]], extra={k: v for k, v in d.items() if k not in known})

    @classmethod
    def from_pretrained(cls, pathname: str) -> "MaferaxConfig":
        path = Path(pathname)
        if path.is_dir():
            path = path / "config.json"
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.extra)
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width, norm={"eps": self.norm_eps},
                 postln_alpha=self.postln_alpha, logit_scale=self.logit_scale, layers=[x.to_dict() for x in self.layers])
        return d

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=1, sort_keys=True)

    def layer_runs(self) -> List[int]:
        return list(range(len(self.layers)))

    def tensor_shapes(self, rank_of: Optional[Dict[int, int]] = None) -> Dict[str, tuple]:
        """Checkpoint tensor names and shapes.  The inner size of the recurrence's decay projection is not in the
        configuration: it is read from the checkpoint (``rank_of[layer]``), 16 where unknown."""
        D, V = self.width, self.vocab
        out: Dict[str, tuple] = {"embed": (V, D), "embed.norm": (), "head": (V, D), "final.norm": ()}
        for i, L in enumerate(self.layers):
            p, m = f"l{i}.", L.mixer
            out[p + "norm1"] = ()
            out[p + "dwa"] = (i + 2,)
            if m.kind == "latent_attention":
                out.update({p + "mix.dq": (m.q_rank, D), p + "mix.dq.norm": (m.q_rank,), p + "mix.uq": (m.heads * (m.dim + m.rot_dim), m.q_rank),
                            p + "mix.dkv": (m.kv_rank + m.rot_dim, D), p + "mix.dkv.norm": (m.kv_rank,),
                            p + "mix.uk": (m.heads * m.dim, m.kv_rank), p + "mix.uv": (m.heads * m.vdim, m.kv_rank),
                            p + "mix.g": (m.heads, D), p + "mix.o": (D, m.heads * m.vdim)})
            else:
                hd, hv, rank = m.heads * m.dim, m.heads * m.vdim, (rank_of or {}).get(i, 16)
                out.update({p + "mix.q": (hd, D), p + "mix.k": (hd, D), p + "mix.v": (hv, D), p + "mix.g": (hv, D), p + "mix.o": (D, hv),
                            p + "mix.norm": (m.vdim,), p + "mix.a1": (rank, D), p + "mix.a2": (hd, rank), p + "mix.a2.b": (hd,)})
            if L.mlp_kind:
                out[p + "norm2"] = ()
            if L.mlp_kind == "dense":
                out.update({p + "mlp.gate": (L.ff, D), p + "mlp.up": (L.ff, D), p + "mlp.down": (D, L.ff)})
            elif L.mlp_kind == "moe":
                total = L.router.experts + L.router.identity
                for e in range(L.router.experts):
                    out.update({f"{p}mlp.e{e}.gate": (L.ff, D), f"{p}mlp.e{e}.up": (L.ff, D), f"{p}mlp.e{e}.down": (D, L.ff)})
                out.update({p + "mlp.router": (total, D), p + "mlp.correction": (total,)})
        return out

    # ---- accounting used by the benchmark ----
    def weight_elements(self, rank: int = 16, active_only: bool = False) -> int:
        """Matrix elements of the model without the embedding table; ``active_only``: those one token touches (``top`` experts)."""
        shapes = self.tensor_shapes({i: rank for i in range(len(self.layers))})
        total = 0
        for k, s in shapes.items():
            if len(s) != 2 or k == "embed":
                continue
            n = s[0] * s[1]
            if active_only and ".mlp.e" in k:
                L = self.layers[int(k[1:k.index(".")])]
                n = n * L.router.top / max(L.router.experts, 1)
            total += n
        return int(total)

    def matmul_flops_per_token(self, rank: int = 16) -> int:
        return 2 * self.weight_elements(rank, active_only=True)


# ---------------------------------------------------------------------------------------------------------------------
# Sunutar: sandwich layers with plain norm weights and one residual multiplier; every mixer is a pair that reads the
# same input -- windowed softmax attention (biases, query/key norm over the whole projection, soft-capped scores, a
# linear distance penalty, a unit term in the softmax denominator) beside a state-space recurrence (short causal
# convolution, one decay per head and step) -- summed with two scales; feed-forwards are clamped gated units, dense or
# routed by sigmoid scores that multiply the experts' inputs.  The logits come from the embedding table.


@dataclass
class WindowAttentionSpec:
    kind = "attention"
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int           # a query at i sees keys 0 <= i - j < window
    scale: float
    softcap: float
    # fixed by the design (parameters of the kernels): head h's distance slope is 2^(-slope_octaves (h + 1) / heads); the
    # softmax denominator holds one extra term exp(sink_logit)
    slope_octaves: float = 8.0
    sink_logit: float = 0.0

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "WindowAttentionSpec":
        spec = cls(int(d["heads"]), int(d["kv_heads"]), int(d["dim"]), int(d["vdim"]), int(d["mask"]["size"]), float(d["scale"]), float(d["softcap"]))
        if spec.heads % spec.kv_heads or spec.window < 1:
            raise ValueError("attention: heads must be a multiple of kv_heads and the window at least 1")
        return spec

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "mask": {"size": self.window},
                "scale": self.scale, "softcap": self.softcap}

    def slopes(self) -> List[float]:
        return [2.0 ** (-self.slope_octaves * (h + 1) / self.heads) for h in range(self.heads)]


@dataclass
class StateSpaceSpec:
    kind = "state_space"
    heads: int
    vdim: int
    state: int            # rows of a head's state
    groups: int           # groups of heads that share the B and C vectors
    conv: int             # taps of the causal convolution
    norm_groups: int      # equal parts of the heads * vdim channels, each divided by its own root mean square

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "StateSpaceSpec":
        spec = cls(int(d["heads"]), int(d["vdim"]), int(d["state"]), int(d["groups"]), int(d["conv"]), int(d["norm_groups"]))
        if spec.heads % spec.groups or (spec.heads * spec.vdim) % spec.norm_groups or spec.conv < 1:
            raise ValueError("state space: heads must be a multiple of groups, heads * vdim of norm_groups, conv at least 1")
        return spec

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups, "conv": self.conv,
                "norm_groups": self.norm_groups}

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def channels(self) -> int:
        """Channels that pass the convolution: x | B | C."""
        return self.inner + 2 * self.groups * self.state

    @property
    def n_in(self) -> int:
        return self.inner + self.channels + self.heads


@dataclass
class SunutarLayer:
    left: WindowAttentionSpec
    right: StateSpaceSpec
    left_scale: float
    right_scale: float
    mlp_kind: Optional[str] = None           # None | "dense" | "moe"
    ff: int = 0                              # dense: feed-forward size; moe: size of one expert
    limit: float = 0.0                       # clamp of the gated unit
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SunutarLayer":
        if d["type"] != "parallel":
            raise ValueError(f"unknown mixer type {d['type']!r}; have ['parallel']")
        m = d["mixer"]
        L = cls(WindowAttentionSpec.from_dict(m["left"]), StateSpaceSpec.from_dict(m["right"]), float(m["left_scale"]), float(m["right_scale"]))
        mlp = d.get("mlp")
        if not mlp:
            return L
        if mlp["kind"] == "dense":
            L.mlp_kind, L.ff, L.limit = "dense", int(mlp["ff"]), float(mlp["limit"])
        elif mlp["kind"] == "moe":
            L.mlp_kind, L.ff, L.limit = "moe", int(mlp["expert"]["ff"]), float(mlp["expert"]["limit"])
            L.experts, L.top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
            if not 1 <= L.top <= L.experts:
                raise ValueError("router: top must lie between 1 and the number of experts")
        else:
            raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
        return L

    def to_dict(self) -> Dict[str, Any]:
        mlp = None
        if self.mlp_kind == "dense":
            mlp = {"kind": "dense", "ff": self.ff, "limit": self.limit}
        elif self.mlp_kind == "moe":
            mlp = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit}, "router": {"experts": self.experts, "top": self.top}}
        return {"type": "parallel", "mixer": {"left": self.left.to_dict(), "right": self.right.to_dict(), "left_scale": self.left_scale,
                                              "right_scale": self.right_scale}, "mlp": mlp}


@dataclass
class SunutarConfig:
    architecture: str = "Sunutar"
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    residual_mult: float = 1.0
    layers: List[SunutarLayer] = field(default_factory=list)
    extra: Dict[str, Any] = field(default_factory=dict, repr=False)
    act_alpha = 1.702             # fixed by the design: the gated unit is g * sigmoid(act_alpha * g) * (u + 1)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SunutarConfig":
        known = {"architecture", "vocab", "width", "norm", "residual_mult", "layers"}
        return cls(architecture=d.get("architecture", "Sunutar"), vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]),
                   residual_mult=float(d["residual_mult"]), layers=[SunutarLayer.from_dict(x) for x in d["layers"]],
                   extra={k: v for k, v in d.items() if k not in known})

    @classmethod
    def from_pretrained(cls, pathname: str) -> "SunutarConfig":
        path = Path(pathname)
        if path.is_dir():
            path = path / "config.json"
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.extra)
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width, norm={"eps": self.norm_eps},
                 residual_mult=self.residual_mult, layers=[x.to_dict() for x in self.layers])
        return d

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=1, sort_keys=True)

    def layer_runs(self) -> List[int]:
        return list(range(len(self.layers)))

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Checkpoint tensor names and shapes (the logits reuse ``embed``)."""
        D, V = self.width, self.vocab
        out: Dict[str, tuple] = {"embed": (V, D), "final.norm": (D,)}
        for i, L in enumerate(self.layers):
            p, a, r = f"l{i}.", L.left, L.right
            for nm in ("norm1", "norm1b"):
                out[p + nm] = (D,)
            q = p + "mix.left."
            nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
            out.update({q + "q": (nq, D), q + "q.b": (nq,), q + "k": (nk, D), q + "k.b": (nk,), q + "v": (nv, D), q + "v.b": (nv,),
                        q + "q.norm": (nq,), q + "k.norm": (nk,), q + "o": (D, a.heads * a.vdim), q + "o.b": (D,)})
            q = p + "mix.right."
            out.update({q + "in": (r.n_in, D), q + "conv": (r.channels, r.conv), q + "conv.b": (r.channels,), q + "dt_bias": (r.heads,),
                        q + "A_log": (r.heads,), q + "D": (r.heads,), q + "norm": (r.inner,), q + "o": (D, r.inner)})
            if L.mlp_kind:
                for nm in ("norm2", "norm2b"):
                    out[p + nm] = (D,)
            if L.mlp_kind == "dense":
                out.update({p + "mlp.gate": (L.ff, D), p + "mlp.up": (L.ff, D), p + "mlp.down": (D, L.ff)})
            elif L.mlp_kind == "moe":
                for e in range(L.experts):
                    out.update({f"{p}mlp.e{e}.gate": (L.ff, D), f"{p}mlp.e{e}.up": (L.ff, D), f"{p}mlp.e{e}.down": (D, L.ff)})
                out[p + "mlp.router"] = (L.experts, D)
        return out

    # ---- accounting used by the benchmark ----
    def weight_elements(self, active_only: bool = False) -> int:
        """Matrix elements of the model (the embedding table counts once, as the logits' matrix); ``active_only``: those one
        token touches (``top`` experts)."""
        total = 0
        for k, s in self.tensor_shapes().items():
            if len(s) != 2 or ".conv" in k:
                continue
            n = s[0] * s[1]
            if active_only and ".mlp.e" in k:
                L = self.layers[int(k[1:k.index(".")])]
                n = n * L.top / max(L.experts, 1)
            total += n
        return int(total)

    def matmul_flops_per_token(self) -> int:
        return 2 * self.weight_elements(active_only=True)


# ---------------------------------------------------------------------------------------------------------------------
# Gunirax: pre-norm layers whose norm is a Dynamic Tanh (no mean, no variance: tanh(alpha x) * weight + shift); a span of
# layers may run several times with shared weights, every pass after the first starting from stream + embedding output.
# Mixers: a pair on the same input -- sigmoid attention (chunked mask, rotary with stretched frequencies, weightless
# query/key norm, values = the key projection, the heads' weight maps mixed by a matrix, one gate per head) beside
# lightning attention (constant decay per head) -- each projected to the width, RMS-normed there and averaged; or HGRN2
# (the forget gate also decides what is written).  Feed-forwards: gated (silu), or routed squared-relu experts with
# grouped choice (a group's rank: its two best choice scores) plus a shared expert.


@dataclass
class RotarySpec:
    base: float
    dims: int             # leading coordinates of a head the rotation acts on, pair (2i, 2i+1) by angle pos * f_i
    # frequency stretching (factor 0: none): wavelengths above original/low are divided by factor, those below
    # original/high kept, the band between blended linearly in original/wavelength
    factor: float = 0.0
    low: float = 1.0
    high: float = 1.0
    original: float = 0.0

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RotarySpec":
        sc = d.get("scaling") or {}
        spec = cls(float(d["base"]), int(d["dims"]), float(sc.get("factor", 0.0)), float(sc.get("low", 1.0)), float(sc.get("high", 1.0)),
                   float(sc.get("original", 0.0)))
        if spec.dims % 2 or spec.dims < 0:
            raise ValueError("rotary: dims must be even")
        return spec

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.factor:
            d["scaling"] = {"factor": self.factor, "low": self.low, "high": self.high, "original": self.original}
        return d

    def frequencies(self) -> List[float]:
        out = []
        for i in range(self.dims // 2):
            f = self.base ** (-2.0 * i / self.dims)
            if self.factor:
                wl = 2.0 * math.pi / f
                if wl > self.original / self.low:
                    f = f / self.factor
                elif wl >= self.original / self.high:
                    s = (self.original / wl - self.low) / (self.high - self.low)
                    f = (1.0 - s) * f / self.factor + s * f
            out.append(f)
        return out


@dataclass
class SigmoidAttentionSpec:
    kind = "sigmoid_attention"
    heads: int
    kv_heads: int
    dim: int
    vdim: int             # = dim: the values are the key projection
    chunk: int            # a query at i sees the keys j <= i with floor(j / chunk) == floor(i / chunk)
    scale: float
    rot: RotarySpec

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SigmoidAttentionSpec":
        spec = cls(int(d["heads"]), int(d["kv_heads"]), int(d["dim"]), int(d["vdim"]), int(d["mask"]["size"]), float(d["scale"]),
                   RotarySpec.from_dict(d["rot"]))
        if spec.heads % spec.kv_heads or spec.chunk < 1 or spec.vdim != spec.dim or spec.rot.dims > spec.dim:
            raise ValueError("sigmoid attention: heads must be a multiple of kv_heads, the chunk at least 1, vdim equal to dim, rot.dims at most dim")
        return spec

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "mask": {"size": self.chunk},
                "scale": self.scale, "rot": self.rot.to_dict()}


@dataclass
class LightningSpec:
    kind = "lightning"
    heads: int
    dim: int
    vdim: int
    decay: List[float]    # one per head

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "LightningSpec":
        decay = d["decay"]
        if isinstance(decay, (int, float)):      # one number: every head's decay
            decay = [decay] * int(d["heads"])
        spec = cls(int(d["heads"]), int(d["dim"]), int(d["vdim"]), [float(v) for v in decay])
        if len(spec.decay) != spec.heads:
            raise ValueError("lightning attention: one decay per head")
        return spec

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass
class Hgrn2Spec:
    kind = "hgrn2"
    heads: int
    dim: int
    vdim: int

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "Hgrn2Spec":
        return cls(int(d["heads"]), int(d["dim"]), int(d["vdim"]))

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}


@dataclass
class GuniraxLayer:
    kind: str                                # "parallel" | "hgrn2"
    left: Optional[SigmoidAttentionSpec] = None
    right: Optional[LightningSpec] = None
    mixer: Optional[Hgrn2Spec] = None
    mlp_kind: Optional[str] = None           # None | "dense" | "moe"
    ff: int = 0                              # dense: feed-forward size; moe: size of one expert
    router: Optional[RouterSpec] = None
    shared_ff: int = 0                       # moe: size of the shared expert (0: none)
    group_score_top = 2                      # fixed by the design: a group's rank is the sum of its two best choice scores

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GuniraxLayer":
        if d["type"] == "parallel":
            L = cls("parallel", SigmoidAttentionSpec.from_dict(d["mixer"]["left"]), LightningSpec.from_dict(d["mixer"]["right"]))
        elif d["type"] == "hgrn2":
            L = cls("hgrn2", mixer=Hgrn2Spec.from_dict(d["mixer"]))
        else:
            raise ValueError(f"unknown mixer type {d['type']!r}; have ['hgrn2', 'parallel']")
        mlp = d.get("mlp")
        if not mlp:
            return L
        if mlp["kind"] == "dense":
            L.mlp_kind, L.ff = "dense", int(mlp["ff"])
        elif mlp["kind"] == "moe":
            L.mlp_kind, L.ff, L.router = "moe", int(mlp["expert"]["ff"]), RouterSpec.from_dict(mlp["router"])
            L.shared_ff = int((mlp.get("shared") or {}).get("ff", 0))
            if L.router.identity:
                raise ValueError("router: this design has no identity outputs")
        else:
            raise ValueError(f"unknown feed-forward kind {mlp['kind']!r}")
        return L

    def to_dict(self) -> Dict[str, Any]:
        mlp = None
        if self.mlp_kind == "dense":
            mlp = {"kind": "dense", "ff": self.ff}
        elif self.mlp_kind == "moe":
            r = self.router
            mlp = {"kind": "moe", "expert": {"ff": self.ff},
                   "router": {"experts": r.experts, "top": r.top, "groups": {"count": r.groups, "keep": r.keep}, "scale": r.scale}}
            if self.shared_ff:
                mlp["shared"] = {"ff": self.shared_ff}
        mixer = {"left": self.left.to_dict(), "right": self.right.to_dict()} if self.kind == "parallel" else self.mixer.to_dict()
        return {"type": self.kind, "mixer": mixer, "mlp": mlp}


@dataclass
class GuniraxConfig:
    architecture: str = "Gunirax"
    vocab: int = 0
    width: int = 0
    embedding_scale: float = 1.0
    norm_eps: float = 1e-6
    layers: List[GuniraxLayer] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    extra: Dict[str, Any] = field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "GuniraxConfig":
        loop = d.get("loop") or {}
        known = {"architecture", "vocab", "width", "embedding", "norm", "layers", "loop"}
        cfg = cls(architecture=d.get("architecture", "Gunirax"), vocab=int(d["vocab"]), width=int(d["width"]),
                  embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), norm_eps=float(d["norm"]["eps"]),
                  layers=[GuniraxLayer.from_dict(x) for x in d["layers"]],
                  loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)), loop_times=int(loop.get("times", 1)),
                  extra={k: v for k, v in d.items() if k not in known})
        cfg.layer_runs()
        return cfg

    @classmethod
    def from_pretrained(cls, pathname: str) -> "GuniraxConfig":
        path = Path(pathname)
        if path.is_dir():
            path = path / "config.json"
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.extra)
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width, embedding={"scale": self.embedding_scale},
                 norm={"eps": self.norm_eps}, layers=[x.to_dict() for x in self.layers],
                 loop={"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times})
        return d

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=1, sort_keys=True)

    def _looped(self) -> bool:
        n, a, b = len(self.layers), self.loop_start, self.loop_stop
        if self.loop_times < 1:
            raise ValueError("loop.times must be at least 1")
        if self.loop_times == 1 or b <= a:
            return False
        if not 0 <= a < b <= n:
            raise ValueError(f"loop {a}..{b} x {self.loop_times} does not fit {n} layers")
        return True

    def layer_runs(self) -> List[int]:
        """Layer index of every layer run, in execution order."""
        n, a, b = len(self.layers), self.loop_start, self.loop_stop
        if not self._looped():
            return list(range(n))
        return list(range(a)) + list(range(a, b)) * self.loop_times + list(range(b, n))

    def run_restarts(self) -> List[int]:
        """1 for the runs that open a pass after the first (the embedding output joins the stream before them), else 0."""
        runs = self.layer_runs()
        out = [0] * len(runs)
        if self._looped():
            a, span = self.loop_start, self.loop_stop - self.loop_start
            for rep in range(1, self.loop_times):
                out[a + rep * span] = 1
        return out

    def tensor_shapes(self) -> Dict[str, tuple]:
        """Checkpoint tensor names and shapes."""
        D, V = self.width, self.vocab
        out: Dict[str, tuple] = {"embed": (V, D), "head": (V, D)}

        def norm(name):
            out.update({name: (D,), name + ".b": (D,), name + ".alpha": ()})

        norm("final.norm")
        for i, L in enumerate(self.layers):
            p = f"l{i}."
            norm(p + "norm1")
            if L.kind == "parallel":
                a, r, q = L.left, L.right, p + "mix.left."
                out.update({q + "q": (a.heads * a.dim, D), q + "q.b": (a.heads * a.dim,), q + "k": (a.kv_heads * a.dim, D),
                            q + "k.b": (a.kv_heads * a.dim,), q + "talk": (a.heads, a.heads), q + "pb": (a.heads,), q + "g": (a.heads, D),
                            q + "o": (D, a.heads * a.vdim), p + "mix.left.out": (D,), p + "mix.right.out": (D,)})
                q = p + "mix.right."
                out.update({q + "q": (r.heads * r.dim, D), q + "k": (r.heads * r.dim, D), q + "v": (r.heads * r.vdim, D),
                            q + "g": (r.heads * r.vdim, D), q + "o": (D, r.heads * r.vdim), q + "norm": (r.heads * r.vdim,)})
            else:
                m, q = L.mixer, p + "mix."
                out.update({q + "q": (m.heads * m.dim, D), q + "f": (m.heads * m.dim, D), q + "f.b": (m.heads * m.dim,),
                            q + "lower": (m.heads * m.dim,), q + "v": (m.heads * m.vdim, D), q + "o": (D, m.heads * m.vdim), q + "norm": (m.vdim,)})
            if L.mlp_kind:
                norm(p + "norm2")
            if L.mlp_kind == "dense":
                out.update({p + "mlp.gate": (L.ff, D), p + "mlp.up": (L.ff, D), p + "mlp.down": (D, L.ff)})
            elif L.mlp_kind == "moe":
                for e in range(L.router.experts):
                    out.update({f"{p}mlp.e{e}.up": (L.ff, D), f"{p}mlp.e{e}.down": (D, L.ff)})
                out.update({p + "mlp.router": (L.router.experts, D), p + "mlp.correction": (L.router.experts,)})
                if L.shared_ff:
                    out.update({p + "mlp.shared.up": (L.shared_ff, D), p + "mlp.shared.down": (D, L.shared_ff)})
        return out

    # ---- accounting used by the benchmark ----
    def weight_elements(self, active_only: bool = False) -> int:
        """Matrix elements of the model without the embedding table (looped layers once: their weights are shared);
        ``active_only``: those one token touches (``top`` experts)."""
        total = 0
        for k, s in self.tensor_shapes().items():
            if len(s) != 2 or k == "embed" or k.endswith(".talk"):
                continue
            n = s[0] * s[1]
            if active_only and ".mlp.e" in k:
                L = self.layers[int(k[1:k.index(".")])]
                n = n * L.router.top / max(L.router.experts, 1)
            total += n
        return int(total)

    def matmul_flops_per_token(self) -> int:
        per_layer = [0.0] * len(self.layers)
        for k, s in self.tensor_shapes().items():
            if len(s) != 2 or not k.startswith("l") or k.endswith(".talk"):
                continue
            i = int(k[1:k.index(".")])
            n = 2.0 * s[0] * s[1]
            if ".mlp.e" in k:
                n = n * self.layers[i].router.top / max(self.layers[i].router.experts, 1)
            per_layer[i] += n
        return int(sum(per_layer[i] for i in self.layer_runs()) + 2 * self.vocab * self.width)
