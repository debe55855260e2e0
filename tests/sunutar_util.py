"""Shared helpers of the Sunutar tests: small configurations, seeded weights, engine + oracle pairs."""
from __future__ import annotations

import torch

from oracle.sunutar_oracle import Oracle, random_weights


def dense(ff=40, limit=1.5):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=5, top=2, ff=24, limit=1.2):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def left(heads=4, kv_heads=2, dim=16, vdim=24, window=12, scale=0.25, softcap=20.0):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": scale, "softcap": softcap}


def right(heads=4, vdim=12, state=16, groups=2, conv=3, norm_groups=4):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def layer(l=None, r=None, left_scale=0.7, right_scale=1.3, mlp=None):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": l or left(), "right": r or right(), "left_scale": left_scale, "right_scale": right_scale}}


def config(layers, vocab=97, width=64, eps=1e-5, mult=0.4):
    return {"architecture": "Sunutar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}


MIXED = config([layer(mlp=dense()),
                layer(left(heads=3, kv_heads=3, dim=8, vdim=8, window=5, scale=0.3, softcap=8.0), right(heads=2, vdim=20, state=8, groups=1, conv=4, norm_groups=1),
                      0.5, 0.9, moe()),
                layer(left(heads=2, kv_heads=1, dim=24, vdim=16, window=40), right(heads=6, vdim=8, state=24, groups=3, conv=2, norm_groups=2), 1.0, 1.0),
                layer(mlp=moe(experts=3, top=3, ff=16, limit=0.8))])


def tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(3000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


_CACHE = {}


def engine_and_oracle(cfg, seed=0, dtype=torch.float32, spread=1.0, edit=None, **engine):
    """(engine, oracle, weights) on identical seeded weights.  ``edit(weights)`` may change them first."""
    from smoltts_b200.lm import SunutarLM
    from smoltts_b200.lm_config import SunutarConfig

    key = (repr(cfg), seed, dtype, spread, edit, tuple(sorted(engine.items())))
    if key not in _CACHE:
        w = random_weights(cfg, seed, spread)
        if edit is not None:
            edit(w)
        kw = dict(max_tokens=1024, max_seqs=4, page_size=16, max_step_tokens=256)
        kw.update(engine)
        model = SunutarLM(SunutarConfig.from_dict(cfg), dtype=dtype, **kw)
        model.load_state_dict(w)
        _CACHE[key] = (model, Oracle(cfg, w), w)
    return _CACHE[key]


def row_errs(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Every row's error of ``got`` against ``want`` relative to the rows' spread (mean taken off both)."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    spread = (want - want.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(-1).sqrt() / spread


def rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """Largest row error."""
    return float(row_errs(got, want).max())


TOL = {torch.float32: 3e-4, torch.bfloat16: 8e-2}
