"""Shared helpers of the Gunirax tests: small configurations, seeded weights, engine + oracle pairs."""
from __future__ import annotations

import torch

from oracle.gunirax_oracle import Oracle, random_weights


def rot(dims=8, base=50.0, scaling=(4.0, 1.0, 4.0, 40)):
    d = {"base": base, "dims": dims}
    if scaling:
        d["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return d


def left(heads=4, kv_heads=2, dim=16, chunk=12, scale=0.25, r=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": chunk}, "scale": scale, "rot": r or rot()}


def right(heads=3, dim=8, vdim=12, decay=None):
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay or [0.5 + 0.49 * (h + 1) / heads for h in range(heads)]}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def moe(experts=8, top=2, ff=24, groups=(4, 2), scale=1.5, shared=16):
    m = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "top": top, "groups": {"count": groups[0], "keep": groups[1]}, "scale": scale}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def par(l=None, r=None, mlp=None):
    return {"type": "parallel", "mixer": {"left": l or left(), "right": r or right()}, "mlp": mlp}


def hg(heads=2, dim=8, vdim=12, mlp=None):
    return {"type": "hgrn2", "mixer": {"heads": heads, "dim": dim, "vdim": vdim}, "mlp": mlp}


def config(layers, vocab=97, width=64, eps=1e-5, scale=3.0, loop=None):
    cfg = {"architecture": "Gunirax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale}, "layers": layers}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# four layers of every kind; layers 1..2 run three times
MIXED = config([hg(mlp=dense()),
                par(mlp=moe()),
                par(left(heads=3, kv_heads=3, dim=10, chunk=5, scale=0.3, r=rot(6, 20.0, None)), right(heads=1, dim=16, vdim=8), dense(24)),
                hg(heads=3, dim=4, vdim=20, mlp=moe(experts=3, top=3, ff=16, groups=(1, 1), scale=0.8, shared=0)),
                par(left(heads=2, kv_heads=1, dim=24, chunk=40, r=rot(24, 1000.0, (8.0, 1.0, 2.0, 64))), right(heads=2, dim=4, vdim=4))],
               loop=(1, 3, 3))


def tokens(n, vocab, seed=0):
    g = torch.Generator().manual_seed(7000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def only_left(w):
    """The sigmoid attention alone: the other branch's weight after its norm is zero."""
    for k in list(w):
        if k.endswith("mix.right.out"):
            w[k] = torch.zeros_like(w[k])


def only_right(w):
    for k in list(w):
        if k.endswith("mix.left.out"):
            w[k] = torch.zeros_like(w[k])


_CACHE = {}


def engine_and_oracle(cfg, seed=0, dtype=torch.float32, spread=1.0, edit=None, **engine):
    """(engine, oracle, weights) on identical seeded weights.  ``edit(weights)`` may change them first."""
    from smoltts_b200.lm import GuniraxLM
    from smoltts_b200.lm_config import GuniraxConfig

    key = (repr(cfg), seed, dtype, spread, edit, tuple(sorted(engine.items())))
    if key not in _CACHE:
        w = random_weights(cfg, seed, spread)
        if edit is not None:
            edit(w)
        kw = dict(max_tokens=1024, max_seqs=4, page_size=16, max_step_tokens=256)
        kw.update(engine)
        model = GuniraxLM(GuniraxConfig.from_dict(cfg), dtype=dtype, **kw)
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


def close_enough(got: torch.Tensor, want: torch.Tensor, dtype, flips: int = 0, tol=None) -> bool:
    """fp32: every row within the tolerance.  bf16: a router's close call may go the other way, and the recurrences and the
    layers above carry that row's difference on to later rows (at a width of 64 and nine layer runs rounding alone reaches
    half the tolerance) -- the bulk of the rows is held to the tolerance (the median to three quarters of it, three rows in
    four to all of it), not every row."""
    errs = row_errs(got, want)
    tol = tol or TOL[dtype]
    if dtype == torch.float32:
        return int((errs > tol).sum()) <= flips
    return float(errs.median()) < 0.75 * tol and float((errs > tol).double().mean()) <= 0.25
