"""Prefill and decode throughput of the hybrid language-model engine at layer sizes that resemble a real model's:
the Pamasun design beside the DualAR slow transformer (the package's closest model: attention + gated MLP layers), and the
Maferax and Sunutar designs beside Pamasun at equal width, depth and head count (``--lm-design maferax`` / ``sunutar``),
and the Gunirax design beside Sunutar (``--lm-design gunirax``).

``python bench.py --lm`` prints one JSON line: for every size, tokens/s of a whole-prompt prefill and of single-token
decode steps against a filled cache, each with its distance from the roofline (matrix-product + attention flops over the
measured bf16 peak for prefill; weight + cache + state bytes over the measured copy bandwidth for decode).  Weights are
random, inputs synthetic; every timed region is bracketed by CUDA events after warm-up, and the working set of a
step (the weights) is larger than L2 for the sizes below.
"""
from __future__ import annotations

import json
import os
import time
from typing import Dict, List

import torch

SIZES = {
    # name: width, layers, heads, kv_heads, head size, feed-forward, vocab, pattern (d = generalized delta rule, a = attention)
    "w768": dict(width=768, layers=10, heads=12, kv_heads=4, dim=64, ff=4608, vocab=2368, pattern="daa"),
    "w1536": dict(width=1536, layers=12, heads=12, kv_heads=4, dim=128, ff=6144, vocab=8192, pattern="daa"),
    "w768attn": dict(width=768, layers=10, heads=12, kv_heads=4, dim=64, ff=4608, vocab=2368, pattern="a"),
}


MAFERAX_SIZES = {
    # recurrence: heads x (dim keys, vdim values); latent attention: heads x (dim + rot | vdim) through latents q_rank / kv_rank;
    # feed-forward: dense gated (ff) on recurrent layers, routed experts on attention layers (top of experts, expert size eff)
    "w768": dict(width=768, layers=10, heads=12, dim=64, rot=32, vdim=64, q_rank=384, kv_rank=128, ff=3072, experts=16, identity=2, top=3,
                 groups=3, keep=2, eff=1024, vocab=2368, pattern="gll"),
    "w1536": dict(width=1536, layers=12, heads=12, dim=128, rot=64, vdim=128, q_rank=768, kv_rank=128, ff=4096, experts=32, identity=4, top=4,
                  groups=4, keep=2, eff=1024, vocab=8192, pattern="gll"),
    "w768dense": dict(width=768, layers=10, heads=12, dim=64, rot=32, vdim=64, q_rank=384, kv_rank=128, ff=3072, experts=0, identity=0, top=0,
                      groups=1, keep=1, eff=0, vocab=2368, pattern="gll"),
}


def maferax_config(width, layers, heads, dim, rot, vdim, q_rank, kv_rank, ff, experts, identity, top, groups, keep, eff, vocab, pattern) -> dict:
    ls = []
    for i in range(layers):
        if pattern[i % len(pattern)] == "l":
            mlp = ({"kind": "moe", "expert": {"ff": eff}, "router": {"experts": experts, "identity": identity, "top": top,
                                                                    "groups": {"count": groups, "keep": keep}, "scale": 2.0}}
                   if experts else {"kind": "dense", "ff": ff})
            ls.append({"type": "latent_attention", "mlp": mlp,
                       "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                                 "scale": (dim + rot) ** -0.5, "rot": {"base": 10000.0, "dims": rot}}})
        else:
            ls.append({"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": 16.0}, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Maferax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "postln_alpha": 2.0, "logit_scale": 1.0, "layers": ls}


def maferax_state_dict(cfg, seed: int = 0, rank: int = 16) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for k, s in cfg.tensor_shapes({i: rank for i in range(len(cfg.layers))}).items():
        if len(s) == 2:
            sd[k] = (torch.randn(*s, generator=g) * (s[1] ** -0.5)).bfloat16()
        elif len(s) == 0:
            sd[k] = torch.ones(()).bfloat16()
        elif k.endswith("dwa"):
            sd[k] = torch.cat([torch.full((s[0] - 1,), 0.1), torch.ones(1)]).bfloat16()
        elif k.endswith(("dq.norm", "dkv.norm", "mix.norm")):
            sd[k] = torch.ones(s).bfloat16()
        elif k.endswith("a2.b"):
            sd[k] = torch.full(s, 3.0).bfloat16()
        else:
            sd[k] = (torch.randn(*s, generator=g) * 0.05).bfloat16()
    sd["embed"] = torch.randn(*sd["embed"].shape, generator=g).bfloat16()
    return sd


def bench_maferax(name: str, prompt: int, batch: int, decode_steps: int, warmup: int, steps: int, peaks) -> dict:
    """Like bench_pamasun.  Prefill flops: matrix products of the weights one token touches, attention in the latent space
    (per visible key 2 (kv_rank + rot) + 2 kv_rank flops per head) and the recurrence (6 dim vdim per head); decode bytes:
    the weights one step touches (every expert only if the batch's choices can cover them all), the latent cache and the states."""
    from .lm import MaferaxLM
    from .lm_config import MaferaxConfig

    hbm, tflops, _ = peaks
    spec = MAFERAX_SIZES[name]
    cfg = MaferaxConfig.from_dict(maferax_config(**spec))
    rank = 16
    model = MaferaxLM(cfg, dtype=torch.bfloat16, max_tokens=batch * (prompt + 64 + decode_steps), max_seqs=batch, page_size=64,
                      max_step_tokens=2048, max_want=batch)
    model.load_state_dict(maferax_state_dict(cfg, 0, rank))
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab, (batch, prompt + decode_steps), generator=g).tolist()
    n_attn = sum(L.mixer.kind == "latent_attention" for L in cfg.layers)
    n_rec = len(cfg.layers) - n_attn
    H, d, dv, kr, rot = spec["heads"], spec["dim"], spec["vdim"], spec["kv_rank"], spec["rot"]
    mm_flops = cfg.matmul_flops_per_token(rank) - 2 * cfg.vocab * cfg.width

    def prefill():
        seq = model.open_sequence()
        for lo in range(0, prompt, model.max_step_tokens):
            part = toks[0][lo:min(prompt, lo + model.max_step_tokens)]
            model.forward([(seq, part, [len(part) - 1] if lo + len(part) == prompt else [])])
        model.close_sequence(seq)

    l0 = model.launch_count
    ms_p = _timed(prefill, warmup, steps)
    launches = model.launch_count - l0
    flops_p = prompt * mm_flops + n_attn * H * (4 * kr + 2 * rot) * prompt * (prompt + 1) / 2 + n_rec * 6 * H * d * dv * prompt
    seqs = [model.open_sequence() for _ in range(batch)]
    for b, s in enumerate(seqs):
        for lo in range(0, prompt, model.max_step_tokens):
            model.forward([(s, toks[b][lo:min(prompt, lo + model.max_step_tokens)], [])])

    def decode():
        for i in range(decode_steps):
            model.forward([(s, [toks[b][prompt + i]], [0]) for b, s in enumerate(seqs)])
        for s in seqs:
            s.length = prompt

    l0 = model.launch_count
    ms_d = _timed(decode, 2, steps) / decode_steps
    launches += model.launch_count - l0
    ctx = prompt + decode_steps / 2
    # weights a decode step reads: everything but the experts, plus min(batch * top, experts) experts per routed layer
    all_w, act_w = cfg.weight_elements(rank), cfg.weight_elements(rank, active_only=True)
    touched = act_w
    if spec["experts"]:
        per_expert = (all_w - act_w) / max(spec["experts"] - spec["top"], 1)
        touched = all_w - per_expert * max(spec["experts"] - min(batch * spec["top"], spec["experts"]), 0)
    kv_bytes = n_attn * (kr + rot) * 2 * ctx * batch
    st_bytes = n_rec * 2 * H * d * dv * 4 * batch
    bytes_d = 2 * touched + kv_bytes + st_bytes
    model.check_device_errors()
    for s in seqs:
        model.close_sequence(s)
    return {"model": f"Maferax {name}", "spec": spec, "parameters_m": round(all_w / 1e6, 1), "active_parameters_m": round(act_w / 1e6, 1),
            "prefill": {"prompt": prompt, "tokens_per_s": prompt / ms_p * 1e3, "ms": ms_p, "tflops": flops_p / ms_p / 1e9,
                        "of_peak": flops_p / ms_p / 1e9 / tflops},
            "decode": {"batch": batch, "context": prompt, "tokens_per_s": batch / ms_d * 1e3, "ms_per_step": ms_d,
                       "gbs": bytes_d / ms_d / 1e6, "of_peak": bytes_d / ms_d / 1e6 / hbm},
            "gpu_launches": int(launches)}


SUNUTAR_SIZES = {
    # every layer: windowed attention heads x (dim | vdim) over kv_heads beside a state-space recurrence s_heads x (state, s_vdim)
    # in s_groups groups; feed-forward: dense clamped gated units (ff), on every second layer routed experts (top of experts, size eff)
    "w768": dict(width=768, layers=10, heads=12, kv_heads=4, dim=64, vdim=64, window=1024, s_heads=12, s_vdim=64, state=128, s_groups=1,
                 ff=3072, experts=16, top=2, eff=1024, vocab=2368),
    "w768dense": dict(width=768, layers=10, heads=12, kv_heads=4, dim=64, vdim=64, window=1024, s_heads=12, s_vdim=64, state=128, s_groups=1,
                      ff=3072, experts=0, top=0, eff=0, vocab=2368),
    "w1536": dict(width=1536, layers=12, heads=12, kv_heads=4, dim=128, vdim=128, window=1024, s_heads=24, s_vdim=64, state=128, s_groups=2,
                  ff=4096, experts=32, top=4, eff=1024, vocab=8192),
}


def sunutar_config(width, layers, heads, kv_heads, dim, vdim, window, s_heads, s_vdim, state, s_groups, ff, experts, top, eff, vocab) -> dict:
    ls = []
    for i in range(layers):
        mlp = ({"kind": "moe", "expert": {"ff": eff, "limit": 7.0}, "router": {"experts": experts, "top": top}} if experts and i % 2
               else {"kind": "dense", "ff": ff, "limit": 7.0})
        ls.append({"type": "parallel", "mlp": mlp,
                   "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window}, "scale": dim ** -0.5,
                                      "softcap": 30.0},
                             "right": {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": s_groups, "conv": 4, "norm_groups": s_groups},
                             "left_scale": 0.5, "right_scale": 0.5}})
    return {"architecture": "Sunutar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.5, "layers": ls}


def sunutar_state_dict(cfg, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for k, s in cfg.tensor_shapes().items():
        if k.endswith(".conv"):
            sd[k] = (torch.randn(*s, generator=g) * 0.3).bfloat16()
        elif len(s) == 2:
            sd[k] = (torch.randn(*s, generator=g) * (s[1] ** -0.5)).bfloat16()
        elif k.endswith("A_log"):
            sd[k] = torch.log(torch.rand(s, generator=g) * 0.5 + 0.01).bfloat16()
        elif "norm" in k or k.endswith(".D"):
            sd[k] = torch.ones(s).bfloat16()
        else:
            sd[k] = (torch.randn(*s, generator=g) * 0.05).bfloat16()
    sd["embed"] = torch.randn(*sd["embed"].shape, generator=g).bfloat16()
    return sd


def bench_sunutar(name: str, prompt: int, batch: int, decode_steps: int, warmup: int, steps: int, peaks) -> dict:
    """Like bench_pamasun.  Prefill flops: matrix products of the weights one token touches, attention over the keys inside the
    window (2 dim + 2 vdim flops per visible key and head) and the recurrence (6 state vdim per head and token); decode bytes:
    the weights one step touches (every expert only if the batch's choices can cover them all), the keys and values inside
    the window, and the states (read and written)."""
    from .lm import SunutarLM
    from .lm_config import SunutarConfig

    hbm, tflops, _ = peaks
    spec = SUNUTAR_SIZES[name]
    cfg = SunutarConfig.from_dict(sunutar_config(**spec))
    model = SunutarLM(cfg, dtype=torch.bfloat16, max_tokens=batch * (prompt + 64 + decode_steps), max_seqs=batch, page_size=64,
                      max_step_tokens=2048, max_want=batch)
    model.load_state_dict(sunutar_state_dict(cfg, 0))
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab, (batch, prompt + decode_steps), generator=g).tolist()
    n_layers = len(cfg.layers)
    H, G, d, dv, W = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"], spec["window"]
    sH, sdv, N = spec["s_heads"], spec["s_vdim"], spec["state"]
    mm_flops = cfg.matmul_flops_per_token() - 2 * cfg.vocab * cfg.width

    def prefill():
        seq = model.open_sequence()
        for lo in range(0, prompt, model.max_step_tokens):
            part = toks[0][lo:min(prompt, lo + model.max_step_tokens)]
            model.forward([(seq, part, [len(part) - 1] if lo + len(part) == prompt else [])])
        model.close_sequence(seq)

    l0 = model.launch_count
    ms_p = _timed(prefill, warmup, steps)
    launches = model.launch_count - l0
    visible = sum(min(i + 1, W) for i in range(prompt))
    flops_p = prompt * mm_flops + n_layers * (H * (2 * d + 2 * dv) * visible + 6 * sH * N * sdv * prompt)
    seqs = [model.open_sequence() for _ in range(batch)]
    for b, s in enumerate(seqs):
        for lo in range(0, prompt, model.max_step_tokens):
            model.forward([(s, toks[b][lo:min(prompt, lo + model.max_step_tokens)], [])])

    def decode():
        for i in range(decode_steps):
            model.forward([(s, [toks[b][prompt + i]], [0]) for b, s in enumerate(seqs)])
        for s in seqs:
            s.length = prompt

    l0 = model.launch_count
    ms_d = _timed(decode, 2, steps) / decode_steps
    launches += model.launch_count - l0
    ctx = min(prompt + decode_steps / 2, W)
    all_w, act_w = cfg.weight_elements(), cfg.weight_elements(active_only=True)
    touched = act_w
    if spec["experts"]:
        per_expert = (all_w - act_w) / max(spec["experts"] - spec["top"], 1)
        touched = all_w - per_expert * max(spec["experts"] - min(batch * spec["top"], spec["experts"]), 0)
    kv_bytes = n_layers * G * (d + dv) * 2 * ctx * batch
    st_bytes = n_layers * 2 * sH * N * sdv * 4 * batch
    bytes_d = 2 * touched + kv_bytes + st_bytes
    model.check_device_errors()
    for s in seqs:
        model.close_sequence(s)
    return {"model": f"Sunutar {name}", "spec": spec, "parameters_m": round(all_w / 1e6, 1), "active_parameters_m": round(act_w / 1e6, 1),
            "prefill": {"prompt": prompt, "tokens_per_s": prompt / ms_p * 1e3, "ms": ms_p, "tflops": flops_p / ms_p / 1e9,
                        "of_peak": flops_p / ms_p / 1e9 / tflops},
            "decode": {"batch": batch, "context": prompt, "tokens_per_s": batch / ms_d * 1e3, "ms_per_step": ms_d,
                       "gbs": bytes_d / ms_d / 1e6, "of_peak": bytes_d / ms_d / 1e6 / hbm},
            "gpu_launches": int(launches)}


GUNIRAX_SIZES = {
    # parallel layers: sigmoid attention heads x dim over kv_heads in chunks of `chunk` beside lightning attention r_heads x (r_dim keys,
    # r_vdim values); every fifth layer is HGRN2 with the lightning attention's sizes; feed-forward: dense gated units (ff), on every
    # second layer routed squared-relu experts (top of experts, size eff, 4 groups of which 2 are kept) and a shared expert of size eff
    "w768": dict(width=768, layers=10, heads=12, kv_heads=4, dim=64, chunk=1024, r_heads=12, r_dim=128, r_vdim=64, ff=3072, experts=16, top=2,
                 eff=1024, vocab=2368),
    "w768dense": dict(width=768, layers=10, heads=12, kv_heads=4, dim=64, chunk=1024, r_heads=12, r_dim=128, r_vdim=64, ff=3072, experts=0, top=0,
                      eff=0, vocab=2368),
    "w1536": dict(width=1536, layers=12, heads=12, kv_heads=4, dim=128, chunk=1024, r_heads=24, r_dim=128, r_vdim=64, ff=4096, experts=32, top=4,
                  eff=1024, vocab=8192),
}


def gunirax_config(width, layers, heads, kv_heads, dim, chunk, r_heads, r_dim, r_vdim, ff, experts, top, eff, vocab) -> dict:
    ls = []
    for i in range(layers):
        mlp = ({"kind": "moe", "expert": {"ff": eff}, "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}, "scale": 1.5},
                "shared": {"ff": eff}} if experts and i % 2 else {"kind": "dense", "ff": ff})
        if i % 5 == 4:
            ls.append({"type": "hgrn2", "mixer": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim}, "mlp": mlp})
            continue
        ls.append({"type": "parallel", "mlp": mlp,
                   "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": chunk}, "scale": dim ** -0.5,
                                      "rot": {"base": 10000.0, "dims": dim, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 2048}}},
                             "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim,
                                       "decay": [1.0 - 2.0 ** (-5 - 3 * h / max(r_heads - 1, 1)) for h in range(r_heads)]}}})
    return {"architecture": "Gunirax", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": ls}


def gunirax_state_dict(cfg, seed: int = 0) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for k, s in cfg.tensor_shapes().items():
        if k.endswith(".talk"):
            sd[k] = (torch.eye(s[0]) * 0.7 + torch.randn(*s, generator=g) * 0.1).bfloat16()
        elif len(s) == 2:
            sd[k] = (torch.randn(*s, generator=g) * (s[1] ** -0.5)).bfloat16()
        elif k.endswith(".alpha"):
            sd[k] = torch.tensor(0.5).bfloat16()
        elif k.endswith(".lower"):
            sd[k] = (torch.rand(s, generator=g) * 0.9).bfloat16()
        elif k.endswith((".b", ".pb", "correction")):
            sd[k] = (torch.randn(*s, generator=g) * 0.05).bfloat16()
        else:
            sd[k] = torch.ones(s).bfloat16()
    sd["embed"] = torch.randn(*sd["embed"].shape, generator=g).bfloat16()
    return sd


def bench_gunirax(name: str, prompt: int, batch: int, decode_steps: int, warmup: int, steps: int, peaks) -> dict:
    """Like bench_sunutar.  Prefill flops: matrix products of the weights one token touches, sigmoid attention over the keys of
    the query's chunk (2 dim for the score, 2 heads for mixing the heads' weights, 2 dim for the values, per visible key and
    head) and the recurrences (6 dim vdim per head and token); decode bytes: the weights one step touches (every expert only
    if the batch's choices can cover them all), the keys and values of the current chunk, and the states (read and written)."""
    from .lm import GuniraxLM
    from .lm_config import GuniraxConfig

    hbm, tflops, _ = peaks
    spec = GUNIRAX_SIZES[name]
    cfg = GuniraxConfig.from_dict(gunirax_config(**spec))
    model = GuniraxLM(cfg, dtype=torch.bfloat16, max_tokens=batch * (prompt + 64 + decode_steps), max_seqs=batch, page_size=64,
                      max_step_tokens=2048, max_want=batch)
    model.load_state_dict(gunirax_state_dict(cfg, 0))
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab, (batch, prompt + decode_steps), generator=g).tolist()
    n_par = sum(1 for L in cfg.layers if L.kind == "parallel")
    n_rec = len(cfg.layers)                                    # every layer carries one recurrence of the same size
    H, G, d, C = spec["heads"], spec["kv_heads"], spec["dim"], spec["chunk"]
    rH, rd, rdv = spec["r_heads"], spec["r_dim"], spec["r_vdim"]
    mm_flops = cfg.matmul_flops_per_token() - 2 * cfg.vocab * cfg.width

    def prefill():
        seq = model.open_sequence()
        for lo in range(0, prompt, model.max_step_tokens):
            part = toks[0][lo:min(prompt, lo + model.max_step_tokens)]
            model.forward([(seq, part, [len(part) - 1] if lo + len(part) == prompt else [])])
        model.close_sequence(seq)

    l0 = model.launch_count
    ms_p = _timed(prefill, warmup, steps)
    launches = model.launch_count - l0
    visible = sum(i % C + 1 for i in range(prompt))
    flops_p = prompt * mm_flops + n_par * H * (4 * d + 2 * H) * visible + n_rec * 6 * rH * rd * rdv * prompt
    seqs = [model.open_sequence() for _ in range(batch)]
    for b, s in enumerate(seqs):
        for lo in range(0, prompt, model.max_step_tokens):
            model.forward([(s, toks[b][lo:min(prompt, lo + model.max_step_tokens)], [])])

    def decode():
        for i in range(decode_steps):
            model.forward([(s, [toks[b][prompt + i]], [0]) for b, s in enumerate(seqs)])
        for s in seqs:
            s.length = prompt

    l0 = model.launch_count
    ms_d = _timed(decode, 2, steps) / decode_steps
    launches += model.launch_count - l0
    ctx = sum((prompt + i) % C + 1 for i in range(decode_steps)) / decode_steps
    all_w, act_w = cfg.weight_elements(), cfg.weight_elements(active_only=True)
    touched = act_w
    if spec["experts"]:
        per_expert = (all_w - act_w) / max(spec["experts"] - spec["top"], 1)
        touched = all_w - per_expert * max(spec["experts"] - min(batch * spec["top"], spec["experts"]), 0)
    kv_bytes = n_par * G * 2 * d * 2 * ctx * batch
    st_bytes = n_rec * 2 * rH * rd * rdv * 4 * batch
    bytes_d = 2 * touched + kv_bytes + st_bytes
    model.check_device_errors()
    for s in seqs:
        model.close_sequence(s)
    return {"model": f"Gunirax {name}", "spec": spec, "parameters_m": round(all_w / 1e6, 1), "active_parameters_m": round(act_w / 1e6, 1),
            "prefill": {"prompt": prompt, "tokens_per_s": prompt / ms_p * 1e3, "ms": ms_p, "tflops": flops_p / ms_p / 1e9,
                        "of_peak": flops_p / ms_p / 1e9 / tflops},
            "decode": {"batch": batch, "context": prompt, "tokens_per_s": batch / ms_d * 1e3, "ms_per_step": ms_d,
                       "gbs": bytes_d / ms_d / 1e6, "of_peak": bytes_d / ms_d / 1e6 / hbm},
            "gpu_launches": int(launches)}


def pamasun_config(width, layers, heads, kv_heads, dim, ff, vocab, pattern) -> dict:
    ls = []
    for i in range(layers):
        if pattern[i % len(pattern)] == "a":
            ls.append({"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5},
                       "mlp": {"kind": "dense", "ff": ff}})
        else:
            ls.append({"type": "general_delta", "mixer": {"heads": heads, "dim": dim}, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Pamasun", "vocab": vocab, "width": width, "embedding": {"scale": width ** 0.5}, "norm": {"eps": 1e-5},
            "layers": ls, "loop": {"start": 0, "stop": 0, "times": 1}}


def random_state_dict(cfg, seed: int = 0, rank: int = 64) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    shapes = cfg.tensor_shapes({i: rank for i in range(len(cfg.layers))})
    sd = {}
    for k, s in shapes.items():
        if len(s) == 2:
            sd[k] = (torch.randn(*s, generator=g) * (s[1] ** -0.5)).bfloat16()
        elif k.endswith(("ls1", "ls2")):
            sd[k] = torch.full(s, 0.5).bfloat16()
        elif k.endswith(("q.norm", "k.norm", "mix.norm")):
            sd[k] = torch.ones(s).bfloat16()
        elif k.endswith("act"):
            sd[k] = torch.tensor([0.6, 0.3, 0.1, 0.0]).bfloat16()
        elif k.endswith(("r1", "r2")):
            sd[k] = torch.full(s, 0.5).bfloat16()
        else:
            sd[k] = (torch.randn(*s, generator=g) * 0.05).bfloat16()
    sd["embed"] = (torch.randn(*shapes["embed"], generator=g) * (shapes["embed"][1] ** -0.5)).bfloat16()
    return sd


def _timed(fn, warmup: int, steps: int) -> float:
    """Mean milliseconds of fn() over `steps` calls, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def _peaks(root: str):
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def bench_pamasun(name: str, prompt: int, batch: int, decode_steps: int, warmup: int, steps: int, peaks) -> dict:
    from .lm import PamasunLM
    from .lm_config import PamasunConfig

    hbm, tflops, _ = peaks
    spec = SIZES[name]
    cfg = PamasunConfig.from_dict(pamasun_config(**spec))
    rank = 64
    model = PamasunLM(cfg, dtype=torch.bfloat16, max_tokens=batch * (prompt + 64 + decode_steps), max_seqs=batch, page_size=64,
                      max_step_tokens=2048, max_want=batch)
    model.load_state_dict(random_state_dict(cfg, 0, rank))
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab, (batch, prompt + decode_steps), generator=g).tolist()
    n_attn = sum(cfg.layers[i].mixer.kind == "attention" for i in cfg.layer_runs())
    n_delta = len(cfg.layer_runs()) - n_attn
    H, d = spec["heads"], spec["dim"]
    mm_flops = cfg.matmul_flops_per_token(rank) - 2 * cfg.vocab * cfg.width            # the head runs on wanted rows only
    wbytes = 2 * cfg.weight_elements(rank)

    # ---- prefill: one sequence, the whole prompt, logits of its last token
    def prefill():
        seq = model.open_sequence()
        for lo in range(0, prompt, model.max_step_tokens):
            part = toks[0][lo:min(prompt, lo + model.max_step_tokens)]
            model.forward([(seq, part, [len(part) - 1] if lo + len(part) == prompt else [])])
        model.close_sequence(seq)

    l0 = model.launch_count
    ms_p = _timed(prefill, warmup, steps)
    launches = model.launch_count - l0
    flops_p = prompt * mm_flops + n_attn * 4 * H * d * prompt * (prompt + 1) / 2 + n_delta * 6 * H * d * d * prompt
    # ---- decode: `batch` sequences with `prompt` cached positions, one token each per step
    seqs = [model.open_sequence() for _ in range(batch)]
    for b, s in enumerate(seqs):
        for lo in range(0, prompt, model.max_step_tokens):
            model.forward([(s, toks[b][lo:min(prompt, lo + model.max_step_tokens)], [])])

    def decode():
        for i in range(decode_steps):
            model.forward([(s, [toks[b][prompt + i]], [0]) for b, s in enumerate(seqs)])
        for s in seqs:
            s.length = prompt                                 # the next timed pass decodes against the same context

    l0 = model.launch_count
    ms_d = _timed(decode, 2, steps) / decode_steps
    launches += model.launch_count - l0
    ctx = prompt + decode_steps / 2
    kv_bytes = n_attn * 2 * spec["kv_heads"] * d * 2 * ctx * batch
    st_bytes = n_delta * 2 * H * d * d * 4 * batch
    bytes_d = wbytes + kv_bytes + st_bytes
    model.check_device_errors()
    for s in seqs:
        model.close_sequence(s)
    return {"model": f"Pamasun {name}", "spec": spec, "parameters_m": round(cfg.weight_elements(rank) / 1e6, 1),
            "prefill": {"prompt": prompt, "tokens_per_s": prompt / ms_p * 1e3, "ms": ms_p, "tflops": flops_p / ms_p / 1e9,
                        "of_peak": flops_p / ms_p / 1e9 / tflops},
            "decode": {"batch": batch, "context": prompt, "tokens_per_s": batch / ms_d * 1e3, "ms_per_step": ms_d,
                       "gbs": bytes_d / ms_d / 1e6, "of_peak": bytes_d / ms_d / 1e6 / hbm},
            "gpu_launches": int(launches)}


def bench_dualar(prompt: int, batch: int, decode_steps: int, warmup: int, steps: int, peaks) -> dict:
    """The slow transformer of smoltts_byte_150m (width 768, 10 layers, 12/4 heads of 64, gated MLP 3072): prefill of one
    prompt and single-position slow steps of `batch` sequences."""
    from . import RQTransformer, named_config
    from .synth import make_state_dict

    hbm, tflops, _ = peaks
    cfg = named_config("smoltts_byte_150m")
    model = RQTransformer(cfg, max_batch=max(batch, 1), max_seq_len=prompt + decode_steps + 64)
    model.load_state_dict(make_state_dict(cfg, seed=0))
    R = cfg.n_rows
    g = torch.Generator().manual_seed(2)
    grid = torch.zeros(1, R, prompt + 1, dtype=torch.int32)
    grid[:, 0] = torch.randint(0, 256, (1, prompt + 1), generator=g).to(torch.int32)
    d_grid = grid.to(model.device)
    lens = torch.tensor([prompt + 1], dtype=torch.int32, device=model.device)
    l0 = model.launch_count

    def prefill():
        b = model.new_batch(1, max_positions=prompt + 8)
        model.prefill(b, d_grid, lens)
        b.release()

    ms_p = _timed(prefill, warmup, steps)
    slow = cfg.n_layer * cfg.layer_params()
    flops_p = prompt * 2 * slow + cfg.n_layer * 4 * cfg.n_head * 64 * prompt * (prompt + 1) / 2
    bb = model.new_batch(batch, max_positions=prompt + decode_steps + 8)
    gridb = d_grid.expand(batch, R, prompt + 1).contiguous()
    model.prefill(bb, gridb, lens.expand(batch).contiguous())
    torch.cuda.synchronize()
    len0, host0 = bb.seq_len.clone(), list(bb.host_len)

    def decode():
        for _ in range(decode_steps):
            model.slow_step(bb, advance=True)
        bb.seq_len.copy_(len0)
        bb.host_len[:] = host0

    ms_d = _timed(decode, 2, steps) / decode_steps
    ctx = prompt + decode_steps / 2
    bytes_d = 2 * (slow + cfg.vocab_size * cfg.dim) + cfg.kv_bytes_per_position() * ctx * batch
    return {"model": "DualAR slow transformer smoltts_byte_150m", "parameters_m": round((slow + cfg.vocab_size * cfg.dim) / 1e6, 1),
            "prefill": {"prompt": prompt, "tokens_per_s": prompt / ms_p * 1e3, "ms": ms_p, "tflops": flops_p / ms_p / 1e9,
                        "of_peak": flops_p / ms_p / 1e9 / tflops},
            "decode": {"batch": batch, "context": prompt, "tokens_per_s": batch / ms_d * 1e3, "ms_per_step": ms_d,
                       "gbs": bytes_d / ms_d / 1e6, "of_peak": bytes_d / ms_d / 1e6 / hbm, "call": "slow_step (one launch per phase)"},
            "gpu_launches": int(model.launch_count - l0)}


def run(args, root: str) -> None:
    assert torch.cuda.is_available(), "the language-model benchmark needs a CUDA device"
    peaks = _peaks(root)
    t0 = time.time()
    entries: List[dict] = []
    if getattr(args, "lm_design", "pamasun") == "gunirax":
        # Gunirax beside Sunutar (the engine's closest design: every mixer a pair of an attention and a recurrence on the same input,
        # dense and routed feed-forwards) at equal width, depth, heads and state sizes
        names = [n for n in (args.lm_sizes.split(",") if args.lm_sizes else ["w768", "w768dense", "w1536"])]
        for n in names:
            for batch in (1, 4):
                entries.append(bench_gunirax(n, args.lm_prompt, batch, 16, args.warmup, args.steps, peaks))
        for n in names:
            for batch in (1, 4):
                entries.append(bench_sunutar(n, args.lm_prompt, batch, 16, args.warmup, args.steps, peaks))
    elif getattr(args, "lm_design", "pamasun") == "sunutar":
        # Sunutar beside Pamasun (the engine's closest design: the same block, attention and a recurrence) at equal width, depth and heads
        names = [n for n in (args.lm_sizes.split(",") if args.lm_sizes else ["w768", "w768dense", "w1536"])]
        for n in names:
            for batch in (1, 4):
                entries.append(bench_sunutar(n, args.lm_prompt, batch, 16, args.warmup, args.steps, peaks))
        for n in sorted({"w1536" if n == "w1536" else "w768" for n in names}):
            for batch in (1, 4):
                entries.append(bench_pamasun(n, args.lm_prompt, batch, 16, args.warmup, args.steps, peaks))
    elif getattr(args, "lm_design", "pamasun") == "maferax":
        # Maferax beside Pamasun (the engine's closest design) at equal width, depth, heads and layer pattern
        names = [n for n in (args.lm_sizes.split(",") if args.lm_sizes else ["w768", "w768dense", "w1536"])]
        for n in names:
            for batch in (1, 4):
                entries.append(bench_maferax(n, args.lm_prompt, batch, 16, args.warmup, args.steps, peaks))
        for n in sorted({"w1536" if n == "w1536" else "w768" for n in names}):
            for batch in (1, 4):
                entries.append(bench_pamasun(n, args.lm_prompt, batch, 16, args.warmup, args.steps, peaks))
    else:
        names = [n for n in (args.lm_sizes.split(",") if args.lm_sizes else ["w768", "w768attn", "w1536"])]
        for n in names:
            for batch in (1, 4):
                entries.append(bench_pamasun(n, args.lm_prompt, batch, 16, args.warmup, args.steps, peaks))
        for batch in (1, 4):
            entries.append(bench_dualar(args.lm_prompt, batch, 16, args.warmup, args.steps, peaks))
    print(json.dumps({"metric": "language-model prefill and decode tokens/s", "dtype": "bf16", "data": "synthetic, random weights",
                      "peaks": {"hbm_gbs": peaks[0], "bf16_tflops": peaks[1], "source": peaks[2]}, "steps": args.steps,
                      "warmup": args.warmup, "entries": entries, "gpu_launches": sum(e["gpu_launches"] for e in entries),
                      "seconds": round(time.time() - t0, 1)}), flush=True)
