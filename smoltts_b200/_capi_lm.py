"""ctypes binding of ``include/smoltts_b200_lm.h`` (hybrid language-model engine, ``libsmoltts_b200_lm.so``).

Like ``_capi``: the library is built in-tree on first use when its sources changed, and loading never falls back to
another implementation.  Struct layouts mirror the header field by field.
"""
from __future__ import annotations

import ctypes as C
import os

from . import build as _build
from ._errors import SMOL_OK, SmolError

SMOL_LM_ABI_VERSION = 4
SMOL_LM_BF16, SMOL_LM_F32 = 0, 1


class SmolLmLayer(C.Structure):
    pass


# `side` points to another SmolLmLayer (host memory), so the fields are set after the class exists
SmolLmLayer._fields_ = [(n, C.c_int32) for n in ("mixer", "heads", "kv_heads", "dim", "vdim", "rank", "mlp", "ff")] + [
    (n, C.c_float) for n in ("score_scale", "decay_coef", "unit_eps")] + [
    (n, C.c_void_p) for n in ("w_in", "w_out", "w_up", "w_down", "norm1", "norm1b", "norm2", "norm2b", "ls1", "ls2",
                              "q_norm", "k_norm", "dist_r1", "dist_r2", "sink", "rate_bias", "decay_w2", "decay_bias",
                              "out_norm", "act")] + [
    (n, C.c_int32) for n in ("rot_dim", "rot_dims", "q_rank", "kv_rank", "mlp_act", "n_experts", "n_identity", "top_k", "n_groups", "keep_groups")] + [
    (n, C.c_float) for n in ("rot_base", "decay_tau", "router_scale")] + [
    (n, C.c_void_p) for n in ("w_q_up", "w_k_up_t", "w_v_up", "q_lat_norm", "kv_lat_norm", "w_experts_in", "w_experts_out", "w_router",
                              "route_bias", "depth_mix")] + [
    (n, C.c_int32) for n in ("window", "norm_whole", "no_gate")] + [("softcap", C.c_float)] + [
    (n, C.c_void_p) for n in ("dist_slope", "in_bias", "out_bias")] + [("mix_scale", C.c_float), ("side", C.POINTER(SmolLmLayer))] + [
    (n, C.c_int32) for n in ("n_state", "bc_groups", "conv_taps", "norm_parts")] + [
    (n, C.c_void_p) for n in ("conv_w", "conv_b", "dt_bias", "a_log", "skip")] + [
    (n, C.c_float) for n in ("act_limit", "act_alpha")] + [
    (n, C.c_int32) for n in ("router_score", "router_plain", "route_input")] + [
    (n, C.c_void_p) for n in ("norm1_shift", "norm1_alpha", "norm2_shift", "norm2_alpha")] + [("chunk", C.c_int32)] + [
    (n, C.c_void_p) for n in ("head_bias", "talk")] + [(n, C.c_float) for n in ("rot_stretch", "rot_low", "rot_high", "rot_original")] + [
    (n, C.c_void_p) for n in ("head_decay", "forget_lower", "proj_norm")] + [
    (n, C.c_int32) for n in ("ff_plain", "group_rank_top", "shared_ff")] + [(n, C.c_void_p) for n in ("w_shared_in", "w_shared_out")]


class SmolLmConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("dtype", "vocab", "width", "n_layers", "n_runs", "page_size", "max_step_tokens",
                                         "max_step_seqs", "max_want", "max_context", "use_graph")] + [
        ("embed_scale", C.c_float), ("norm_eps", C.c_float), ("block", C.c_int32), ("residual_alpha", C.c_float), ("logit_scale", C.c_float),
        ("norm_plain", C.c_int32), ("norm_kind", C.c_int32), ("run_flags", C.POINTER(C.c_int32))]


class SmolLmGlobals(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("embed", "head", "final_norm", "embed_norm", "final_norm_shift", "final_norm_alpha")]


class SmolLmStep(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_tokens", "n_seqs", "n_want", "max_pages", "min_seq_tokens", "max_seq_tokens", "max_pos")] + [
        (n, C.c_void_p) for n in ("tokens", "tok_seq", "tok_pos", "seq_start", "seq_pos0", "seq_slot", "block_table", "want_rows",
                                  "logits", "trace")]


PROTOTYPES = {
    "smol_lm_abi_version": (C.c_int, []),
    "smol_lm_struct_bytes": (C.c_size_t, [C.c_int]),
    "smol_lm_last_error": (C.c_char_p, []),
    "smol_lm_create": (C.c_int, [C.POINTER(SmolLmConfig), C.POINTER(SmolLmLayer), C.POINTER(C.c_int32), C.POINTER(C.c_void_p)]),
    "smol_lm_destroy": (None, [C.c_void_p]),
    "smol_lm_page_bytes": (C.c_size_t, [C.c_void_p]),
    "smol_lm_slot_bytes": (C.c_size_t, [C.c_void_p]),
    "smol_lm_workspace_bytes": (C.c_size_t, [C.c_void_p]),
    "smol_lm_bind": (C.c_int, [C.c_void_p, C.POINTER(SmolLmGlobals), C.c_void_p, C.c_size_t, C.c_void_p, C.c_int32, C.c_void_p, C.c_int32]),
    "smol_lm_step": (C.c_int, [C.c_void_p, C.POINTER(SmolLmStep), C.c_void_p]),
    "smol_lm_sample": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_float, C.c_float, C.c_uint64,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "smol_lm_linear": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "smol_lm_launch_count": (C.c_int64, [C.c_void_p]),
    "smol_lm_error_word": (C.c_void_p, [C.c_void_p]),
}

_lib = None


def library_path() -> str:
    return _build.LM_LIB_PATH


def load() -> C.CDLL:
    """Loads (building first if necessary) the language-model library.  Raises if it cannot."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("SMOLTTS_B200_LM_LIB") or _build.build(target="lm")
    lib = C.CDLL(path)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.smol_lm_abi_version() != SMOL_LM_ABI_VERSION:
        raise RuntimeError(f"{path}: ABI version {lib.smol_lm_abi_version()} != {SMOL_LM_ABI_VERSION}")
    for which, mirror in enumerate((SmolLmLayer, SmolLmConfig, SmolLmGlobals, SmolLmStep)):
        if lib.smol_lm_struct_bytes(which) != C.sizeof(mirror):
            raise RuntimeError(f"{path}: {mirror.__name__} is {lib.smol_lm_struct_bytes(which)} bytes in the library, {C.sizeof(mirror)} in the binding")
    _lib = lib
    return lib


def check(rc: int) -> None:
    if rc != SMOL_OK:
        msg = load().smol_lm_last_error()
        raise SmolError(rc, msg.decode() if msg else "")
