"""Host side of the hybrid language-model engine: checkpoint loading, pools, and the ragged-batch step.

``HybridLM`` is the engine of every design; a design's class says how its checkpoint maps onto the engine's layers.
``PamasunLM`` serves the Pamasun design: a decoder-only model whose layers mix tokens either by causal attention with a
softmax sink (keys and values in a paged pool) or by a generalized delta rule (a matrix state per head, kept in a
per-sequence slot), with PolyNorm feed-forwards, pre- and post-norms around every sublayer and layer scales.
``MaferaxLM`` serves the Maferax design: post-norm layers with one gain per norm and a depth-weighted average of all
earlier layer results; latent attention (one cached latent and one rotated shared key part per position, in the paged
pool) or a gated linear recurrence (state per head in the slot); gated feed-forwards or a routed mixture of experts.
``SunutarLM`` serves the Sunutar design: sandwich layers whose mixer is a pair on the same input -- windowed attention
(keys and values in the paged pool) beside a state-space recurrence (state and convolution inputs in the slot) -- with
clamped gated feed-forwards, dense or routed by sigmoid scores; the logits reuse the embedding table.
``GuniraxLM`` serves the Gunirax design: pre-norm layers with Dynamic-Tanh norms, a looped span of layers whose later
passes restart from stream + embedding output; mixers are a pair -- chunked sigmoid attention with mixed heads (keys and
values in the paged pool) beside lightning attention (state in the slot), each projected and normed on its own -- or
HGRN2; feed-forwards are gated or routed squared-relu experts with a shared expert.

The engine owns two pools -- key/value pages (``PagePool``) and state slots (``SlotPool``) -- and one step function,
``forward``: any number of sequences, each with its next tokens (a portion of a prompt or a single decoded token).
Schedulers (``serving.TokenBatcher``) and the trace replayer both drive this one function.  torch is used for device
memory and streams only; all arithmetic runs in the CUDA library behind the C ABI (``_capi_lm``).  There is no CPU
fallback: constructing a model without a CUDA device raises.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import struct
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _capi_lm
from ._errors import SMOL_ERR_CAPACITY, SmolError
from .lm_config import (ACT_CLAMPED, ACT_GELU_TANH, ACT_RELU_SQUARED, ACT_SILU, BLOCK_POSTNORM, BLOCK_PRENORM, BLOCK_SANDWICH, MAFERAX_MLP_KINDS,
                        MIXER_KINDS, MLP_KINDS, NORM_DYT, ROUTE_SIGMOID, GuniraxConfig, MaferaxConfig, PamasunConfig, SunutarConfig)
from .pool import PagePool, SlotPool

_ST_DTYPES = {"BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """A safetensors file: 8-byte little-endian header length, a JSON header (name -> dtype, shape, data_offsets), data."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=_ST_DTYPES[meta["dtype"]]) if hi > lo else torch.empty(0, dtype=_ST_DTYPES[meta["dtype"]])
        out[name] = t.reshape(meta["shape"])          # () for a single number
    return out


class Sequence_:
    """What the engine holds for one live sequence: its pages (in order), its state slot, and how many positions are cached."""

    __slots__ = ("uid", "pages", "slot", "length")

    def __init__(self, uid, slot: int):
        self.uid = uid
        self.pages: List[int] = []
        self.slot = slot
        self.length = 0


class HybridLM:
    """B200 engine of one hybrid language-model checkpoint.  Subclasses name the design's configuration class and map
    its checkpoint onto the engine's layer structs (``_describe``)."""

    architecture = ""
    config_class = None

    def __init__(self, config, dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None,
                 max_tokens: int = 8192, max_seqs: int = 4, page_size: int = 64, max_step_tokens: int = 2048,
                 max_want: Optional[int] = None, use_graph: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("smoltts_b200 needs a CUDA device: there is no CPU fallback")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be torch.bfloat16 or torch.float32")
        self.lib = _capi_lm.load()
        self.config = config
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.page_size = page_size
        self.max_seqs = max_seqs
        self.max_step_tokens = max_step_tokens
        self.max_want = max_want or max_step_tokens
        self.use_graph = use_graph
        self.runs = config.layer_runs()
        self.page_pool = PagePool((max_tokens + page_size - 1) // page_size, page_size)
        self.slot_pool = SlotPool(max_seqs)
        self.max_pages = self.page_pool.n            # a lone sequence may own the whole pool
        self.weights: Dict[str, torch.Tensor] = {}
        self._h: Optional[C.c_void_p] = None
        self._keep: List[torch.Tensor] = []
        self._meta_copied: Optional[torch.cuda.Event] = None
        self.steps = 0

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_pretrained(cls, path: str, dtype: torch.dtype = torch.bfloat16, **engine_kwargs):
        config = cls.config_class.from_pretrained(str(path))
        model = cls(config, dtype=dtype, **engine_kwargs)
        model.load_state_dict(read_safetensors(str(Path(path) / "model.safetensors")))
        return model

    # -- what a design's class provides --
    def _shapes(self, sd: Dict[str, torch.Tensor]) -> Dict[str, tuple]:
        """Tensor names and shapes the checkpoint must hold (sizes the configuration leaves open are read from ``sd``)."""
        raise NotImplementedError

    def _describe(self, sd, layers, mat, vec) -> Dict[str, object]:
        """Fills the engine's layer structs from the checkpoint; ``mat(*names)`` uploads matrices (stacked along the output
        axis) in the engine's element type, ``vec(name)`` a vector or single number in fp32; both return device tensors that
        the engine keeps alive.  Returns {"config": extra SmolLmConfig fields, "globals": SmolLmGlobals fields as tensors}."""
        raise NotImplementedError

    def load_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        """Binds a checkpoint: matrices in the engine's element type (per-mixer input projections fused into one matrix),
        vectors in fp32; creates the engine for the sizes found and carves its pools."""
        cfg, dev, dt = self.config, self.device, self.dtype
        want = self._shapes(sd)
        missing = [k for k in want if k not in sd]
        if missing:
            raise KeyError(f"checkpoint is missing {missing[:4]}{'...' if len(missing) > 4 else ''}")
        for k, shape in want.items():
            if tuple(sd[k].shape) != tuple(shape):
                raise ValueError(f"shape mismatch for {k}: {tuple(sd[k].shape)} vs {tuple(shape)}")
        self.weights = {k: sd[k] for k in want}

        def keep(t: torch.Tensor) -> torch.Tensor:
            self._keep.append(t)
            return t

        def mat(*names: str) -> torch.Tensor:
            return keep(torch.cat([(sd[n] if isinstance(n, str) else n).to(torch.float32) for n in names], 0).to(device=dev, dtype=dt).contiguous())

        def vec(name) -> torch.Tensor:
            return keep((sd[name] if isinstance(name, str) else name).to(device=dev, dtype=torch.float32).reshape(-1).contiguous())

        self._keep = []
        layers = (_capi_lm.SmolLmLayer * len(cfg.layers))()
        for c in layers:
            c.mix_scale = 1.0
        desc = self._describe(sd, layers, mat, vec)
        ccfg = _capi_lm.SmolLmConfig(
            dtype=_capi_lm.SMOL_LM_F32 if dt == torch.float32 else _capi_lm.SMOL_LM_BF16, vocab=cfg.vocab, width=cfg.width,
            n_layers=len(cfg.layers), n_runs=len(self.runs), page_size=self.page_size, max_step_tokens=self.max_step_tokens,
            max_step_seqs=self.max_seqs, max_want=self.max_want,
            max_context=self.page_pool.n * self.page_size, use_graph=int(self.use_graph), embed_scale=1.0, norm_eps=cfg.norm_eps,
            block=BLOCK_SANDWICH, residual_alpha=1.0, logit_scale=1.0)
        for k, v in desc["config"].items():
            setattr(ccfg, k, v)
        runs = (C.c_int32 * len(self.runs))(*self.runs)
        flags = desc.get("run_flags")
        if flags is not None:
            run_flags = (C.c_int32 * len(self.runs))(*flags)          # stays alive until create has copied it
            ccfg.run_flags = C.cast(run_flags, C.POINTER(C.c_int32))
        if self._h:
            self.lib.smol_lm_destroy(self._h)
        h = C.c_void_p()
        _capi_lm.check(self.lib.smol_lm_create(C.byref(ccfg), layers, runs, C.byref(h)))
        self._h = h
        g = _capi_lm.SmolLmGlobals(**{k: v.data_ptr() for k, v in desc["globals"].items()})
        with torch.cuda.device(dev):
            self.page_bytes = self.lib.smol_lm_page_bytes(h)
            self.slot_bytes = self.lib.smol_lm_slot_bytes(h)
            ws = self.lib.smol_lm_workspace_bytes(h)
            self._workspace = torch.zeros(ws + 256, dtype=torch.uint8, device=dev)
            self._ws_ptr = (self._workspace.data_ptr() + 255) // 256 * 256
            self._kv_pool = torch.zeros(self.page_pool.n * self.page_bytes, dtype=torch.uint8, device=dev)
            self._state_pool = torch.zeros(self.slot_pool.n * self.slot_bytes, dtype=torch.uint8, device=dev)
            _capi_lm.check(self.lib.smol_lm_bind(h, C.byref(g), C.c_void_p(self._ws_ptr), ws, C.c_void_p(self._kv_pool.data_ptr()),
                                                 self.page_pool.n, C.c_void_p(self._state_pool.data_ptr()), self.slot_pool.n))
            # one pinned staging buffer and its device twin carry every step's index arrays in a single copy
            n = self._meta_ints()
            self._meta_host = torch.zeros(n, dtype=torch.int32, pin_memory=True)
            self._meta_dev = torch.zeros(n, dtype=torch.int32, device=dev)
            self._logits = torch.zeros(self.max_want, cfg.vocab, dtype=torch.float32, device=dev)

    def _meta_ints(self) -> int:
        T, S = self.max_step_tokens, self.max_seqs
        return 3 * T + (S + 1) + 2 * S + S * self.max_pages + self.max_want + 64

    def state_dict(self) -> Dict[str, torch.Tensor]:
        return dict(self.weights)

    def save_pretrained(self, pathname: str) -> None:
        from safetensors.torch import save_file

        os.makedirs(pathname, exist_ok=True)
        self.config.save(os.path.join(pathname, "config.json"))
        save_file({k: v.to(torch.bfloat16).contiguous().cpu() for k, v in self.weights.items()}, os.path.join(pathname, "model.safetensors"))

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                self.lib.smol_lm_destroy(self._h)
                self._h = None
        except Exception:
            pass

    # ------------------------------------------------------------------ sequences
    def open_sequence(self, uid=None) -> Sequence_:
        """Admits a sequence: takes a state slot (its state starts at zero with the first token).  Pages are taken as tokens arrive."""
        return Sequence_(uid, self.slot_pool.allocate(1)[0])

    def close_sequence(self, seq: Sequence_) -> None:
        """Gives the sequence's pages and slot back to the pools."""
        if seq.pages:
            self.page_pool.free(seq.pages)
            seq.pages = []
        if seq.slot >= 0:
            self.slot_pool.free([seq.slot])
            seq.slot = -1

    def _reserve(self, seq: Sequence_, n_new: int) -> None:
        need = self.page_pool.pages_for(seq.length + n_new) - len(seq.pages)
        if need > 0:
            seq.pages.extend(self.page_pool.allocate(need))

    # ------------------------------------------------------------------ the step
    def _stream(self) -> C.c_void_p:
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def forward(self, entries: Sequence[Tuple[Sequence_, Sequence[int], Sequence[int]]], trace: bool = False):
        """One engine step.  ``entries``: (sequence, its next token ids, indices among these whose logits are wanted).
        Appends the tokens to every sequence's cache and state and returns the wanted logits ``[n_want, vocab]`` fp32
        (a view of the engine's buffer, valid until the next step), in the order of the entries; with ``trace`` also the
        residual stream after every layer run ``[runs, tokens, width]``."""
        n_tok = sum(len(t) for _, t, _ in entries)
        n_want = sum(len(w) for _, _, w in entries)
        if n_tok == 0:
            raise ValueError("a step needs at least one token")
        if n_tok > self.max_step_tokens or len(entries) > self.max_seqs or n_want > self.max_want:
            raise SmolError(SMOL_ERR_CAPACITY, f"step of {n_tok} tokens / {len(entries)} sequences / {n_want} wanted rows exceeds "
                                               f"{self.max_step_tokens} / {self.max_seqs} / {self.max_want}")
        if len({id(s) for s, _, _ in entries}) != len(entries):
            raise ValueError("a sequence may appear once per step")
        for seq, toks, _ in entries:
            if len(toks) == 0:
                raise ValueError("an entry needs at least one token")
            self._reserve(seq, len(toks))
        T, S, P = n_tok, len(entries), self.max_pages
        if self._meta_copied is not None:
            self._meta_copied.synchronize()          # the previous step's copy has left the pinned buffer
        host = self._meta_host
        o_tok, o_seq, o_pos = 0, T, 2 * T
        o_start = 3 * T
        o_pos0 = o_start + S + 1
        o_slot = o_pos0 + S
        o_bt = o_slot + S
        o_want = o_bt + S * P
        used = o_want + n_want
        hv = host[:used].numpy()
        row = 0
        wn = 0
        for i, (seq, toks, want) in enumerate(entries):
            n = len(toks)
            hv[o_tok + row:o_tok + row + n] = toks
            hv[o_seq + row:o_seq + row + n] = i
            hv[o_pos + row:o_pos + row + n] = range(seq.length, seq.length + n)
            hv[o_start + i] = row
            hv[o_pos0 + i] = seq.length
            hv[o_slot + i] = seq.slot
            hv[o_bt + i * P:o_bt + i * P + len(seq.pages)] = seq.pages
            hv[o_bt + i * P + len(seq.pages):o_bt + (i + 1) * P] = -1
            for w in want:
                if not 0 <= w < n:
                    raise ValueError(f"wanted index {w} outside the entry's {n} tokens")
                hv[o_want + wn] = row + w
                wn += 1
            row += n
        hv[o_start + S] = row
        self._meta_dev[:used].copy_(host[:used], non_blocking=True)
        self._meta_copied = torch.cuda.Event()
        self._meta_copied.record(torch.cuda.current_stream(self.device))
        base = self._meta_dev.data_ptr()
        tr = torch.empty(len(self.runs), T, self.config.width, dtype=torch.float32, device=self.device) if trace else None
        step = _capi_lm.SmolLmStep(
            n_tokens=T, n_seqs=S, n_want=n_want, max_pages=P, min_seq_tokens=min(len(t) for _, t, _ in entries),
            max_seq_tokens=max(len(t) for _, t, _ in entries), max_pos=max(q.length + len(t) for q, t, _ in entries) - 1, tokens=base + 4 * o_tok, tok_seq=base + 4 * o_seq,
            tok_pos=base + 4 * o_pos, seq_start=base + 4 * o_start, seq_pos0=base + 4 * o_pos0, seq_slot=base + 4 * o_slot,
            block_table=base + 4 * o_bt, want_rows=base + 4 * o_want, logits=self._logits.data_ptr(),
            trace=tr.data_ptr() if trace else None)
        _capi_lm.check(self.lib.smol_lm_step(self._h, C.byref(step), self._stream()))
        for seq, toks, _ in entries:
            seq.length += len(toks)
        self.steps += 1
        out = self._logits[:n_want]
        return (out, tr) if trace else out

    def sample(self, logits: torch.Tensor, temp: float = 0.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, seed: int = 0,
               seq_ids: Optional[torch.Tensor] = None, steps: Optional[torch.Tensor] = None) -> torch.Tensor:
        """logits [rows, n] fp32 device -> ids [rows] int32: the library's sampler (temp 0: arg-max)."""
        rows, n = logits.shape
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
        _capi_lm.check(self.lib.smol_lm_sample(self._h, C.c_void_p(logits.data_ptr()), rows, n, float(temp), int(top_k), float(top_p),
                                               float(min_p), int(seed), C.c_void_p(seq_ids.data_ptr()) if seq_ids is not None else None,
                                               C.c_void_p(steps.data_ptr()) if steps is not None else None, C.c_void_p(out.data_ptr()),
                                               self._stream()))
        return out

    def linear(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """a [M, K] . w [N, K]^T -> fp32 [M, N] through the engine's matrix-product kernels (tests and benchmarks)."""
        M, K = a.shape
        N = w.shape[0]
        y = torch.empty(M, N, dtype=torch.float32, device=a.device)
        _capi_lm.check(self.lib.smol_lm_linear(self._h, C.c_void_p(a.data_ptr()), C.c_void_p(w.data_ptr()), C.c_void_p(y.data_ptr()),
                                               M, N, K, self._stream()))
        return y

    def check_device_errors(self) -> None:
        """Raises if a step addressed a page or slot outside the pools (reads the device-side error word; synchronises)."""
        ptr = self.lib.smol_lm_error_word(self._h)
        off = ptr - self._workspace.data_ptr()
        word = int(self._workspace[off:off + 4].view(torch.int32).item())
        if word:
            raise SmolError(SMOL_ERR_CAPACITY, f"device-side error word {word}: a step addressed outside its pools")

    @property
    def launch_count(self) -> int:
        return int(self.lib.smol_lm_launch_count(self._h))


class PamasunLM(HybridLM):
    """B200 engine of one Pamasun checkpoint."""

    architecture = "Pamasun"
    config_class = PamasunConfig

    def _rank_of(self, sd) -> Dict[int, int]:
        return {i: int(sd[f"l{i}.mix.w1"].shape[0]) for i, L in enumerate(self.config.layers)
                if L.mixer.kind == "general_delta" and f"l{i}.mix.w1" in sd}

    def _shapes(self, sd):
        return self.config.tensor_shapes(self._rank_of(sd))

    def _describe(self, sd, layers, mat, vec):
        cfg, rank_of = self.config, self._rank_of(sd)
        for i, L in enumerate(cfg.layers):
            p, m, c = f"l{i}.", L.mixer, layers[i]
            c.mixer, c.heads, c.kv_heads, c.dim, c.vdim = MIXER_KINDS[m.kind], m.heads, m.kv_heads, m.dim, m.vdim
            c.mlp, c.ff = MLP_KINDS[L.mlp_kind], L.ff
            c.score_scale, c.decay_coef, c.unit_eps = m.scale, m.decay_coef, m.unit_eps
            for nm in ("norm1", "norm1b", "ls1"):
                setattr(c, nm, vec(p + nm).data_ptr())
            if m.kind == "attention":
                c.rank = 0
                c.w_in = mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g").data_ptr()
                c.q_norm, c.k_norm = vec(p + "mix.q.norm").data_ptr(), vec(p + "mix.k.norm").data_ptr()
                c.dist_r1, c.dist_r2, c.sink = vec(p + "mix.r1").data_ptr(), vec(p + "mix.r2").data_ptr(), vec(p + "mix.sink").data_ptr()
            else:
                c.rank = rank_of[i]
                c.w_in = mat(p + "mix.r", p + "mix.k", p + "mix.v", p + "mix.g", p + "mix.a", p + "mix.w1").data_ptr()
                c.rate_bias = vec(p + "mix.a.b").data_ptr()
                c.decay_w2 = vec(sd[p + "mix.w2"].to(torch.float32).t().contiguous()).data_ptr()      # [rank, heads * dim]: coalesced per channel
                c.decay_bias, c.out_norm = vec(p + "mix.w0").data_ptr(), vec(p + "mix.norm").data_ptr()
            c.w_out = mat(p + "mix.o").data_ptr()
            if L.mlp_kind:
                c.w_up, c.w_down = mat(p + "mlp.up").data_ptr(), mat(p + "mlp.down").data_ptr()
                for nm in ("norm2", "norm2b", "ls2"):
                    setattr(c, nm, vec(p + nm).data_ptr())
                c.act = vec(p + "mlp.act").data_ptr()
        return {"config": {"embed_scale": cfg.embedding_scale},
                "globals": {"embed": mat("embed"), "head": mat("head"), "final_norm": vec("final.norm")}}


class MaferaxLM(HybridLM):
    """B200 engine of one Maferax checkpoint."""

    architecture = "Maferax"
    config_class = MaferaxConfig

    def _rank_of(self, sd) -> Dict[int, int]:
        return {i: int(sd[f"l{i}.mix.a1"].shape[0]) for i, L in enumerate(self.config.layers)
                if L.mixer.kind == "gla" and f"l{i}.mix.a1" in sd}

    def _shapes(self, sd):
        return self.config.tensor_shapes(self._rank_of(sd))

    def _describe(self, sd, layers, mat, vec):
        cfg, rank_of = self.config, self._rank_of(sd)
        for i, L in enumerate(cfg.layers):
            p, m, c = f"l{i}.", L.mixer, layers[i]
            c.mixer, c.heads, c.dim, c.vdim = MIXER_KINDS[m.kind], m.heads, m.dim, m.vdim
            c.norm1 = vec(p + "norm1").data_ptr()
            c.depth_mix = vec(p + "dwa").data_ptr()
            if m.kind == "latent_attention":
                c.kv_heads, c.rank = 1, 0
                c.rot_dim, c.rot_dims, c.q_rank, c.kv_rank, c.rot_base, c.score_scale = m.rot_dim, m.rot_dims, m.q_rank, m.kv_rank, m.rot_base, m.scale
                c.w_in = mat(p + "mix.dq", p + "mix.dkv", p + "mix.g").data_ptr()
                c.w_q_up = mat(p + "mix.uq").data_ptr()
                # the key expansion of every head, transposed: [heads][kv_rank][dim] (exact: a change of layout only)
                uk = sd[p + "mix.uk"].to(torch.float32).view(m.heads, m.dim, m.kv_rank).transpose(1, 2).reshape(m.heads * m.kv_rank, m.dim)
                c.w_k_up_t = mat(uk).data_ptr()
                c.w_v_up = mat(p + "mix.uv").data_ptr()
                c.q_lat_norm, c.kv_lat_norm = vec(p + "mix.dq.norm").data_ptr(), vec(p + "mix.dkv.norm").data_ptr()
            else:
                c.kv_heads, c.rank = m.heads, rank_of[i]
                c.score_scale, c.decay_tau = m.dim ** -0.5, m.tau
                c.w_in = mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g", p + "mix.a1").data_ptr()
                c.decay_w2 = vec(sd[p + "mix.a2"].to(torch.float32).t().contiguous()).data_ptr()      # [rank, heads * dim]
                c.decay_bias, c.out_norm = vec(p + "mix.a2.b").data_ptr(), vec(p + "mix.norm").data_ptr()
            c.w_out = mat(p + "mix.o").data_ptr()
            c.mlp, c.ff = MAFERAX_MLP_KINDS[L.mlp_kind], L.ff
            if L.mlp_kind:
                c.norm2 = vec(p + "norm2").data_ptr()
            if L.mlp_kind == "dense":
                c.mlp_act = ACT_GELU_TANH
                c.w_up, c.w_down = mat(p + "mlp.gate", p + "mlp.up").data_ptr(), mat(p + "mlp.down").data_ptr()
            elif L.mlp_kind == "moe":
                r = L.router
                c.mlp_act = ACT_SILU
                c.n_experts, c.n_identity, c.top_k, c.n_groups, c.keep_groups, c.router_scale = r.experts, r.identity, r.top, r.groups, r.keep, r.scale
                if r.experts:
                    c.w_experts_in = mat(*[f"{p}mlp.e{e}.{nm}" for e in range(r.experts) for nm in ("gate", "up")]).data_ptr()
                    c.w_experts_out = mat(*[f"{p}mlp.e{e}.down" for e in range(r.experts)]).data_ptr()
                c.w_router, c.route_bias = vec(p + "mlp.router").data_ptr(), vec(p + "mlp.correction").data_ptr()
        return {"config": {"block": BLOCK_POSTNORM, "residual_alpha": cfg.postln_alpha, "logit_scale": cfg.logit_scale},
                "globals": {"embed": mat("embed"), "head": mat("head"), "final_norm": vec("final.norm"), "embed_norm": vec("embed.norm")}}


class SunutarLM(HybridLM):
    """B200 engine of one Sunutar checkpoint."""

    architecture = "Sunutar"
    config_class = SunutarConfig

    def _shapes(self, sd):
        return self.config.tensor_shapes()

    def _describe(self, sd, layers, mat, vec):
        cfg, D = self.config, self.config.width
        self._sides = []                                   # the side mixers' structs live as long as the engine's create call needs them
        residual = vec(torch.full((D,), cfg.residual_mult, dtype=torch.float32))
        for i, L in enumerate(cfg.layers):
            p, a, r, c = f"l{i}.", L.left, L.right, layers[i]
            q = p + "mix.left."
            # the attention is the layer's own mixer, the recurrence its side mixer: one input product, one output product
            c.mixer, c.heads, c.kv_heads, c.dim, c.vdim = MIXER_KINDS["attention"], a.heads, a.kv_heads, a.dim, a.vdim
            c.score_scale, c.window, c.softcap, c.norm_whole, c.no_gate, c.mix_scale = a.scale, a.window, a.softcap, 1, 1, L.left_scale
            c.q_norm, c.k_norm = vec(q + "q.norm").data_ptr(), vec(q + "k.norm").data_ptr()
            c.dist_slope = vec(torch.tensor(a.slopes(), dtype=torch.float32)).data_ptr()
            c.sink = vec(torch.full((a.heads,), a.sink_logit, dtype=torch.float32)).data_ptr()
            t = p + "mix.right."
            c.w_in = mat(q + "q", q + "k", q + "v", t + "in").data_ptr()
            c.in_bias = vec(torch.cat([sd[q + "q.b"].float(), sd[q + "k.b"].float(), sd[q + "v.b"].float(), torch.zeros(r.n_in)])).data_ptr()
            c.w_out = mat(torch.cat([sd[q + "o"].float(), sd[t + "o"].float()], 1)).data_ptr()
            c.out_bias = vec(sd[q + "o.b"].float() * L.left_scale).data_ptr()
            side = _capi_lm.SmolLmLayer()
            side.mixer, side.heads, side.vdim, side.n_state, side.bc_groups = MIXER_KINDS["state_space"], r.heads, r.vdim, r.state, r.groups
            side.conv_taps, side.norm_parts, side.mix_scale = r.conv, r.norm_groups, L.right_scale
            side.conv_w, side.conv_b = vec(t + "conv").data_ptr(), vec(t + "conv.b").data_ptr()
            side.dt_bias, side.a_log, side.skip = vec(t + "dt_bias").data_ptr(), vec(t + "A_log").data_ptr(), vec(t + "D").data_ptr()
            side.out_norm = vec(t + "norm").data_ptr()
            self._sides.append(side)
            c.side = C.pointer(side)
            c.norm1, c.norm1b = vec(p + "norm1").data_ptr(), vec(p + "norm1b").data_ptr()
            c.ls1 = c.ls2 = residual.data_ptr()
            if L.mlp_kind:
                c.norm2, c.norm2b = vec(p + "norm2").data_ptr(), vec(p + "norm2b").data_ptr()
                c.ff, c.mlp_act, c.act_limit, c.act_alpha = L.ff, ACT_CLAMPED, L.limit, cfg.act_alpha
            c.mlp = MAFERAX_MLP_KINDS[L.mlp_kind]          # none / gated / routed experts
            if L.mlp_kind == "dense":
                c.w_up, c.w_down = mat(p + "mlp.gate", p + "mlp.up").data_ptr(), mat(p + "mlp.down").data_ptr()
            elif L.mlp_kind == "moe":
                c.n_experts, c.n_identity, c.top_k, c.n_groups, c.keep_groups, c.router_scale = L.experts, 0, L.top, 1, 1, 1.0
                c.router_score, c.router_plain, c.route_input = ROUTE_SIGMOID, 1, 1
                c.w_experts_in = mat(*[f"{p}mlp.e{e}.{nm}" for e in range(L.experts) for nm in ("gate", "up")]).data_ptr()
                c.w_experts_out = mat(*[f"{p}mlp.e{e}.down" for e in range(L.experts)]).data_ptr()
                c.w_router = vec(p + "mlp.router").data_ptr()
        embed = mat("embed")
        return {"config": {"norm_plain": 1}, "globals": {"embed": embed, "head": embed, "final_norm": vec("final.norm")}}


class GuniraxLM(HybridLM):
    """B200 engine of one Gunirax checkpoint."""

    architecture = "Gunirax"
    config_class = GuniraxConfig

    def _shapes(self, sd):
        return self.config.tensor_shapes()

    def _describe(self, sd, layers, mat, vec):
        cfg = self.config
        self._sides = []                                   # the side mixers' structs live as long as the engine's create call needs them

        def norm(c, field, name):
            setattr(c, field, vec(name).data_ptr())
            setattr(c, field + "_shift", vec(name + ".b").data_ptr())
            setattr(c, field + "_alpha", vec(name + ".alpha").data_ptr())

        for i, L in enumerate(cfg.layers):
            p, c = f"l{i}.", layers[i]
            norm(c, "norm1", p + "norm1")
            if L.kind == "parallel":
                a, r, q, t = L.left, L.right, p + "mix.left.", p + "mix.right."
                # the sigmoid attention is the layer's own mixer, the lightning attention its side mixer: one input product,
                # then each its own output product, a norm over the width and half the weight
                c.mixer, c.heads, c.kv_heads, c.dim, c.vdim = MIXER_KINDS["sigmoid_attention"], a.heads, a.kv_heads, a.dim, a.vdim
                c.score_scale, c.chunk, c.mix_scale = a.scale, a.chunk, 0.5
                c.rot_dims, c.rot_base = a.rot.dims, a.rot.base
                c.rot_stretch, c.rot_low, c.rot_high, c.rot_original = a.rot.factor, a.rot.low, a.rot.high, a.rot.original
                c.head_bias, c.talk = vec(q + "pb").data_ptr(), vec(q + "talk").data_ptr()
                c.w_in = mat(q + "q", q + "k", q + "g", t + "q", t + "k", t + "v", t + "g").data_ptr()
                n_right = 2 * r.heads * r.dim + 2 * r.heads * r.vdim
                c.in_bias = vec(torch.cat([sd[q + "q.b"].float(), sd[q + "k.b"].float(), torch.zeros(a.heads + n_right)])).data_ptr()
                c.w_out, c.proj_norm = mat(q + "o").data_ptr(), vec(p + "mix.left.out").data_ptr()
                side = _capi_lm.SmolLmLayer()
                side.mixer, side.heads, side.kv_heads, side.dim, side.vdim = MIXER_KINDS["lightning"], r.heads, r.heads, r.dim, r.vdim
                side.mix_scale = 0.5
                side.head_decay = vec(torch.tensor(r.decay, dtype=torch.float32)).data_ptr()
                side.out_norm = vec(t + "norm").data_ptr()
                side.w_out, side.proj_norm = mat(t + "o").data_ptr(), vec(p + "mix.right.out").data_ptr()
                self._sides.append(side)
                c.side = C.pointer(side)
            else:
                m, q = L.mixer, p + "mix."
                c.mixer, c.heads, c.kv_heads, c.dim, c.vdim = MIXER_KINDS["hgrn2"], m.heads, m.heads, m.dim, m.vdim
                c.w_in = mat(q + "q", q + "f", q + "v").data_ptr()
                c.rate_bias, c.forget_lower, c.out_norm = vec(q + "f.b").data_ptr(), vec(q + "lower").data_ptr(), vec(q + "norm").data_ptr()
                c.w_out = mat(q + "o").data_ptr()
            c.mlp = MAFERAX_MLP_KINDS[L.mlp_kind]          # none / gated / routed experts
            if L.mlp_kind:
                norm(c, "norm2", p + "norm2")
                c.ff = L.ff
            if L.mlp_kind == "dense":
                c.mlp_act = ACT_SILU
                c.w_up, c.w_down = mat(p + "mlp.gate", p + "mlp.up").data_ptr(), mat(p + "mlp.down").data_ptr()
            elif L.mlp_kind == "moe":
                r = L.router
                c.mlp_act, c.ff_plain = ACT_RELU_SQUARED, 1
                c.n_experts, c.n_identity, c.top_k, c.n_groups, c.keep_groups, c.router_scale = r.experts, 0, r.top, r.groups, r.keep, r.scale
                c.router_score, c.group_rank_top = ROUTE_SIGMOID, L.group_score_top
                c.w_experts_in = mat(*[f"{p}mlp.e{e}.up" for e in range(r.experts)]).data_ptr()
                c.w_experts_out = mat(*[f"{p}mlp.e{e}.down" for e in range(r.experts)]).data_ptr()
                c.w_router, c.route_bias = vec(p + "mlp.router").data_ptr(), vec(p + "mlp.correction").data_ptr()
                if L.shared_ff:
                    c.shared_ff = L.shared_ff
                    c.w_shared_in, c.w_shared_out = mat(p + "mlp.shared.up").data_ptr(), mat(p + "mlp.shared.down").data_ptr()
        return {"config": {"block": BLOCK_PRENORM, "norm_kind": NORM_DYT, "embed_scale": cfg.embedding_scale},
                "run_flags": cfg.run_restarts(),
                "globals": {"embed": mat("embed"), "head": mat("head"), "final_norm": vec("final.norm"),
                            "final_norm_shift": vec("final.norm.b"), "final_norm_alpha": vec("final.norm.alpha")}}
