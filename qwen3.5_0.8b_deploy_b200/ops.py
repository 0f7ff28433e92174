"""ctypes binding of ``libb200attn.so`` and thin operator classes over it.

Class and method names follow the reference's operator layer (``qwen::cuda::CudaFullAttention``,
``CudaKVCache``, ``CudaLinearAttention``, ``CudaLinearAttnState``, ``CudaEngine``; see the
citations in ``include/b200attn.h``); torch is used only to own device memory and streams.
Every call goes through the C ABI.  A missing library, a missing symbol or a non-zero status
raises: there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libb200attn.so")

OK, ERR_INVALID, ERR_CUDA, ERR_NOMEM, ERR_NOT_READY, ERR_UNSUPPORTED, ERR_DEVICE = 0, -1, -2, -3, -4, -5, -6
PROJ_FP32, PROJ_FP16 = 0, 1
KV_INT8, KV_FP16 = 0, 1

# Every symbol include/b200attn.h declares (tests check the library exports exactly these).
ABI_SYMBOLS = [
    "b200attn_last_error", "b200attn_abi_version", "b200attn_launch_count",
    "b200attn_kv_pool_create", "b200attn_kv_pool_destroy", "b200attn_kv_seq_alloc", "b200attn_kv_seq_reserve",
    "b200attn_kv_seq_free", "b200attn_kv_seq_shrink", "b200attn_kv_clear", "b200attn_kv_seq_len", "b200attn_kv_pages", "b200attn_kv_append",
    "b200attn_kv_export", "b200attn_kv_device_status",
    "b200attn_fa_create", "b200attn_fa_destroy", "b200attn_fa_set_weights", "b200attn_fa_prefill", "b200attn_fa_decode",
    "b200attn_fa_decode_core", "b200attn_fa_decode_core_static", "b200attn_fa_prefill_core",
    "b200attn_la_create", "b200attn_la_destroy", "b200attn_la_set_weights", "b200attn_la_device_status", "b200attn_la_state_create",
    "b200attn_la_state_destroy", "b200attn_la_state_clear", "b200attn_la_state_import", "b200attn_la_state_export",
    "b200attn_la_prefill", "b200attn_la_decode", "b200attn_la_decode_core", "b200attn_la_prefill_core",
    "b200attn_profile_enable", "b200attn_profile_reset", "b200attn_profile_read",
    "b200attn_stack_create", "b200attn_stack_destroy", "b200attn_stack_set_layer_weights",
    "b200attn_stack_set_embedding", "b200attn_stack_init_embedding_random", "b200attn_stack_reset",
    "b200attn_stack_device_status",
    "b200attn_stack_prefill", "b200attn_stack_decode", "b200attn_decode_graph_capture",
    "b200attn_decode_graph_launch", "b200attn_stack_set_tokens", "b200attn_stack_get_tokens",
    "b200attn_stack_begin_batching", "b200attn_stack_admit", "b200attn_stack_retire", "b200attn_stack_rows", "b200attn_stack_step",
]


class B200AttnError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"b200attn status {status}: {message}")
        self.status = status


class InvalidArgument(B200AttnError, ValueError):
    """Maps B200ATTN_ERR_INVALID, the counterpart of the reference's std::invalid_argument."""


def load_library() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python __graft_entry__.py build` "
                          "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    for name in ABI_SYMBOLS:
        if not hasattr(lib, name):
            raise ImportError(f"{LIB_PATH} does not export {name}")
    lib.b200attn_last_error.restype = C.c_char_p
    lib.b200attn_launch_count.restype = C.c_longlong
    return lib


_lib = load_library()
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int)


def lib() -> C.CDLL:
    return _lib


def _check(status: int) -> None:
    if status != 0:
        msg = _lib.b200attn_last_error().decode(errors="replace")
        raise (InvalidArgument if status == ERR_INVALID else B200AttnError)(status, msg)


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _dev(t: torch.Tensor | None) -> C.c_void_p:
    if t is None:
        return C.c_void_p(0)
    assert t.is_cuda and t.is_contiguous(), "device pointer arguments must be contiguous CUDA tensors"
    return C.c_void_p(t.data_ptr())


def _host_f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _host_i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def launch_count(reset: bool = False) -> int:
    return int(_lib.b200attn_launch_count(C.c_int(1 if reset else 0)))


# ---- POD structs -----------------------------------------------------------------------------------
class KvConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("num_layers", "num_kv_heads", "head_dim", "page_tokens", "num_pages",
                                       "max_seqs", "max_pages_per_seq", "kv_dtype")]


class FaConfig(C.Structure):
    _fields_ = [("hidden_size", C.c_int), ("num_heads", C.c_int), ("num_kv_heads", C.c_int), ("head_dim", C.c_int),
                ("rotary_dim", C.c_int), ("rope_theta", C.c_float), ("proj_precision", C.c_int), ("max_batch", C.c_int),
                ("max_prefill_rows", C.c_int)]


class FaWeights(C.Structure):
    _fields_ = [(n, _f32p) for n in ("q_proj", "k_proj", "v_proj", "q_norm", "k_norm", "o_proj")]


class LaConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("hidden_size", "num_heads", "key_dim", "value_dim", "conv_kernel",
                                       "proj_precision", "max_batch", "max_prefill_rows")]


class LaWeights(C.Structure):
    _fields_ = [(n, _f32p) for n in ("in_proj_qkv", "in_proj_a", "in_proj_b", "in_proj_z", "conv1d", "a_log",
                                     "dt_bias", "norm", "out_proj")]


class LaStateConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("num_layers", "max_seqs", "num_heads", "key_dim", "value_dim", "conv_kernel")]


class StackConfig(C.Structure):
    _fields_ = [("num_layers", C.c_int), ("hidden_size", C.c_int), ("intermediate_size", C.c_int),
                ("vocab_size", C.c_int), ("max_seqs", C.c_int), ("max_seq_len", C.c_int),
                ("prefill_chunk_seqs", C.c_int), ("kv_dtype", C.c_int), ("int8_weights", C.c_int),
                ("rms_eps", C.c_float)]


class LayerWeights(C.Structure):
    _fields_ = [("input_norm", _f32p), ("post_norm", _f32p), ("ffn_gate", _f32p), ("ffn_up", _f32p),
                ("ffn_down", _f32p), ("fa", C.POINTER(FaWeights)), ("la", C.POINTER(LaWeights))]


def _fa_weights_struct(w: dict):
    keep = {k: _host_f32(w[k]) for k in ("wq", "wk", "wv", "q_norm", "k_norm", "wo")}
    s = FaWeights(*[keep[k].ctypes.data_as(_f32p) for k in ("wq", "wk", "wv", "q_norm", "k_norm", "wo")])
    return s, keep


def _la_weights_struct(w: dict):
    order = ("w_qkv", "w_a", "w_b", "w_z", "conv_w", "a_log", "dt_bias", "norm_w", "w_out")
    keep = {k: _host_f32(w[k]) for k in order}
    s = LaWeights(*[keep[k].ctypes.data_as(_f32p) for k in order])
    return s, keep


# ---- paged KV cache ------------------------------------------------------------------------------------
class KVCache:
    """Paged INT8 / FP16 KV cache for all full-attention layers (CudaKVCache + PagedKVCache)."""

    def __init__(self, num_layers: int, max_seqs: int, max_tokens_per_seq: int, kv_dtype: int = KV_INT8,
                 num_pages: int | None = None, num_kv_heads: int = 2, head_dim: int = 256, page_tokens: int = 64):
        pages_per_seq = (max_tokens_per_seq + page_tokens - 1) // page_tokens
        cfg = KvConfig(num_layers, num_kv_heads, head_dim, page_tokens,
                       num_pages if num_pages is not None else pages_per_seq * max_seqs, max_seqs, pages_per_seq, kv_dtype)
        self.cfg = cfg
        self.h = C.c_void_p()
        _check(_lib.b200attn_kv_pool_create(C.byref(cfg), C.byref(self.h)))

    def allocate_sequence(self, reserve_tokens: int = 0) -> int:
        slot = C.c_int(-1)
        _check(_lib.b200attn_kv_seq_alloc(self.h, C.c_int(reserve_tokens), C.byref(slot)))
        return slot.value

    def reserve(self, slot: int, total_tokens: int) -> None:
        _check(_lib.b200attn_kv_seq_reserve(self.h, C.c_int(slot), C.c_int(total_tokens)))

    def release_sequence(self, slot: int) -> None:
        _check(_lib.b200attn_kv_seq_free(self.h, C.c_int(slot)))

    def shrink_sequence(self, slot: int, new_len: int) -> None:
        """PagedKVCache::shrink_sequence: truncate to new_len tokens in every layer, pages behind the end go back to the pool."""
        _check(_lib.b200attn_kv_seq_shrink(self.h, C.c_int(slot), C.c_int(new_len)))

    def clear(self) -> None:
        _check(_lib.b200attn_kv_clear(self.h, _stream()))

    def length(self, layer: int, slot: int) -> int:
        n = C.c_int(0)
        _check(_lib.b200attn_kv_seq_len(self.h, C.c_int(layer), C.c_int(slot), C.byref(n)))
        return n.value

    def pages(self) -> tuple[int, int]:
        total, used = C.c_int(0), C.c_int(0)
        _check(_lib.b200attn_kv_pages(self.h, C.byref(total), C.byref(used)))
        return total.value, used.value

    def device_status(self) -> int:
        code = C.c_int(0)
        _check(_lib.b200attn_kv_device_status(self.h, C.byref(code)))
        return code.value

    def append(self, layer: int, slots, counts, k: torch.Tensor, v: torch.Tensor) -> None:
        """Quantise-on-append of fp32 rows [sum(counts), kv_heads*head_dim]."""
        s, c = _host_i32(slots), _host_i32(counts)
        _check(_lib.b200attn_kv_append(self.h, C.c_int(layer), s.ctypes.data_as(_i32p), c.ctypes.data_as(_i32p),
                                       C.c_int(len(s)), _dev(k), _dev(v), _stream()))

    def export(self, layer: int, slot: int):
        """Token-major copy of one sequence: (k, v, k_scale, v_scale); scales are None for FP16."""
        n = self.length(layer, slot)
        kvh, hd = self.cfg.num_kv_heads, self.cfg.head_dim
        fp16 = self.cfg.kv_dtype == KV_FP16
        dt = torch.float16 if fp16 else torch.int8
        k = torch.empty((max(n, 1), kvh, hd), dtype=dt, device="cuda")
        v = torch.empty_like(k)
        ks = None if fp16 else torch.empty((max(n, 1), kvh), dtype=torch.float32, device="cuda")
        vs = None if fp16 else torch.empty_like(ks)
        _check(_lib.b200attn_kv_export(self.h, C.c_int(layer), C.c_int(slot), _dev(k), _dev(v), _dev(ks), _dev(vs),
                                       C.c_int(max(n, 1)), _stream()))
        torch.cuda.synchronize()
        return k[:n], v[:n], (None if fp16 else ks[:n]), (None if fp16 else vs[:n])

    def __del__(self):
        try:
            if getattr(self, "h", None) and self.h.value:
                _lib.b200attn_kv_pool_destroy(self.h)
        except Exception:
            pass


# ---- gated full attention ---------------------------------------------------------------------------------
class FullAttention:
    """CudaFullAttention: set_weights, forward_batch_prefill (causal, per sequence), forward (decode)."""

    def __init__(self, proj_precision: int = PROJ_FP32, max_batch: int = 128, max_prefill_rows: int = 4096,
                 hidden_size=1024, num_heads=8, num_kv_heads=2, head_dim=256, rotary_dim=64, rope_theta=1e7):
        self.cfg = FaConfig(hidden_size, num_heads, num_kv_heads, head_dim, rotary_dim, rope_theta, proj_precision,
                            max_batch, max_prefill_rows)
        self.h = C.c_void_p()
        _check(_lib.b200attn_fa_create(C.byref(self.cfg), C.byref(self.h)))

    def set_weights(self, w: dict) -> None:
        s, _keep = _fa_weights_struct(w)
        _check(_lib.b200attn_fa_set_weights(self.h, C.byref(s)))

    def forward_batch_prefill(self, x: torch.Tensor, kv: KVCache, layer: int, slots, counts) -> torch.Tensor:
        s, c = _host_i32(slots), _host_i32(counts)
        y = torch.empty_like(x)
        _check(_lib.b200attn_fa_prefill(self.h, kv.h, C.c_int(layer), s.ctypes.data_as(_i32p), c.ctypes.data_as(_i32p),
                                        C.c_int(len(s)), _dev(x), _dev(y), _stream()))
        return y

    def forward(self, x: torch.Tensor, kv: KVCache, layer: int, d_slots: torch.Tensor) -> torch.Tensor:
        y = torch.empty_like(x)
        _check(_lib.b200attn_fa_decode(self.h, kv.h, C.c_int(layer), _dev(d_slots), C.c_int(d_slots.numel()), _dev(x),
                                       _dev(y), _stream()))
        return y

    def decode_core(self, q: torch.Tensor, kv: KVCache, layer: int, d_slots: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(q)
        _check(_lib.b200attn_fa_decode_core(self.h, kv.h, C.c_int(layer), _dev(d_slots), C.c_int(d_slots.numel()),
                                            _dev(q), _dev(out), _stream()))
        return out

    def prefill_core(self, q, k, v, counts, use_tensor_cores: bool = True) -> torch.Tensor:
        c = _host_i32(counts)
        out = torch.empty_like(q)
        _check(_lib.b200attn_fa_prefill_core(self.h, c.ctypes.data_as(_i32p), C.c_int(len(c)), _dev(q), _dev(k), _dev(v),
                                             _dev(out), C.c_int(1 if use_tensor_cores else 0), _stream()))
        return out

    def __del__(self):
        try:
            if getattr(self, "h", None) and self.h.value:
                _lib.b200attn_fa_destroy(self.h)
        except Exception:
            pass


# ---- Gated DeltaNet -----------------------------------------------------------------------------------------
class LinearAttnState:
    """CudaLinearAttnState for `num_layers` layers and `max_seqs` sequences."""

    def __init__(self, num_layers: int, max_seqs: int, num_heads=16, key_dim=128, value_dim=128, conv_kernel=4):
        self.cfg = LaStateConfig(num_layers, max_seqs, num_heads, key_dim, value_dim, conv_kernel)
        self.h = C.c_void_p()
        _check(_lib.b200attn_la_state_create(C.byref(self.cfg), C.byref(self.h)))

    def clear(self, slot: int = -1) -> None:
        _check(_lib.b200attn_la_state_clear(self.h, C.c_int(slot), _stream()))

    def import_state(self, layer: int, slot: int, recurrent: torch.Tensor | None, conv: torch.Tensor | None) -> None:
        _check(_lib.b200attn_la_state_import(self.h, C.c_int(layer), C.c_int(slot), _dev(recurrent), _dev(conv), _stream()))

    def export_state(self, layer: int, slot: int):
        c = self.cfg
        rec = torch.empty((c.num_heads, c.key_dim, c.value_dim), dtype=torch.float32, device="cuda")
        conv = torch.empty((c.num_heads * (2 * c.key_dim + c.value_dim), c.conv_kernel - 1), dtype=torch.float32, device="cuda")
        _check(_lib.b200attn_la_state_export(self.h, C.c_int(layer), C.c_int(slot), _dev(rec), _dev(conv), _stream()))
        torch.cuda.synchronize()
        return rec, conv

    def __del__(self):
        try:
            if getattr(self, "h", None) and self.h.value:
                _lib.b200attn_la_state_destroy(self.h)
        except Exception:
            pass


class LinearAttention:
    """CudaLinearAttention: set_weights, forward_batch (causal sequence pass), forward (decode)."""

    def __init__(self, proj_precision: int = PROJ_FP32, max_batch: int = 128, max_prefill_rows: int = 4096,
                 hidden_size=1024, num_heads=16, key_dim=128, value_dim=128, conv_kernel=4):
        self.cfg = LaConfig(hidden_size, num_heads, key_dim, value_dim, conv_kernel, proj_precision, max_batch,
                            max_prefill_rows)
        self.h = C.c_void_p()
        _check(_lib.b200attn_la_create(C.byref(self.cfg), C.byref(self.h)))

    def set_weights(self, w: dict) -> None:
        s, _keep = _la_weights_struct(w)
        _check(_lib.b200attn_la_set_weights(self.h, C.byref(s)))

    def forward_batch(self, x: torch.Tensor, state: LinearAttnState, layer: int, slots, counts) -> torch.Tensor:
        s, c = _host_i32(slots), _host_i32(counts)
        y = torch.empty_like(x)
        _check(_lib.b200attn_la_prefill(self.h, state.h, C.c_int(layer), s.ctypes.data_as(_i32p), c.ctypes.data_as(_i32p),
                                        C.c_int(len(s)), _dev(x), _dev(y), _stream()))
        return y

    def forward(self, x: torch.Tensor, state: LinearAttnState, layer: int, d_slots: torch.Tensor) -> torch.Tensor:
        y = torch.empty_like(x)
        _check(_lib.b200attn_la_decode(self.h, state.h, C.c_int(layer), _dev(d_slots), C.c_int(d_slots.numel()), _dev(x),
                                       _dev(y), _stream()))
        return y

    def device_status(self) -> int:
        code = C.c_int(0)
        _check(_lib.b200attn_la_device_status(self.h, C.byref(code)))
        return code.value

    def decode_core(self, mixed: torch.Tensor, state: LinearAttnState, layer: int, d_slots: torch.Tensor) -> torch.Tensor:
        out = torch.empty((mixed.shape[0], 2048), dtype=torch.float32, device="cuda")
        _check(_lib.b200attn_la_decode_core(self.h, state.h, C.c_int(layer), _dev(d_slots), C.c_int(d_slots.numel()),
                                            _dev(mixed), _dev(out), _stream()))
        return out

    def prefill_core(self, q, k, v, g, beta, state: LinearAttnState, layer: int, slots, counts,
                     use_tensor_cores: bool = True) -> torch.Tensor:
        s, c = _host_i32(slots), _host_i32(counts)
        out = torch.empty_like(v)
        _check(_lib.b200attn_la_prefill_core(self.h, state.h, C.c_int(layer), s.ctypes.data_as(_i32p),
                                             c.ctypes.data_as(_i32p), C.c_int(len(s)), _dev(q), _dev(k), _dev(v), _dev(g),
                                             _dev(beta), _dev(out), C.c_int(1 if use_tensor_cores else 0), _stream()))
        return out

    def __del__(self):
        try:
            if getattr(self, "h", None) and self.h.value:
                _lib.b200attn_la_destroy(self.h)
        except Exception:
            pass


# ---- hybrid stack + graph-captured decode -------------------------------------------------------------------------
class HybridStack:
    """CudaEngine for the attention-facing part: set_layer_weights, forward_batch_prefill,
    forward_batch_decode, reset_cache, and the captured decode step."""

    def __init__(self, num_layers=24, intermediate_size=3584, vocab_size=248320, max_seqs=128, max_seq_len=1536,
                 prefill_chunk_seqs=8, kv_dtype=KV_FP16, int8_weights=True, rms_eps=1e-6):
        self.cfg = StackConfig(num_layers, 1024, intermediate_size, vocab_size, max_seqs, max_seq_len, prefill_chunk_seqs,
                               kv_dtype, 1 if int8_weights else 0, rms_eps)
        self.h = C.c_void_p()
        _check(_lib.b200attn_stack_create(C.byref(self.cfg), C.byref(self.h)))

    def set_layer_weights(self, layer: int, norms: dict, ffn: dict, fa: dict | None = None, la: dict | None = None) -> None:
        keep = [_host_f32(norms["input_norm"]), _host_f32(norms["post_norm"]), _host_f32(ffn["gate"]),
                _host_f32(ffn["up"]), _host_f32(ffn["down"])]
        fa_s = la_s = None
        if fa is not None:
            fa_s, k2 = _fa_weights_struct(fa)
            keep.append(k2)
        if la is not None:
            la_s, k3 = _la_weights_struct(la)
            keep.append(k3)
        lw = LayerWeights(*[a.ctypes.data_as(_f32p) for a in keep[:5]],
                          C.pointer(fa_s) if fa_s is not None else None, C.pointer(la_s) if la_s is not None else None)
        _check(_lib.b200attn_stack_set_layer_weights(self.h, C.c_int(layer), C.byref(lw)))

    def set_embedding(self, embed: np.ndarray, final_norm: np.ndarray) -> None:
        e, f = _host_f32(embed), _host_f32(final_norm)
        _check(_lib.b200attn_stack_set_embedding(self.h, e.ctypes.data_as(_f32p), f.ctypes.data_as(_f32p)))

    def init_embedding_random(self, seed: int, std: float, final_norm: np.ndarray) -> None:
        f = _host_f32(final_norm)
        _check(_lib.b200attn_stack_init_embedding_random(self.h, C.c_uint64(seed), C.c_float(std), f.ctypes.data_as(_f32p)))

    def device_status(self) -> int:
        code = C.c_int(0)
        _check(_lib.b200attn_stack_device_status(self.h, C.byref(code)))
        return code.value

    def reset_cache(self) -> None:
        _check(_lib.b200attn_stack_reset(self.h, _stream()))

    def forward_batch_prefill(self, tokens: torch.Tensor, want_hidden: bool = False):
        n, length = tokens.shape
        nxt = torch.empty(n, dtype=torch.int32, device="cuda")
        hid = torch.empty((n, 1024), dtype=torch.float32, device="cuda") if want_hidden else None
        _check(_lib.b200attn_stack_prefill(self.h, C.c_int(n), C.c_int(length), _dev(tokens), _dev(nxt), _dev(hid), _stream()))
        return (nxt, hid) if want_hidden else nxt

    def forward_batch_decode(self, tokens: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(tokens)
        _check(_lib.b200attn_stack_decode(self.h, C.c_int(tokens.numel()), _dev(tokens), _dev(out), _stream()))
        return out

    def capture_decode(self, n_seqs: int) -> None:
        _check(_lib.b200attn_decode_graph_capture(self.h, C.c_int(n_seqs), _stream()))

    def launch_decode(self, steps: int) -> None:
        _check(_lib.b200attn_decode_graph_launch(self.h, C.c_int(steps), _stream()))

    def set_tokens(self, tokens: torch.Tensor) -> None:
        _check(_lib.b200attn_stack_set_tokens(self.h, _dev(tokens), C.c_int(tokens.numel()), _stream()))

    def get_tokens(self, n_seqs: int) -> torch.Tensor:
        out = torch.empty(n_seqs, dtype=torch.int32, device="cuda")
        _check(_lib.b200attn_stack_get_tokens(self.h, _dev(out), C.c_int(n_seqs), _stream()))
        return out

    # ---- continuous batching ----
    def begin_batching(self) -> None:
        _check(_lib.b200attn_stack_begin_batching(self.h, _stream()))

    def admit(self, prompt: torch.Tensor, reserve_tokens: int) -> int:
        """Admit one sequence (prompt: int32 device tensor); returns its row."""
        row = C.c_int(-1)
        _check(_lib.b200attn_stack_admit(self.h, _dev(prompt), C.c_int(prompt.numel()), C.c_int(reserve_tokens), C.byref(row), _stream()))
        return row.value

    def retire(self, row: int) -> None:
        _check(_lib.b200attn_stack_retire(self.h, C.c_int(row), _stream()))

    def rows(self) -> tuple[int, list[int]]:
        n = C.c_int(0)
        slots = (C.c_int * self.cfg.max_seqs)()
        _check(_lib.b200attn_stack_rows(self.h, C.byref(n), slots))
        return n.value, list(slots)

    def step(self, n_rows: int) -> None:
        _check(_lib.b200attn_stack_step(self.h, C.c_int(n_rows), _stream()))

    def __del__(self):
        try:
            if getattr(self, "h", None) and self.h.value:
                _lib.b200attn_stack_destroy(self.h)
        except Exception:
            pass


def fa_decode_core_static(q: torch.Tensor, kv: KVCache, layer: int, d_slots: torch.Tensor, out: torch.Tensor) -> None:
    """Decode attention core through the allocation-free entry point; `out` is supplied by the caller."""
    _check(_lib.b200attn_fa_decode_core_static(kv.h, C.c_int(layer), _dev(d_slots), C.c_int(d_slots.numel()), _dev(q),
                                               _dev(out), _stream()))


def profile_enable(on: bool) -> None:
    _check(_lib.b200attn_profile_enable(C.c_int(1 if on else 0)))


def profile_reset() -> None:
    _check(_lib.b200attn_profile_reset())


def profile_read(name: str) -> tuple[float, int]:
    """(summed device milliseconds, launches) of one kernel class since the last reset."""
    ms, n = C.c_double(0.0), C.c_longlong(0)
    _check(_lib.b200attn_profile_read(name.encode(), C.byref(ms), C.byref(n)))
    return ms.value, n.value
