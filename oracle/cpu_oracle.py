"""TEST INFRASTRUCTURE ONLY — ctypes front ends for the two CPU checkers.

* ``Ref*``    : the reference's own CPU classes (qwen::FullAttention, qwen::LinearAttention,
                qwen::MLP) compiled from the reference checkout into ``oracle/_ref/libqwen_ref.so``
                by ``oracle/Makefile`` (shim: ``oracle/ref_shim.cpp``).
* ``Oracle*`` : this repository's C restatement, ``oracle/oracle.c`` -> ``oracle/liboracle.so``.

Both expose the same token-at-a-time interface so tests can swap them.  Only tests, the smoke
check and the benchmark's CPU-baseline leg import this module; the product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = C.POINTER(C.c_float)
_i8p = C.POINTER(C.c_int8)


def _fp(a):
    if a is None:
        return None
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f32p)


def reference_root() -> str:
    """Where the reference checkout lies: QWEN_REFERENCE_ROOT, else a directory named ``reference`` next to this
    repository.  It is only needed at build time; the GPU box runs the prebuilt files under oracle/_ref."""
    return os.environ.get("QWEN_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(force: bool = False) -> None:
    """Compile liboracle.so (always possible) and, when the reference checkout is present,
    oracle/_ref/libqwen_ref.so.  Building the checker is not using it."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so", "-B"], stdout=subprocess.DEVNULL)
    ref_so = os.path.join(_HERE, "_ref", "libqwen_ref.so")
    ref_root = reference_root()
    if os.path.isdir(os.path.join(ref_root, "src", "backend", "cpu", "core", "attention")):
        shim = os.path.join(_HERE, "ref_shim.cpp")
        if force or not os.path.exists(ref_so) or os.path.getmtime(ref_so) < os.path.getmtime(shim):
            subprocess.check_call(["make", "-C", _HERE, "ref", f"REF={ref_root}"], stdout=subprocess.DEVNULL)


def have_ref() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libqwen_ref.so"))


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(os.path.join(_HERE, "liboracle.so"))
        _lib.oracle_fa_forward.restype = C.c_int
        _lib.oracle_la_forward.restype = C.c_int
        _lib.oracle_count_ties.restype = C.c_int
        _lib.oracle_mlp.restype = C.c_int
    return _lib


def ref():
    global _ref
    if _ref is None:
        _ref = C.CDLL(os.path.join(_HERE, "_ref", "libqwen_ref.so"))
        _ref.ref_fa_create.restype = C.c_void_p
        _ref.ref_la_create.restype = C.c_void_p
        _ref.ref_mlp_create.restype = C.c_void_p
        _ref.ref_last_error.restype = C.c_char_p
    return _ref


# ------------------------------------------------------------------------------------------------
# Restatement (oracle.c)
# ------------------------------------------------------------------------------------------------
class _FaParams(C.Structure):
    _fields_ = [("hidden", C.c_int), ("heads", C.c_int), ("kv_heads", C.c_int), ("head_dim", C.c_int),
                ("rotary_dim", C.c_int), ("rope_theta", C.c_float),
                ("wq", _f32p), ("wk", _f32p), ("wv", _f32p), ("q_norm", _f32p), ("k_norm", _f32p),
                ("wo", _f32p)]


class _LaParams(C.Structure):
    _fields_ = [("hidden", C.c_int), ("heads", C.c_int), ("kd", C.c_int), ("vd", C.c_int),
                ("conv_k", C.c_int),
                ("w_qkv", _f32p), ("w_a", _f32p), ("w_b", _f32p), ("w_z", _f32p), ("conv_w", _f32p),
                ("a_log", _f32p), ("dt_bias", _f32p), ("norm_w", _f32p), ("w_out", _f32p)]


def quantize_head(x: np.ndarray):
    """INT8 codes + fp32 scale of one (token, kv head) row; see oracle.c:oracle_quantize_head."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    codes = np.empty(x.shape[0], dtype=np.int8)
    scale = C.c_float()
    lib().oracle_quantize_head(_fp(x), C.c_int(x.shape[0]), codes.ctypes.data_as(_i8p), C.byref(scale))
    return codes, np.float32(scale.value)


def quantize_rows(x: np.ndarray):
    """Vectorised numpy form of the same quantiser for [rows, n] inputs (bit-identical: IEEE fp32
    division, half-away-from-zero rounding, clamp)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    amax = np.max(np.abs(x), axis=-1).astype(np.float32)
    scale = (amax / np.float32(127.0)).astype(np.float32)
    scale = np.where(scale > np.float32(1e-8), scale, np.float32(1.0)).astype(np.float32)
    q = (x / scale[..., None]).astype(np.float32)
    r = np.sign(q) * np.floor(np.abs(q) + np.float32(0.5))          # roundf: half away from zero
    r = np.clip(r, -127.0, 127.0)
    return r.astype(np.int8), scale


def count_ties(x: np.ndarray, scale: float) -> int:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return int(lib().oracle_count_ties(_fp(x), C.c_int(x.size), C.c_float(scale)))


class OracleFullAttention:
    """Token-at-a-time gated full attention with an external fp32 cache (oracle_fa_forward)."""

    def __init__(self, w: dict, max_tokens: int, kv_mode: int = 0, hidden=1024, heads=8, kv_heads=2,
                 head_dim=256, rotary_dim=64, rope_theta=1e7):
        self.w = {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in w.items()}
        self.p = _FaParams(hidden, heads, kv_heads, head_dim, rotary_dim, rope_theta,
                           _fp(self.w["wq"]), _fp(self.w["wk"]), _fp(self.w["wv"]),
                           _fp(self.w["q_norm"]), _fp(self.w["k_norm"]), _fp(self.w["wo"]))
        self.kv_mode = kv_mode
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.k_cache = np.zeros((max_tokens, kv_heads * head_dim), np.float32)
        self.v_cache = np.zeros_like(self.k_cache)
        self.k_codes = np.zeros((max_tokens, kv_heads * head_dim), np.int8)
        self.v_codes = np.zeros_like(self.k_codes)
        self.k_scale = np.zeros((max_tokens, kv_heads), np.float32)
        self.v_scale = np.zeros_like(self.k_scale)
        self.len = C.c_int(0)
        self.q = np.zeros((max_tokens, heads * head_dim), np.float32)
        self.gate = np.zeros_like(self.q)
        self.attn = np.zeros_like(self.q)

    def forward(self, x: np.ndarray, position: int | None = None) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(self.hidden, np.float32)
        t = self.len.value
        pos = t if position is None else position
        rc = lib().oracle_fa_forward(
            C.byref(self.p), _fp(x), _fp(y), _fp(self.k_cache), _fp(self.v_cache), C.byref(self.len),
            C.c_int(pos), C.c_int(self.kv_mode),
            self.k_codes[t].ctypes.data_as(_i8p), self.v_codes[t].ctypes.data_as(_i8p),
            _fp(self.k_scale[t]), _fp(self.v_scale[t]), _fp(self.q[t]), _fp(self.gate[t]), _fp(self.attn[t]))
        assert rc == 0
        return y

    def forward_sequence(self, xs: np.ndarray) -> np.ndarray:
        return np.stack([self.forward(x) for x in xs])


class OracleLinearAttention:
    """Token-at-a-time Gated DeltaNet with external state (oracle_la_forward)."""

    def __init__(self, w: dict, hidden=1024, heads=16, kd=128, vd=128, conv_k=4):
        self.w = {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in w.items()}
        self.p = _LaParams(hidden, heads, kd, vd, conv_k,
                           _fp(self.w["w_qkv"]), _fp(self.w["w_a"]), _fp(self.w["w_b"]), _fp(self.w["w_z"]),
                           _fp(self.w["conv_w"]), _fp(self.w["a_log"]), _fp(self.w["dt_bias"]),
                           _fp(self.w["norm_w"]), _fp(self.w["w_out"]))
        self.hidden, self.heads, self.kd, self.vd, self.conv_k = hidden, heads, kd, vd, conv_k
        self.conv_dim = heads * (2 * kd + vd)
        self.recurrent = np.zeros((heads, kd, vd), np.float32)
        self.conv_state = np.zeros((self.conv_dim, conv_k - 1), np.float32)   # [:, 0] = newest

    def forward(self, x: np.ndarray, taps: dict | None = None) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(self.hidden, np.float32)
        t = {}
        if taps is not None:
            t = dict(q=np.empty(self.heads * self.kd, np.float32), k=np.empty(self.heads * self.kd, np.float32),
                     v=np.empty(self.heads * self.vd, np.float32), g=np.empty(self.heads, np.float32),
                     beta=np.empty(self.heads, np.float32), core=np.empty(self.heads * self.vd, np.float32))
            taps.update(t)
        rc = lib().oracle_la_forward(C.byref(self.p), _fp(x), _fp(y), _fp(self.recurrent), _fp(self.conv_state),
                                     _fp(t.get("q")), _fp(t.get("k")), _fp(t.get("v")), _fp(t.get("g")),
                                     _fp(t.get("beta")), _fp(t.get("core")))
        assert rc == 0
        return y

    def forward_sequence(self, xs: np.ndarray) -> np.ndarray:
        return np.stack([self.forward(x) for x in xs])


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w, dtype=np.float32)
    y = np.empty_like(x)
    lib().oracle_rmsnorm(_fp(x), _fp(w), _fp(y), C.c_int(x.shape[0]), C.c_float(eps))
    return y


def mlp(gate_w, up_w, down_w, x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty_like(x)
    inter, hidden = gate_w.shape
    rc = lib().oracle_mlp(_fp(gate_w), _fp(up_w), _fp(down_w), _fp(x), _fp(y), C.c_int(hidden), C.c_int(inter))
    assert rc == 0
    return y


def quantize_weight_rows(w: np.ndarray):
    """Returns (dequantised weight, codes, scales) for per-output-channel INT8 weights."""
    w = np.array(w, dtype=np.float32, order="C", copy=True)
    codes = np.empty(w.shape, np.int8)
    scales = np.empty(w.shape[0], np.float32)
    lib().oracle_quantize_weight_rows(_fp(w), C.c_int(w.shape[0]), C.c_int(w.shape[1]),
                                      codes.ctypes.data_as(_i8p), _fp(scales))
    return w, codes, scales


# ------------------------------------------------------------------------------------------------
# Compiled reference (oracle/_ref)
# ------------------------------------------------------------------------------------------------
class RefFullAttention:
    """qwen::FullAttention + qwen::KVCache from the reference, one layer."""

    def __init__(self, w: dict, max_tokens: int, hidden=1024, heads=8, kv_heads=2, head_dim=256):
        r = ref()
        self.hidden, self.kvw = hidden, kv_heads * head_dim
        self.h = C.c_void_p(r.ref_fa_create(hidden, heads, kv_heads, head_dim, head_dim, 1, max_tokens))
        assert self.h.value, r.ref_last_error()
        ws = [np.ascontiguousarray(w[k], dtype=np.float32) for k in ("wq", "wk", "wv", "q_norm", "k_norm", "wo")]
        rc = r.ref_fa_set_weights(self.h, *[_fp(a) for a in ws])
        assert rc == 0, r.ref_last_error()

    def forward(self, x: np.ndarray, position: int | None = None) -> np.ndarray:
        r = ref()
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(self.hidden, np.float32)
        pos = r.ref_fa_cache_len(self.h, 0) if position is None else position
        rc = r.ref_fa_forward(self.h, _fp(x), _fp(y), 0, pos)
        assert rc == 0, r.ref_last_error()
        return y

    def forward_sequence(self, xs):
        return np.stack([self.forward(x) for x in xs])

    def cache(self):
        r = ref()
        n = r.ref_fa_cache_len(self.h, 0)
        k = np.empty((n, self.kvw), np.float32)
        v = np.empty((n, self.kvw), np.float32)
        r.ref_fa_cache_read(self.h, 0, _fp(k), _fp(v))
        return k, v

    def __del__(self):
        try:
            ref().ref_fa_destroy(self.h)
        except Exception:
            pass


class RefLinearAttention:
    """qwen::LinearAttention + qwen::LinearAttnState from the reference."""

    def __init__(self, w: dict, hidden=1024, heads=16, kd=128, vd=128, conv_k=4):
        r = ref()
        self.hidden, self.heads, self.kd, self.vd, self.conv_k = hidden, heads, kd, vd, conv_k
        self.conv_dim = heads * (2 * kd + vd)
        self.h = C.c_void_p(r.ref_la_create(hidden, heads, kd, vd, conv_k))
        assert self.h.value, r.ref_last_error()
        order = ("w_qkv", "w_a", "w_b", "w_z", "conv_w", "a_log", "dt_bias", "norm_w", "w_out")
        ws = [np.ascontiguousarray(w[k], dtype=np.float32) for k in order]
        rc = r.ref_la_set_weights(self.h, *[_fp(a) for a in ws])
        assert rc == 0, r.ref_last_error()

    def forward(self, x):
        r = ref()
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty(self.hidden, np.float32)
        rc = r.ref_la_forward(self.h, _fp(x), _fp(y))
        assert rc == 0, r.ref_last_error()
        return y

    def forward_sequence(self, xs):
        return np.stack([self.forward(x) for x in xs])

    def state(self):
        rec = np.empty((self.heads, self.kd, self.vd), np.float32)
        conv = np.empty((self.conv_dim, self.conv_k - 1), np.float32)
        ref().ref_la_state_get(self.h, _fp(rec), _fp(conv))
        return rec, conv

    def set_state(self, rec, conv):
        rec = np.ascontiguousarray(rec, dtype=np.float32)
        conv = np.ascontiguousarray(conv, dtype=np.float32)
        ref().ref_la_state_set(self.h, _fp(rec), _fp(conv))

    def __del__(self):
        try:
            ref().ref_la_destroy(self.h)
        except Exception:
            pass


class RefMLP:
    def __init__(self, gate_w, up_w, down_w):
        self.ws = [np.ascontiguousarray(a, dtype=np.float32) for a in (gate_w, up_w, down_w)]
        inter, hidden = self.ws[0].shape
        self.hidden = hidden
        self.h = C.c_void_p(ref().ref_mlp_create(hidden, inter, *[_fp(a) for a in self.ws]))
        assert self.h.value

    def forward(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        rc = ref().ref_mlp_forward(self.h, _fp(x), _fp(y), C.c_int(self.hidden))
        assert rc == 0
        return y

    def __del__(self):
        try:
            ref().ref_mlp_destroy(self.h)
        except Exception:
            pass
