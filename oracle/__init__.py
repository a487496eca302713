"""numpy front end of the CPU oracle (``w8a8_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline legs of ``bench.py``.  The shipped package never imports it.

bf16 and f16 tensors travel as ``uint16`` arrays of raw bits; int8 codes as ``int8``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it; returns the library path."""
    src = os.path.join(_HERE, "w8a8_oracle.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.oracle_exp.restype = ctypes.c_float
        _lib.oracle_exp.argtypes = [ctypes.c_float]
        _lib.oracle_threads.restype = ctypes.c_int
        _lib.oracle_dynamic_mu.restype = ctypes.c_double
        _lib.oracle_dynamic_mu.argtypes = [ctypes.c_size_t]
        _lib.oracle_sigma.restype = ctypes.c_float
        _lib.oracle_sigma.argtypes = [ctypes.c_size_t, ctypes.c_size_t, ctypes.c_double]
        _lib.oracle_next_sigma.restype = ctypes.c_float
        _lib.oracle_next_sigma.argtypes = [ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_double]
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


def _sz(v: int):
    return ctypes.c_size_t(int(v))


def threads() -> int:
    return int(lib().oracle_threads())


def set_threads(n: int) -> None:
    """OpenMP threads for later calls, overriding an inherited OMP_NUM_THREADS."""
    lib().oracle_set_threads(int(n))


# ------------------------------------------------------------------ conversions
def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_f32_to_f16(_p(x), _p(out), _sz(x.size))
    return out


def f16_bits_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().oracle_f16_to_f32(_p(x), _p(out), _sz(x.size))
    return out


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16(_p(x), _p(out), _sz(x.size))
    return out


def bf16_bits_to_f32(x: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(x, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def exp(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    return np.array([lib().oracle_exp(float(v)) for v in x.ravel()], dtype=np.float32).reshape(x.shape)


# ------------------------------------------------------------------ prologues
def _q_out(tokens: int, out_stride: int, fill: int) -> np.ndarray:
    return np.full((tokens, out_stride), fill, dtype=np.uint8).view(np.int8)


def prepare_norm_i8(h, norm_scale, mod_scale, mod_shift, width, out_stride, eps=1e-5, fill=0):
    """h: uint16 bf16 bits [tokens][width] -> (q int8 [tokens][out_stride], q_scale f32 [tokens])."""
    h = np.ascontiguousarray(h, dtype=np.uint16).reshape(-1, width)
    tokens = h.shape[0]
    ns, ms, sh = (np.ascontiguousarray(v, dtype=np.float32) for v in (norm_scale, mod_scale, mod_shift))
    q, s = _q_out(tokens, out_stride, fill), np.zeros(tokens, dtype=np.float32)
    lib().oracle_prepare_norm_i8(_sz(tokens), _p(h), _p(ns), _p(ms), _p(sh), _p(q), _p(s), _sz(width),
                                 _sz(out_stride), ctypes.c_float(eps))
    return q, s


def norm_modulate(h, norm_scale, mod_scale, mod_shift, width, eps=1e-5):
    """The front half of prepare_norm_i8 -- RMSNorm with `1 + norm_scale`, then adaLN -- as bf16 bits [tokens][width]:
    what the Hadamard rotation receives."""
    h = np.ascontiguousarray(h, dtype=np.uint16).reshape(-1, width)
    ns, ms, sh = (np.ascontiguousarray(v, dtype=np.float32) for v in (norm_scale, mod_scale, mod_shift))
    out = np.zeros_like(h)
    lib().oracle_norm_modulate(_sz(h.shape[0]), _p(h), _p(ns), _p(ms), _p(sh), _p(out), _sz(width), ctypes.c_float(eps))
    return out


def gate_attention(attn, gate, width, gate_stride):
    """The front half of prepare_gated_i8 -- attention output times bf16(sigmoid(gate)), rounded to bf16 -- as bf16
    bits [tokens][width]; attn and gate are f16 bits."""
    attn = np.ascontiguousarray(attn, dtype=np.uint16).reshape(-1, width)
    gate = np.ascontiguousarray(gate, dtype=np.uint16).reshape(-1, gate_stride)
    out = np.zeros_like(attn)
    lib().oracle_gate_attention(_sz(attn.shape[0]), _p(attn), _p(gate), _p(out), _sz(width), _sz(gate_stride))
    return out


def prepare_gated_i8(attn, gate, width, out_stride, gate_stride, fill=0):
    """attn: f16 bits [tokens][width]; gate: f16 bits [tokens][gate_stride]."""
    attn = np.ascontiguousarray(attn, dtype=np.uint16).reshape(-1, width)
    gate = np.ascontiguousarray(gate, dtype=np.uint16).reshape(-1, gate_stride)
    tokens = attn.shape[0]
    q, s = _q_out(tokens, out_stride, fill), np.zeros(tokens, dtype=np.float32)
    lib().oracle_prepare_gated_i8(_sz(tokens), _p(attn), _p(gate), _p(q), _p(s), _sz(width), _sz(out_stride),
                                  _sz(gate_stride))
    return q, s


def prepare_plain_i8(h, width, out_stride, fill=0):
    """h: f16 bits [tokens][width]."""
    h = np.ascontiguousarray(h, dtype=np.uint16).reshape(-1, width)
    tokens = h.shape[0]
    q, s = _q_out(tokens, out_stride, fill), np.zeros(tokens, dtype=np.float32)
    lib().oracle_prepare_plain_i8(_sz(tokens), _p(h), _p(q), _p(s), _sz(width), _sz(out_stride))
    return q, s


# ------------------------------------------------------------------ GEMMs
def gemm_i8_acc(a, w, k_size, k_stride, n_size):
    """a: int8 [m][k_stride], w: int8 [n][k_stride] -> i32 [m][n]."""
    a = np.ascontiguousarray(a, dtype=np.int8).reshape(-1, k_stride)
    w = np.ascontiguousarray(w, dtype=np.int8).reshape(n_size, k_stride)
    m = a.shape[0]
    acc = np.empty((m, n_size), dtype=np.int32)
    lib().oracle_gemm_i8_acc(_sz(m), _p(a), _p(w), _p(acc), _sz(k_size), _sz(k_stride), _sz(n_size))
    return acc


def epilogue_plain(acc, scale, a_scale):
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    m, n = acc.shape
    scale, a_scale = np.ascontiguousarray(scale, np.float32), np.ascontiguousarray(a_scale, np.float32)
    c = np.empty((m, n), dtype=np.uint16)
    lib().oracle_epilogue_plain(_sz(m), _p(acc), _p(scale), _p(a_scale), _p(c), _sz(n))
    return c


def epilogue_resid(acc, scale, a_scale, c, gate):
    """Returns the updated bf16 residual (the input array is not modified)."""
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    m, n = acc.shape
    scale, a_scale, gate = (np.ascontiguousarray(v, np.float32) for v in (scale, a_scale, gate))
    out = np.array(c, dtype=np.uint16, copy=True).reshape(m, n)
    lib().oracle_epilogue_resid(_sz(m), _p(acc), _p(scale), _p(a_scale), _p(out), _p(gate), _sz(n))
    return out


def epilogue_swiglu(acc, scale, a_scale):
    acc = np.ascontiguousarray(acc, dtype=np.int32)
    m, n = acc.shape
    scale, a_scale = np.ascontiguousarray(scale, np.float32), np.ascontiguousarray(a_scale, np.float32)
    c = np.empty((m, n // 2), dtype=np.uint16)
    lib().oracle_epilogue_swiglu(_sz(m), _p(acc), _p(scale), _p(a_scale), _p(c), _sz(n))
    return c


def gemm_i8_256(a, w, scale, a_scale, k_size, k_stride, n_size):
    return epilogue_plain(gemm_i8_acc(a, w, k_size, k_stride, n_size), scale, a_scale)


def gemm_i8_resid_256(a, w, scale, a_scale, c, gate, k_size, k_stride, n_size):
    return epilogue_resid(gemm_i8_acc(a, w, k_size, k_stride, n_size), scale, a_scale, c, gate)


def gemm_i8_swiglu_256(a, w, scale, a_scale, k_size, k_stride, n_size):
    return epilogue_swiglu(gemm_i8_acc(a, w, k_size, k_stride, n_size), scale, a_scale)


def transport_bf16_to_f16(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty_like(x)
    lib().oracle_transport_bf16_to_f16(_p(x), _p(out), _sz(x.size))
    return out


def transport_f16_to_bf16(x):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty_like(x)
    lib().oracle_transport_f16_to_bf16(_p(x), _p(out), _sz(x.size))
    return out


# ------------------------------------------------------------------ the rest of a block
def rope_qknorm_f16(qkv, q_scale, k_scale, cos, sin, row_stride, q_heads, kv_heads, k_offset, eps=1e-5):
    qkv = np.ascontiguousarray(qkv, dtype=np.uint16).reshape(-1, row_stride)
    tokens = qkv.shape[0]
    qs, ks, cos, sin = (np.ascontiguousarray(v, dtype=np.float32) for v in (q_scale, k_scale, cos, sin))
    q = np.zeros((tokens, q_heads * 128), dtype=np.uint16)
    k = np.zeros((tokens, kv_heads * 128), dtype=np.uint16)
    v = np.zeros((tokens, kv_heads * 128), dtype=np.uint16)
    lib().oracle_rope_qknorm_f16(_sz(tokens), _p(qkv), _p(qs), _p(ks), _p(cos), _p(sin), _p(q), _p(k), _p(v),
                                 _sz(row_stride), _sz(q_heads), _sz(kv_heads), _sz(k_offset), ctypes.c_float(eps))
    return q, k, v


def v_transpose(x, width, capacity, out=None):
    x = np.ascontiguousarray(x, dtype=np.uint16).reshape(-1, width)
    out = np.zeros((width, capacity), dtype=np.uint16) if out is None else out
    lib().oracle_v_transpose(_sz(x.shape[0]), _p(x), _p(out), _sz(width), _sz(capacity))
    return out


def attention_gqa(q, k, v, q_heads, kv_heads, scale):
    """q [tokens][q_heads*128], k, v [tokens][kv_heads*128] as f16 bits -> f64 [tokens][q_heads*128]."""
    q = np.ascontiguousarray(q, dtype=np.uint16)
    queries = q.reshape(-1, q_heads * 128).shape[0]  # may be a subset of the rows: every query sees all keys
    k, v = np.ascontiguousarray(k, dtype=np.uint16), np.ascontiguousarray(v, dtype=np.uint16)
    tokens = k.reshape(-1, kv_heads * 128).shape[0]
    out = np.zeros((queries, q_heads * 128), dtype=np.float64)
    lib().oracle_attention_gqa(_sz(queries), _sz(tokens), _sz(q_heads), _sz(kv_heads), _p(q), _p(k), _p(v), _p(out),
                               ctypes.c_double(scale))
    return out


# ------------------------------------------------------------------ the outer step
def modulation(x, tables):
    """x: bf16 bits [xsize]; tables: bf16 bits [count] -> f32 [count] (bf16-rounded sums)."""
    x, tables = np.ascontiguousarray(x, dtype=np.uint16), np.ascontiguousarray(tables, dtype=np.uint16)
    y = np.empty(tables.size, dtype=np.float32)
    lib().oracle_modulation(_sz(tables.size), _p(x), _p(tables), _p(y), _sz(x.size))
    return y.reshape(tables.shape)


def euler(sample, velocity, delta):
    """Returns the updated bf16 sample (the input array is not modified)."""
    out = np.array(sample, dtype=np.uint16, copy=True)
    velocity = np.ascontiguousarray(velocity, dtype=np.uint16)
    lib().oracle_euler(_sz(out.size), ctypes.c_float(delta), _p(out), _p(velocity))
    return out


def guidance(cond, uncond, scale):
    """Returns the updated bf16 conditional velocity (the input array is not modified)."""
    out = np.array(cond, dtype=np.uint16, copy=True)
    uncond = np.ascontiguousarray(uncond, dtype=np.uint16)
    lib().oracle_guidance(_sz(out.size), ctypes.c_float(scale), _p(out), _p(uncond))
    return out


def dynamic_mu(image_tokens: int) -> float:
    return float(lib().oracle_dynamic_mu(image_tokens))


def sigma(step: int, steps: int, mu: float) -> float:
    return float(lib().oracle_sigma(step, steps, mu))


def next_sigma(step: int, last: int, steps: int, mu: float) -> float:
    return float(lib().oracle_next_sigma(step, last, steps, mu))
