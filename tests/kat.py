"""Known-answer recipes of the reference's own tests, restated in numpy.

Each generator and each expected-value routine follows one test of krea2-hrx and is
written independently of the C oracle (dense f64 Hadamard matrices, numpy float16),
so that agreeing with them pins the oracle; the GPU tests reuse the same recipes
against the CUDA kernels.
"""
from __future__ import annotations

import numpy as np

H4 = np.array([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], dtype=np.float64)


def values(n: int, scale: float) -> np.ndarray:
    """tests/quantized.rs:80-82: ((i*37 % 101) as f32 - 50) * scale / 50, all in f32."""
    i = np.arange(n, dtype=np.int64)
    base = ((i * 37) % 101).astype(np.float32) - np.float32(50.0)
    return (base * np.float32(scale)) / np.float32(50.0)


# ------------------------------------------------------------------ roundings
def bf16_bits_from_f32(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bits (finite inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def _f32_round_to_odd(x: np.ndarray) -> np.ndarray:
    """f64 -> f32 with round-to-odd, so a following RNE to fewer bits rounds once."""
    x = np.asarray(x, dtype=np.float64)
    f = x.astype(np.float32)
    over = np.abs(f.astype(np.float64)) > np.abs(x)
    t = np.where(over, np.nextafter(f, np.float32(0.0)), f).astype(np.float32)
    inexact = t.astype(np.float64) != x
    bits = t.view(np.uint32)
    bits = np.where(inexact, bits | np.uint32(1), bits).astype(np.uint32)
    return bits.view(np.float32)


def bf16_round_f64(x: np.ndarray) -> np.ndarray:
    """`bf16::from_f64(x).to_f64()` of the half crate: one direct RNE rounding."""
    return bf16_to_f32(bf16_bits_from_f32(_f32_round_to_odd(x))).astype(np.float64)


def bf16_round_f32(x: np.ndarray) -> np.ndarray:
    return bf16_to_f32(bf16_bits_from_f32(x))


def f16_bits(x: np.ndarray) -> np.ndarray:
    """f32/f64 -> f16 bits through numpy's IEEE conversion."""
    return np.asarray(x).astype(np.float16).view(np.uint16)


def f16_from_bits(bits: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(bits, dtype=np.uint16).view(np.float16)


def close(actual: np.ndarray, expected: np.ndarray, abs_tol: float, rel_tol: float) -> None:
    """tests/common/mod.rs:7-15."""
    actual = np.asarray(actual, dtype=np.float64).ravel()
    expected = np.asarray(expected, dtype=np.float64).ravel()
    assert actual.shape == expected.shape
    assert np.all(np.isfinite(actual))
    bad = np.abs(actual - expected) > abs_tol + rel_tol * np.abs(expected)
    assert not bad.any(), f"{bad.sum()} elements differ, first at {np.argmax(bad)}: " \
                          f"{actual[np.argmax(bad)]} vs {expected[np.argmax(bad)]}"


# ------------------------------------------------------------------ Hadamard
def kronecker_h256() -> np.ndarray:
    """tests/quantized.rs:390-399: H4 (x) H4 (x) H4 (x) H4 / 16, coefficient(i, j)."""
    h = np.ones((1, 1))
    for _ in range(4):
        h = np.kron(H4, h)  # digit d of i, j indexes the d-th factor, least significant first
    return h / 16.0


def staged_f16_rotation(row_f16: np.ndarray) -> np.ndarray:
    """tests/quantized.rs:538-552: 4x4 products per radix with an f16 rounding after each.

    `row_f16` is a float16 vector; returns float16."""
    row = row_f16.astype(np.float16).copy()
    width = row.shape[0]
    for step in (1, 4, 16, 64):
        v = row.astype(np.float64).reshape(width // (4 * step), 4, step)
        out = np.einsum("ij,bjs->bis", H4, v) * 0.25
        row = out.reshape(width).astype(np.float16)
    return row


# ------------------------------------------------------------------ GEMM KAT (tests/quantized.rs:171-280)
GEMM_SHAPES = [(17, 128, 128, 0), (17, 128, 128, 128), (257, 384, 256, 0), (257, 384, 256, 128)]
GEMM_MODES = [("plain", None), ("resid", None), ("swiglu", None), ("resid", False), ("resid", True)]


def gemm_case(m: int, k: int, n: int, pad: int):
    stride = k + pad
    a = ((np.arange(m * stride, dtype=np.int64) * 3) % 15 - 7).astype(np.int8).reshape(m, stride)
    w = ((np.arange(n * stride, dtype=np.int64) * 7) % 15 - 7).astype(np.int8).reshape(n, stride)
    ws = np.full(n, 0.01, dtype=np.float32)
    ws[3] = 0.0
    scales = np.full(m, 0.02, dtype=np.float32)
    scales[m - 1] = 0.0
    residual = bf16_bits_from_f32(values(m * n, 0.5)).reshape(m, n)
    gates = values(n, 0.3)
    dot = a[:, :k].astype(np.int64) @ w[:, :k].astype(np.int64).T
    full = dot.astype(np.float64) * ws.astype(np.float64)[None, :] * scales.astype(np.float64)[:, None]
    return dict(a=a, w=w, ws=ws, scales=scales, residual=residual, gates=gates, full=full, dot=dot,
                stride=stride)


def gemm_expected(mode: str, case) -> np.ndarray:
    full, n = case["full"], case["full"].shape[1]
    if mode == "resid":
        x = bf16_round_f32(full.astype(np.float32))
        gated = bf16_round_f32(case["gates"][None, :] * x)
        return bf16_round_f32(bf16_to_f32(case["residual"]) + gated).astype(np.float64)
    if mode == "swiglu":
        c = np.arange(n // 2)
        gate_col = (c // 16) * 32 + c % 16
        a = bf16_round_f64(full[:, gate_col])
        b = bf16_round_f64(full[:, gate_col + 16])
        return bf16_round_f64(bf16_round_f64(a / (1.0 + np.exp(-a))) * b)
    return bf16_round_f64(full)


# ------------------------------------------------------------------ prologue KATs
def preparation_case():
    """tests/quantized.rs:385-409: tokens 3, width 2048, out_stride 2176."""
    tokens, width, stride = 3, 2048, 2176
    norm_input = bf16_bits_from_f32(values(tokens * width, 1.5)).reshape(tokens, width)
    half_input = f16_bits(values(tokens * width, 0.5)).reshape(tokens, width)
    norm = values(width, 0.1)
    modulation = values(width, 0.2)
    shift = values(width, 0.15)
    gate = f16_bits(values(tokens * stride, 0.7)).reshape(tokens, stride)
    gate_stride = stride + 128
    padded = np.zeros((tokens, gate_stride), dtype=np.uint16)
    padded[:, :width] = gate[:, :width]
    return dict(tokens=tokens, width=width, stride=stride, norm_input=norm_input, half_input=half_input,
                norm=norm, modulation=modulation, shift=shift, gate=padded, gate_stride=gate_stride)


def preparation_formed(kind: str, case) -> np.ndarray:
    """The f64 row each prologue forms before rotating (tests/quantized.rs:410-445)."""
    width = case["width"]
    if kind == "norm":
        x = bf16_to_f32(case["norm_input"]).astype(np.float64)
        mean_square = (x ** 2).sum(axis=1, keepdims=True) / width
        normalized = bf16_round_f64(x / np.sqrt(mean_square + 1e-5) * (1.0 + case["norm"].astype(np.float64)))
        mod = bf16_round_f64(1.0 + case["modulation"].astype(np.float64))
        return bf16_round_f64(bf16_round_f64(mod * normalized) + case["shift"].astype(np.float64))
    half = f16_from_bits(case["half_input"]).astype(np.float64)
    if kind == "gated":
        attention = bf16_round_f64(half)
        g = f16_from_bits(case["gate"][:, :width]).astype(np.float64)
        sigmoid = bf16_round_f64(1.0 / (1.0 + np.exp(-g)))
        return bf16_round_f64(attention * sigmoid)
    return half


def check_preparation(kind: str, case, q: np.ndarray, q_scale: np.ndarray, fill: int = 0xA5) -> None:
    """tests/quantized.rs:477-510: scale within 0.2 %, codes within +-1 with < 2 % mismatches,
    padding bytes untouched."""
    tokens, width, stride = case["tokens"], case["width"], case["stride"]
    formed = preparation_formed(kind, case)
    h = kronecker_h256()
    rotated = (formed.reshape(tokens, width // 256, 256) @ h.T).reshape(tokens, width)
    scale = np.maximum(np.abs(rotated).max(axis=1), 1e-30) / 127.0
    actual_scale = q_scale.astype(np.float64)
    assert np.all(np.abs(actual_scale - scale) <= scale * 0.002 + 1e-30), f"{kind} scale"
    want = np.clip(np.rint(rotated / scale[:, None]), -127, 127).astype(np.int32)
    codes = q.reshape(tokens, stride)[:, :width].astype(np.int32)
    assert np.abs(codes - want).max() <= 1, f"{kind}: codes off by more than one"
    mismatches = int((codes != want).sum())
    assert mismatches / (tokens * width) < 0.02, f"{kind}: {mismatches} rounding mismatches"
    pad = q.reshape(tokens, stride)[:, width:].view(np.uint8)
    assert np.all(pad == fill), f"{kind}: padding was written"


def plain_boundary_case(width: int):
    """tests/quantized.rs:520-531: rows scaled 0, 0.5, 0.00001; out_stride = width + 64."""
    tokens = 3
    i = np.arange(tokens * width, dtype=np.int64)
    scale = np.array([0.0, 0.5, 0.00001], dtype=np.float32)[i // width]
    x = (((i * 37) % 101).astype(np.float32) - np.float32(50.0)) * scale / np.float32(50.0)
    return f16_bits(x).reshape(tokens, width), width + 64


def plain_boundary_expected(inp_bits: np.ndarray):
    """tests/quantized.rs:533-563: bit-exact scale and codes."""
    tokens, width = inp_bits.shape
    scales = np.zeros(tokens, dtype=np.float32)
    codes = np.zeros((tokens, width), dtype=np.int8)
    for t in range(tokens):
        row = staged_f16_rotation(f16_from_bits(inp_bits[t]))
        mx = np.abs(row.astype(np.float32)).max() if width else np.float32(0)
        scale = np.float32(max(np.float32(mx * np.float32(16.0)), np.float32(1e-30))) / np.float32(127.0)
        inv = np.float32(16.0) / np.float32(scale)
        r = row.astype(np.float32) * inv
        codes[t] = np.clip(np.rint(r), -127, 127).astype(np.int8)
        scales[t] = scale
    return codes, scales


def convrot_case(inputs: int):
    """src/training/quantized.rs:131-178: 3 tokens, 128 outputs, first row zero."""
    tokens, outputs = 3, 128
    i = np.arange(outputs * inputs, dtype=np.int64)
    weights = (((i * 37) % 31) - 15).astype(np.int8).reshape(outputs, inputs)
    scales = ((np.arange(outputs) % 7 + 1).astype(np.float32) / np.float32(256.0)).astype(np.float32)
    j = np.arange(tokens * inputs, dtype=np.int64)
    xf = np.where(j < inputs, np.float32(0.0), (((j * 17) % 97).astype(np.float32) - np.float32(48.0)) / np.float32(128.0))
    x_bf16 = bf16_bits_from_f32(xf.astype(np.float32)).reshape(tokens, inputs)
    return weights, scales, x_bf16


def convrot_expected(weights, scales, x_bf16) -> np.ndarray:
    """src/training/quantized.rs:188-221 without the adapter term: bf16 bits of
    bf16((dot as f32 * w_scale) * a_scale)."""
    tokens, inputs = x_bf16.shape
    out = np.zeros((tokens, weights.shape[0]), dtype=np.uint16)
    for t in range(tokens):
        row16 = bf16_to_f32(x_bf16[t]).astype(np.float16)
        rotated = staged_f16_rotation(row16)
        mx = np.abs(rotated.astype(np.float32)).max()
        scale = np.float32(max(np.float32(mx * np.float32(16.0)), np.float32(1e-30))) / np.float32(127.0)
        codes = np.clip(np.rint(rotated.astype(np.float32) * (np.float32(16.0) / scale)), -127, 127).astype(np.int64)
        dot = weights.astype(np.int64) @ codes
        base = (dot.astype(np.float32) * scales) * scale
        out[t] = bf16_bits_from_f32(base.astype(np.float32))
    return out


def swiglu_golden_accumulators(path):
    """tests/golden/swiglu_bf16.npz as the accumulators of a one-row gate|up GEMM: (acc [1][n], channel scales [n],
    expected f32 values [n/2], valid outputs).  Gate and up columns interleave in sixteens as the kernel expects."""
    g = np.load(path)
    gate, up = g["gate_acc"].reshape(-1), g["up_acc"].reshape(-1)
    outputs = gate.size
    padded = -(-outputs // 128) * 128
    gate = np.concatenate([gate, np.zeros(padded - outputs, np.int32)])
    up = np.concatenate([up, np.zeros(padded - outputs, np.int32)])
    acc = np.stack([gate.reshape(-1, 16), up.reshape(-1, 16)], axis=1).reshape(1, -1).astype(np.int32)
    want = (g["product"].reshape(-1).astype(np.uint32) << 16).view(np.float32)
    scale = np.tile(np.concatenate([np.full(16, 2.0 ** -15), np.full(16, 2.0 ** -8)]), acc.shape[1] // 32).astype(np.float32)
    return acc, scale, want, outputs


def weights_for_accumulators(acc_row, k=512):
    """int8 A [1][k] and W [n][k] whose product is `acc_row`: A is 127 over the first k-128 positions and 1 over the
    last 128, so W's first part carries round(acc / 127) spread over entries of at most 127 and its last part the
    remainder."""
    n = acc_row.size
    a = np.concatenate([np.full(k - 128, 127, np.int8), np.ones(128, np.int8)])[None, :]
    coarse = np.rint(acc_row / 127.0).astype(np.int64)
    rest = acc_row.astype(np.int64) - 127 * coarse
    assert np.all(np.abs(rest) <= 64) and np.all(np.abs(coarse) <= 127 * (k - 128))
    w = np.zeros((n, k), np.int64)
    slots = k - 128
    base, extra = np.divmod(np.abs(coarse), slots)
    w[:, :slots] = (base[:, None] + (np.arange(slots)[None, :] < extra[:, None])) * np.sign(coarse)[:, None]
    w[:, slots] = rest  # one position of weight 1 holds the remainder
    assert np.all(np.abs(w) <= 127)
    assert np.array_equal((a.astype(np.int64) @ w.T)[0], acc_row.astype(np.int64))
    return a, w.astype(np.int8)
