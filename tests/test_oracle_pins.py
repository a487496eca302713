"""Pins the CPU oracle to the reference's own known-answer tests (restated in kat.py)."""
import os

import numpy as np
import pytest

import kat
import oracle


def test_f16_conversion_matches_ieee():
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 200000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 70000.0, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0000001,
                  2.0 ** -14, 2.0 ** -14 * 0.9999, 1e-8, 3e-8, 5.96e-8, 8.9e-8, np.inf, -np.inf], dtype=np.float32),
        np.arange(0, 65536, dtype=np.uint16).view(np.float16).astype(np.float32),
    ])
    x = x[np.isfinite(x) | np.isinf(x)]
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = oracle.f32_to_f16_bits(x)
    np.testing.assert_array_equal(got, want)
    every = np.arange(0, 65536, dtype=np.uint16)
    finite = np.isfinite(every.view(np.float16))
    np.testing.assert_array_equal(oracle.f16_bits_to_f32(every[finite]), every[finite].view(np.float16).astype(np.float32))


def test_bf16_conversion_matches_rule():
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(300000) * 10.0 ** rng.integers(-20, 20, 300000)).astype(np.float32)
    np.testing.assert_array_equal(oracle.f32_to_bf16_bits(x), kat.bf16_bits_from_f32(x))
    # adversarial: exact ties
    ties = (np.arange(0x3F80, 0x4000, dtype=np.uint32) << 16 | 0x8000).view(np.float32)
    np.testing.assert_array_equal(oracle.f32_to_bf16_bits(ties), kat.bf16_bits_from_f32(ties))


def test_canonical_exp_is_accurate():
    x = np.linspace(-100, 88, 20001).astype(np.float32)
    got = oracle.exp(x).astype(np.float64)
    want = np.exp(x.astype(np.float64))
    rel = np.abs(got - want) / want
    assert rel[want > 1e-37].max() < 2.5e-7
    assert oracle.exp(np.array([-200.0], np.float32))[0] == 0.0
    assert np.isinf(oracle.exp(np.array([89.0], np.float32))[0])
    assert oracle.exp(np.array([0.0], np.float32))[0] == 1.0


@pytest.mark.parametrize("mode,wide", kat.GEMM_MODES)
@pytest.mark.parametrize("m,k,n,pad", kat.GEMM_SHAPES)
def test_integer_gemms_preserve_pitches_bf16_residuals_and_swiglu_order(mode, wide, m, k, n, pad):
    """tests/quantized.rs:171-280."""
    if wide is not None:
        n *= 2
    case = kat.gemm_case(m, k, n, pad)
    want = kat.gemm_expected(mode, case)
    acc = oracle.gemm_i8_acc(case["a"], case["w"], k, case["stride"], n)
    np.testing.assert_array_equal(acc.astype(np.int64), case["dot"])
    if mode == "plain":
        out = kat.f16_from_bits(oracle.epilogue_plain(acc, case["ws"], case["scales"])).astype(np.float64)
    elif mode == "swiglu":
        out = kat.f16_from_bits(oracle.epilogue_swiglu(acc, case["ws"], case["scales"])).astype(np.float64)
    else:
        out = kat.bf16_to_f32(oracle.epilogue_resid(acc, case["ws"], case["scales"], case["residual"],
                                                    case["gates"])).astype(np.float64)
    assert np.all(kat.bf16_round_f64(out) == out), "outputs must be bf16-representable"
    kat.close(out, want, 2e-3, 4e-3)


@pytest.mark.parametrize("kind", ["norm", "gated", "plain"])
def test_quantized_preparation_matches_the_kronecker_hadamard_and_preserves_padding(kind):
    """tests/quantized.rs:385-512."""
    case = kat.preparation_case()
    w, s = case["width"], case["stride"]
    if kind == "norm":
        q, qs = oracle.prepare_norm_i8(case["norm_input"], case["norm"], case["modulation"], case["shift"], w, s,
                                       1e-5, fill=0xA5)
    elif kind == "gated":
        q, qs = oracle.prepare_gated_i8(case["half_input"], case["gate"], w, s, case["gate_stride"], fill=0xA5)
    else:
        q, qs = oracle.prepare_plain_i8(case["half_input"], w, s, fill=0xA5)
    kat.check_preparation(kind, case, q, qs)


@pytest.mark.parametrize("width", [2048, 6144, 16384])
def test_plain_preparation_preserves_each_half_rounding_boundary(width):
    """tests/quantized.rs:514-569: bit-exact scale bytes and codes."""
    inp, stride = kat.plain_boundary_case(width)
    q, qs = oracle.prepare_plain_i8(inp, width, stride, fill=0xA5)
    codes, scales = kat.plain_boundary_expected(inp)
    np.testing.assert_array_equal(qs.view(np.uint32), scales.view(np.uint32))
    np.testing.assert_array_equal(q[:, :width], codes)
    assert np.all(q[:, width:].view(np.uint8) == 0xA5)


@pytest.mark.parametrize("inputs", [6144, 16384])
def test_convrot_path_matches_integer_cpu_algebra(inputs):
    """src/training/quantized.rs:124-225 (base term): bit-exact bf16 output."""
    weights, scales, x_bf16 = kat.convrot_case(inputs)
    pitch = inputs + 64 if inputs % 8192 == 0 else inputs
    wq = np.zeros((weights.shape[0], pitch), dtype=np.int8)
    wq[:, :inputs] = weights
    transport = oracle.transport_bf16_to_f16(x_bf16)
    q, qs = oracle.prepare_plain_i8(transport, inputs, pitch)
    out16 = oracle.gemm_i8_256(q, wq, scales, qs, inputs, pitch, weights.shape[0])
    got = oracle.transport_f16_to_bf16(out16)
    np.testing.assert_array_equal(got, kat.convrot_expected(weights, scales, x_bf16))


@pytest.mark.parametrize("name", ["small", "hidden"])
def test_oracle_tracks_the_reference_torch_scheme(name):
    """Golden vectors generated from scripts/quantized_reference.py:76-125 (tolerance reference:
    dense f32 rotation, no f16 stage rounding, no bf16 output rounding)."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", f"quantlinear_{name}.npz"))
    x, w, ws = g["x"], g["w"], g["ws"]
    m, k = x.shape
    n = w.shape[0]
    q, qs = oracle.prepare_plain_i8(x, k, k)
    # per-token scales agree to f16-stage rounding noise; codes differ by at most one step
    assert np.abs(qs / g["scales"] - 1).max() < 2e-3
    diff = np.abs(q.astype(np.int32) - g["codes"].astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 0.05
    out = kat.f16_from_bits(oracle.gemm_i8_256(q, w, ws, qs, k, k, n)).astype(np.float64)
    ref = kat.f16_from_bits(g["out"]).astype(np.float64)
    rel_l2 = np.linalg.norm(out - ref) / np.linalg.norm(ref)
    assert rel_l2 < 1e-2, rel_l2


def test_qk_norm_and_rope_equal_the_reference_torch_code_bit_for_bit():
    """tests/golden/rope_qknorm.npz: `rms_norm` and `apply_rope` of scripts/quantized_reference.py (:71-73, :158-162),
    imported unmodified by tests/golden/make_rope_golden.py and applied as `Krea2Ref.attention` applies them (:211-214),
    with the reference's own rope tables.  Both sides round to bf16 after the norm and after the rotation, so the
    oracle's q and k must be the reference's bf16 values exactly (an f16 holds them); V is copied through."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "rope_qknorm.npz"))
    fused = oracle.bf16_bits_to_f32(g["fused"])
    as_f16 = fused.astype(np.float16)
    assert np.array_equal(as_f16.astype(np.float32), fused), "the inputs are exact in f16"
    q, k, v = oracle.rope_qknorm_f16(as_f16.view(np.uint16), g["q_scale"], g["k_scale"], g["cos"], g["sin"], 1536, 8, 2, 8 * 128)
    np.testing.assert_array_equal(q.view(np.float16).astype(np.float32), oracle.bf16_bits_to_f32(g["q"]))
    np.testing.assert_array_equal(k.view(np.float16).astype(np.float32), oracle.bf16_bits_to_f32(g["k"]))
    np.testing.assert_array_equal(v.view(np.float16).astype(np.float32), fused[:, 10 * 128:])


def test_the_swiglu_epilogue_equals_torchs_silu_product_bit_for_bit():
    """tests/golden/swiglu_bf16.npz: `F.silu(g) * u` on bf16 tensors, the statement of `Krea2Ref.swiglu`
    (scripts/quantized_reference.py:222-225), made by tests/golden/make_swiglu_golden.py: every bf16 gate value with an
    exponent from -8 to 6 against eight up values.  Both sides round the SiLU and the product to bf16; the kernel's f16
    output holds every such value of normal f16 magnitude exactly, smaller ones to an f16 subnormal step."""
    acc, scale, want, outputs = kat.swiglu_golden_accumulators(os.path.join(os.path.dirname(__file__), "golden", "swiglu_bf16.npz"))
    c = oracle.epilogue_swiglu(acc, scale, np.ones(1, np.float32))
    got = c.view(np.float16).astype(np.float32)[0][:outputs]
    normal = np.abs(want) >= 2.0 ** -14
    assert normal.sum() > 27000
    np.testing.assert_array_equal(got[normal], want[normal])
    assert np.abs(got - want)[~normal].max() <= 2.0 ** -25


def test_the_residual_epilogue_equals_torchs_gated_update_bit_for_bit():
    """tests/golden/resid_bf16.npz: `x + gate * a` on bf16 tensors, the residual update of `Krea2Ref.block`
    (scripts/quantized_reference.py:262-268), made by tests/golden/make_resid_golden.py: the product and the sum each
    round to bf16, cancellation and absorption included."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "resid_bf16.npz"))
    acc = g["acc"][None, :]
    out = oracle.epilogue_resid(acc, np.full(acc.shape[1], 2.0 ** -12, np.float32), np.ones(1, np.float32), g["x"][None, :],
                                oracle.bf16_bits_to_f32(g["gate"]))
    np.testing.assert_array_equal(out[0], g["out"])


def test_rmsnorm_and_adaln_equal_the_reference_torch_expression_bit_for_bit():
    """tests/golden/norm_modulate.npz: `(1.0 + prescale) * rms_norm(x, scale) + preshift` on bf16 tensors, the argument
    `Krea2Ref.block` hands to its attention and MLP (scripts/quantized_reference.py:265, :267; `rms_norm` imported
    unmodified by tests/golden/make_norm_golden.py).  The front half of prepare_norm_i8 -- the sum of squares in the
    kernel's order, 1/sqrt, and four bf16 roundings -- must give the same bf16 values on all 73,728 of them."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "norm_modulate.npz"))
    got = oracle.norm_modulate(g["x"], g["scale"], oracle.bf16_bits_to_f32(g["prescale"]), oracle.bf16_bits_to_f32(g["preshift"]),
                               g["x"].shape[1])
    np.testing.assert_array_equal(got, g["out"])


def test_the_attention_gate_equals_torchs_sigmoid_product_bit_for_bit():
    """tests/golden/gate_attention.npz: `o * torch.sigmoid(gate)` on bf16 tensors (`Krea2Ref.attention`,
    scripts/quantized_reference.py:219), every bf16 gate value with an exponent from -8 to 6.  The front half of
    prepare_gated_i8 -- the canonical exp, the reciprocal and two bf16 roundings -- must give the same bf16 values."""
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "gate_attention.npz"))
    as_f16 = lambda b: oracle.bf16_bits_to_f32(b).astype(np.float16).view(np.uint16)
    n = g["gate"].size
    got = oracle.gate_attention(as_f16(g["attn"]).reshape(1, n), as_f16(g["gate"]).reshape(1, n), n, n)
    np.testing.assert_array_equal(got.reshape(-1), g["out"].reshape(-1))


def _sdpa_case():
    import importlib.util
    golden = os.path.join(os.path.dirname(__file__), "golden")
    spec = importlib.util.spec_from_file_location("make_attention_golden", os.path.join(golden, "make_attention_golden.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)  # only its seeded `inputs()` is used; torch is imported but not called
    q, k, v = module.inputs()
    want = oracle.bf16_bits_to_f32(np.load(os.path.join(golden, "attention_sdpa.npz"))["out"])
    return q, k, v, want


def test_float64_attention_tracks_torchs_scaled_dot_product_attention():
    """tests/golden/attention_sdpa.npz: `F.scaled_dot_product_attention` on bf16 tensors with the key/value heads
    repeated over their query groups (`Krea2Ref.attention`, scripts/quantized_reference.py:215-218); 208 tokens, eight
    query heads over two key/value heads.  torch's output is bf16, so the float64 oracle is held to the tolerance of the
    reference's attention test (tests/quantized.rs:309-383) and to a relative RMS of half a bf16 step."""
    q, k, v, want = _sdpa_case()
    as_f16 = lambda a: a.astype(np.float16).view(np.uint16)
    got = oracle.attention_gqa(as_f16(q), as_f16(k), as_f16(v), 8, 2, 1.0 / np.sqrt(128.0))
    err = np.abs(got - want)
    assert np.all(err <= 2e-2 + 2e-2 * np.abs(want))
    assert np.sqrt((err ** 2).sum() / (want ** 2).sum()) < 0.003
