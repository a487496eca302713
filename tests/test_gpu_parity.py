"""Parity of the CUDA kernels with the CPU oracle and the reference's known-answer tests,
through the C ABI.  Integer outputs (int8 codes, i32 accumulators) and, because the oracle
fixes every f32 order, the f32 scales and the f16/bf16 outputs are compared bit for bit; the
reference's own tolerances (tests/quantized.rs) are asserted beside that."""
import numpy as np
import pytest
import torch

import kat
import oracle

pytestmark = pytest.mark.gpu

k = pytest.importorskip("krea2_hrx_b200")


@pytest.fixture(scope="module")
def ops():
    from krea2_hrx_b200 import ops as module
    return module


@pytest.fixture(autouse=True)
def healthy_device():
    yield
    assert k.device_status() == 0, "a kernel reported a bounded wait that ran out"


def dev(a: np.ndarray, dtype=None) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.view(dtype)
    return t.cuda()


def host(t: torch.Tensor, dtype) -> np.ndarray:
    torch.cuda.synchronize()
    if t.dtype in (torch.float16, torch.bfloat16):
        t = t.view(torch.int16)
    return t.cpu().numpy().view(dtype)


def q_buffer(tokens, stride, fill=0xA5):
    return torch.full((tokens, stride), fill, dtype=torch.uint8, device="cuda").view(torch.int8)


# ------------------------------------------------------------------ prologues
def run_prologue(ops, kind, case_inputs, tokens, width, stride, gate_stride=None):
    q = q_buffer(tokens, stride)
    qs = torch.zeros(tokens, dtype=torch.float32, device="cuda")
    if kind == "norm":
        h, ns, ms, sh = case_inputs
        ops.prepare_norm_i8(dev(h, torch.bfloat16), dev(ns), dev(ms), dev(sh), q, qs, width, stride, 1e-5)
    elif kind == "gated":
        attn, gate = case_inputs
        ops.prepare_gated_i8(dev(attn, torch.float16), dev(gate, torch.float16), q, qs, width, stride, gate_stride)
    else:
        (h,) = case_inputs
        ops.prepare_plain_i8(dev(h, torch.float16), q, qs, width, stride)
    return host(q, np.int8), host(qs, np.float32)


def oracle_prologue(kind, case_inputs, width, stride, gate_stride=None):
    if kind == "norm":
        return oracle.prepare_norm_i8(*case_inputs, width, stride, 1e-5, fill=0xA5)
    if kind == "gated":
        return oracle.prepare_gated_i8(*case_inputs, width, stride, gate_stride, fill=0xA5)
    return oracle.prepare_plain_i8(*case_inputs, width, stride, fill=0xA5)


@pytest.mark.parametrize("kind", ["norm", "gated", "plain"])
def test_quantized_preparation_matches_the_kronecker_hadamard_and_preserves_padding(ops, kind):
    """tests/quantized.rs:385-512, then bit-exactness against the oracle."""
    case = kat.preparation_case()
    inputs = {"norm": (case["norm_input"], case["norm"], case["modulation"], case["shift"]),
              "gated": (case["half_input"], case["gate"]), "plain": (case["half_input"],)}[kind]
    q, qs = run_prologue(ops, kind, inputs, case["tokens"], case["width"], case["stride"], case["gate_stride"])
    kat.check_preparation(kind, case, q, qs)
    want_q, want_s = oracle_prologue(kind, inputs, case["width"], case["stride"], case["gate_stride"])
    np.testing.assert_array_equal(qs.view(np.uint32), want_s.view(np.uint32))
    np.testing.assert_array_equal(q, want_q)


@pytest.mark.parametrize("width", [2048, 6144, 16384])
def test_plain_preparation_preserves_each_half_rounding_boundary(ops, width):
    """tests/quantized.rs:514-569: bit-exact scale bytes and codes, padding untouched."""
    inp, stride = kat.plain_boundary_case(width)
    q, qs = run_prologue(ops, "plain", (inp,), 3, width, stride)
    codes, scales = kat.plain_boundary_expected(inp)
    np.testing.assert_array_equal(qs.view(np.uint32), scales.view(np.uint32))
    np.testing.assert_array_equal(q[:, :width], codes)
    assert np.all(q[:, width:].view(np.uint8) == 0xA5)


def random_rows(rng, tokens, width, outliers=True):
    x = rng.standard_normal((tokens, width)).astype(np.float32)
    if outliers:
        x[:, rng.choice(width, size=max(1, width // 100), replace=False)] *= 20.0
    return x


@pytest.mark.parametrize("width", [2048, 4096, 6144, 8192, 10240, 16384, 32768])
@pytest.mark.parametrize("kind", ["norm", "gated", "plain"])
def test_prologues_are_bit_exact_on_seeded_activations(ops, kind, width):
    """Every supported width class: N(0,1) rows with 1 % of channels x20, a zero row, a tiny row
    and a huge row; ragged pitches."""
    rng = np.random.default_rng(width + len(kind))
    tokens = 37
    stride = width + 64 * (1 + width // 4096 % 3)
    x = random_rows(rng, tokens, width)
    x[3] = 0.0
    x[5] *= 1e-6
    x[7] *= 300.0
    gate_stride = None
    if kind == "norm":
        inputs = (kat.bf16_bits_from_f32(x), (rng.standard_normal(width) * 0.1).astype(np.float32),
                  (rng.standard_normal(width) * 0.5).astype(np.float32),
                  (rng.standard_normal(width) * 0.5).astype(np.float32))
    elif kind == "gated":
        gate_stride = width + 256
        gate = np.zeros((tokens, gate_stride), dtype=np.uint16)
        g = rng.standard_normal((tokens, width)).astype(np.float32) * 2.0
        g[9] *= 20.0
        gate[:, :width] = kat.f16_bits(g)
        with np.errstate(over="ignore"):
            inputs = (kat.f16_bits(x), gate)
    else:
        with np.errstate(over="ignore"):
            inputs = (kat.f16_bits(np.clip(x, -60000, 60000)),)
    q, qs = run_prologue(ops, kind, inputs, tokens, width, stride, gate_stride)
    want_q, want_s = oracle_prologue(kind, inputs, width, stride, gate_stride)
    np.testing.assert_array_equal(qs.view(np.uint32), want_s.view(np.uint32))
    np.testing.assert_array_equal(q, want_q)  # includes the untouched 0xA5 padding


@pytest.mark.parametrize("kind,tokens,width", [("norm", 4608, 6144), ("gated", 4608, 6144), ("plain", 4608, 16384),
                                               ("norm", 1043, 6144), ("gated", 1043, 4096), ("plain", 1043, 6144),
                                               ("norm", 2311, 2048), ("plain", 16397, 2048)])
def test_prologues_are_bit_exact_over_many_rows_per_worker(ops, kind, tokens, width):
    """The benchmark's shapes and ragged row counts: every persistent block takes several rows per worker,
    through the prefetch buffers of both parities and an uneven split of rows over blocks."""
    rng = np.random.default_rng(tokens + width)
    stride = width + (64 if width % 8192 == 0 else 0)
    x = random_rows(rng, tokens, width)
    x[tokens // 2] = 0.0
    gate_stride = None
    if kind == "norm":
        inputs = (kat.bf16_bits_from_f32(x), (rng.standard_normal(width) * 0.1).astype(np.float32),
                  (rng.standard_normal(width) * 0.5).astype(np.float32),
                  (rng.standard_normal(width) * 0.5).astype(np.float32))
    elif kind == "gated":
        gate_stride = width + 2 * 1536 + width  # the q|k|v|gate row of a fused buffer
        gate = np.zeros((tokens, gate_stride), dtype=np.uint16)
        gate[:, :width] = kat.f16_bits(rng.standard_normal((tokens, width)).astype(np.float32) * 2.0)
        inputs = (kat.f16_bits(x), gate)
    else:
        inputs = (kat.f16_bits(x),)
    q, qs = run_prologue(ops, kind, inputs, tokens, width, stride, gate_stride)
    want_q, want_s = oracle_prologue(kind, inputs, width, stride, gate_stride)
    np.testing.assert_array_equal(qs.view(np.uint32), want_s.view(np.uint32))
    np.testing.assert_array_equal(q, want_q)


def test_gated_prologue_reads_the_gate_through_a_column_view(ops):
    """The session binds the gate as columns GATE_OFFSET.. of the fused buffer
    (src/session/mod.rs:141-144): pitch 15360, view starting 9216 columns in."""
    rng = np.random.default_rng(5)
    tokens, width, qkvg, offset = 19, 6144, 15360, 9216
    attn = kat.f16_bits(rng.standard_normal((tokens, width)).astype(np.float32))
    fused = kat.f16_bits(rng.standard_normal((tokens, qkvg)).astype(np.float32))
    fused_dev = dev(fused, torch.float16)
    q = q_buffer(tokens, width)
    qs = torch.zeros(tokens, dtype=torch.float32, device="cuda")
    ops.prepare_gated_i8(dev(attn, torch.float16), fused_dev.view(-1)[offset:], q, qs, width, width, qkvg,
                         tokens=tokens)
    view = np.zeros((tokens, qkvg), dtype=np.uint16)
    view.reshape(-1)[:tokens * qkvg - offset] = fused.reshape(-1)[offset:]
    want_q, want_s = oracle.prepare_gated_i8(attn, view, width, width, qkvg, fill=0xA5)
    np.testing.assert_array_equal(host(qs, np.float32).view(np.uint32), want_s.view(np.uint32))
    np.testing.assert_array_equal(host(q, np.int8), want_q)


def test_transport_round_trips(ops):
    rng = np.random.default_rng(3)
    x = (rng.standard_normal(100003) * 10.0 ** rng.integers(-6, 5, 100003)).astype(np.float32)
    bits = kat.bf16_bits_from_f32(x)
    src = dev(bits, torch.bfloat16)
    mid = torch.empty(bits.shape, dtype=torch.float16, device="cuda")
    ops.lora_transport(src, mid, 1)
    np.testing.assert_array_equal(host(mid, np.uint16), oracle.transport_bf16_to_f16(bits))
    back = torch.empty(bits.shape, dtype=torch.bfloat16, device="cuda")
    ops.lora_transport(mid, back, 2)
    np.testing.assert_array_equal(host(back, np.uint16), oracle.transport_f16_to_bf16(host(mid, np.uint16)))


# ------------------------------------------------------------------ GEMMs
def run_gemm(ops, mode, wide, m, k_size, stride, n, a, w, ws, a_scale, residual=None, gate=None):
    a_d, w_d, ws_d, as_d = dev(a), dev(w), dev(ws), dev(a_scale)
    if mode == "plain":
        c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
        ops.gemm_i8_256(m, a_d, w_d, ws_d, as_d, c, k_size, stride, n)
    elif mode == "swiglu":
        c = torch.zeros((m, n // 2), dtype=torch.float16, device="cuda")
        ops.gemm_i8_swiglu_256(m, a_d, w_d, ws_d, as_d, c, k_size, stride, n)
    else:
        c = dev(residual, torch.bfloat16).clone()
        if wide is None:
            ops.gemm_i8_resid_256(m, a_d, w_d, ws_d, as_d, c, dev(gate), k_size, stride, n)
        else:
            ops.gemm_i8_resid_256x256(m, a_d, w_d, ws_d, as_d, c, dev(gate), k_size, stride, n, 4, int(wide))
    return host(c, np.uint16)


def run_acc(ops, m, k_size, stride, n, a, w):
    acc = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    ops.gemm_i8_acc(m, dev(a), dev(w), acc, k_size, stride, n)
    return host(acc, np.int32)


def oracle_gemm(mode, acc, ws, a_scale, residual=None, gate=None):
    if mode == "plain":
        return oracle.epilogue_plain(acc, ws, a_scale)
    if mode == "swiglu":
        return oracle.epilogue_swiglu(acc, ws, a_scale)
    return oracle.epilogue_resid(acc, ws, a_scale, residual, gate)


@pytest.mark.parametrize("mode,wide", kat.GEMM_MODES)
@pytest.mark.parametrize("m,kk,n,pad", kat.GEMM_SHAPES)
def test_integer_gemms_preserve_pitches_bf16_residuals_and_swiglu_order(ops, mode, wide, m, kk, n, pad):
    """tests/quantized.rs:171-280 (tolerance 2e-3 + 4e-3 rel, bf16-representable outputs), then
    bit-exactness of the accumulators and of the outputs against the oracle."""
    if wide is not None:
        n *= 2
    case = kat.gemm_case(m, kk, n, pad)
    acc = run_acc(ops, m, kk, case["stride"], n, case["a"], case["w"])
    np.testing.assert_array_equal(acc.astype(np.int64), case["dot"])
    out = run_gemm(ops, mode, wide, m, kk, case["stride"], n, case["a"], case["w"], case["ws"], case["scales"],
                   case["residual"], case["gates"])
    values = (kat.bf16_to_f32(out) if mode == "resid" else kat.f16_from_bits(out)).astype(np.float64)
    assert np.all(kat.bf16_round_f64(values) == values), "outputs must be bf16-representable"
    kat.close(values, kat.gemm_expected(mode, case), 2e-3, 4e-3)
    want = oracle_gemm(mode, acc, case["ws"], case["scales"], case["residual"], case["gates"])
    np.testing.assert_array_equal(out, want)


RANDOM_GEMMS = [
    # m, k_size, k_stride, n
    (1, 128, 128, 128),
    (128, 256, 320, 256),
    (129, 640, 640, 384),
    (300, 1024, 1088, 512),
    (257, 6144, 6144, 256),
    (33, 16384, 16448, 256),
    (1043, 3072, 3072, 768),
    (515, 192, 256, 512),
    (300, 256, 320, 32768),  # three 128-row halves: the launcher takes 128-row tiles here (3 rounds instead of 4)
]


@pytest.mark.parametrize("m,kk,stride,n", RANDOM_GEMMS)
def test_gemms_are_bit_exact_on_seeded_operands(ops, m, kk, stride, n):
    """Full-range int8 operands, ragged rows, padded pitches whose padding holds garbage."""
    rng = np.random.default_rng(m * 7 + n)
    a = rng.integers(-127, 128, size=(m, stride), dtype=np.int64).astype(np.int8)
    w = rng.integers(-127, 128, size=(n, stride), dtype=np.int64).astype(np.int8)
    ws = rng.uniform(1e-3, 1e-2, size=n).astype(np.float32)
    a_scale = (np.abs(rng.standard_normal(m)) * 0.05 + 1e-3).astype(np.float32)
    gate = (rng.standard_normal(n) * 0.5).astype(np.float32)
    residual = kat.bf16_bits_from_f32(rng.standard_normal((m, n)).astype(np.float32))
    want_acc = oracle.gemm_i8_acc(a, w, kk, stride, n)
    if kk % 128 == 0:
        acc = run_acc(ops, m, kk, stride, n, a, w)
        np.testing.assert_array_equal(acc, want_acc)
        for mode in ("plain", "swiglu", "resid"):
            out = run_gemm(ops, mode, None, m, kk, stride, n, a, w, ws, a_scale, residual, gate)
            np.testing.assert_array_equal(out, oracle_gemm(mode, want_acc, ws, a_scale, residual, gate), err_msg=mode)
    if n % 256 == 0:
        out = run_gemm(ops, "resid", True, m, kk, stride, n, a, w, ws, a_scale, residual, gate)
        np.testing.assert_array_equal(out, oracle_gemm("resid", want_acc, ws, a_scale, residual, gate))


def test_gemm_repeated_dispatch_is_deterministic(ops):
    """The reference's race check (tests/softmax_repeat.rs): the same resident dispatch, repeated,
    must give the same bytes every time."""
    rng = np.random.default_rng(99)
    m, kk, n = 700, 2048, 1024
    a = rng.integers(-127, 128, size=(m, kk)).astype(np.int8)
    w = rng.integers(-127, 128, size=(n, kk)).astype(np.int8)
    a_d, w_d = dev(a), dev(w)
    first = None
    for _ in range(10):
        acc = torch.zeros((m, n), dtype=torch.int32, device="cuda")
        ops.gemm_i8_acc(m, a_d, w_d, acc, kk, kk, n)
        got = host(acc, np.int32)
        if first is None:
            first = got
            np.testing.assert_array_equal(first, oracle.gemm_i8_acc(a, w, kk, kk, n))
        else:
            np.testing.assert_array_equal(got, first)


FULL_SIZE = [
    # name, m, k, n, mode: the projections of one 1024x1024 image at the reference's dimensions
    ("qkvg", 4608, 6144, 15360, "plain"),
    ("wo", 4608, 6144, 6144, "resid"),
    ("gate_up", 4608, 6144, 32768, "swiglu"),
    ("down", 4608, 16384, 6144, "wide"),
    ("qkv_3072", 4608, 3072, 9216, "plain"),
    ("ragged", 4115, 6144, 6144, "resid"),
    # row counts with an odd number of 128-row halves, where 128-row tiles save a round over the SMs
    ("quarter_share_qkvg", 1152, 6144, 15360, "plain"),
    ("bench_list_1043_gate_up", 1043, 6144, 32768, "swiglu"),
]


@pytest.mark.parametrize("name,m,kk,n,mode", FULL_SIZE)
def test_full_size_gemms_checksum_and_sampled_rows(ops, name, m, kk, n, mode):
    """At benchmark sizes the oracle cannot recompute every element, so: (1) the sum of all i32
    accumulators must equal sum_k colsum(A)[k] * colsum(W)[k] (every tile contributed exactly
    once), and (2) sampled rows -- first, last, tile edges, random -- match the oracle bit for bit."""
    from krea2_hrx_b200 import shape
    stride = shape.gemm_pitch(kk)
    gen = torch.Generator(device="cuda").manual_seed(kk + n)
    a = torch.randint(-127, 128, (m, stride), generator=gen, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (n, stride), generator=gen, device="cuda", dtype=torch.int8)
    acc = torch.empty((m, n), dtype=torch.int32, device="cuda")
    ops.gemm_i8_acc(m, a, w, acc, kk, stride, n)
    total = acc.to(torch.int64).sum().item()
    col_a = a[:, :kk].to(torch.int64).sum(dim=0)
    col_w = w[:, :kk].to(torch.int64).sum(dim=0)
    assert total == (col_a * col_w).sum().item()
    rows_acc = acc.to(torch.int64).sum(dim=1)
    assert torch.equal(rows_acc, (a[:, :kk].to(torch.int64) * col_w[None, :]).sum(dim=1))
    rng = np.random.default_rng(n)
    rows = sorted(set([0, 1, 127, 128, 255, 256, m - 129, m - 2, m - 1] + rng.integers(0, m, 7).tolist()))
    a_rows = a[rows].cpu().numpy()
    w_host = w.cpu().numpy()
    want_acc = oracle.gemm_i8_acc(a_rows, w_host, kk, stride, n)
    np.testing.assert_array_equal(acc[rows].cpu().numpy(), want_acc)
    ws = torch.rand(n, generator=gen, device="cuda") * 9e-3 + 1e-3
    a_scale = torch.rand(m, generator=gen, device="cuda") * 0.05 + 1e-3
    gate = torch.randn(n, generator=gen, device="cuda") * 0.5
    residual = torch.randn((m, n), generator=gen, device="cuda").to(torch.bfloat16)
    ws_h, as_h, gate_h = ws.cpu().numpy(), a_scale.cpu().numpy(), gate.cpu().numpy()
    if mode == "plain":
        c = torch.empty((m, n), dtype=torch.float16, device="cuda")
        ops.gemm_i8_256(m, a, w, ws, a_scale, c, kk, stride, n)
        want = oracle.epilogue_plain(want_acc, ws_h, as_h[rows])
    elif mode == "swiglu":
        c = torch.empty((m, n // 2), dtype=torch.float16, device="cuda")
        ops.gemm_i8_swiglu_256(m, a, w, ws, a_scale, c, kk, stride, n)
        want = oracle.epilogue_swiglu(want_acc, ws_h, as_h[rows])
    else:
        c = residual.clone()
        if mode == "wide":
            ops.gemm_i8_resid_256x256(m, a, w, ws, a_scale, c, gate, kk, stride, n, 4, 1)
        else:
            ops.gemm_i8_resid_256(m, a, w, ws, a_scale, c, gate, kk, stride, n)
        want = oracle.epilogue_resid(want_acc, ws_h, as_h[rows], host(residual[rows].contiguous(), np.uint16), gate_h)
    np.testing.assert_array_equal(host(c[rows].contiguous(), np.uint16), want)


# ------------------------------------------------------------------ second caller
@pytest.mark.parametrize("inputs", [6144, 16384])
def test_convrot_path_matches_integer_cpu_algebra(ops, inputs):
    """src/training/quantized.rs:124-225 (base term), through Ops.launch: bit-exact bf16."""
    weights, scales, x_bf16 = kat.convrot_case(inputs)
    layer = ops.Quantized(torch.from_numpy(weights), torch.from_numpy(scales), weights.shape[0], inputs)
    x = dev(x_bf16, torch.bfloat16)
    out = layer.forward(ops.Ops(), torch.cuda.current_stream(), x)
    np.testing.assert_array_equal(host(out, np.uint16), kat.convrot_expected(weights, scales, x_bf16))


def test_config0_linear_tracks_the_reference_torch_scheme(ops):
    """Golden vectors from scripts/quantized_reference.py (tolerance reference): relative L2 of the
    f16 output and max-abs are reported against the scheme's own output."""
    import os
    for name in ("small", "hidden"):
        g = np.load(os.path.join(os.path.dirname(__file__), "golden", f"quantlinear_{name}.npz"))
        x, w, ws = g["x"], g["w"], g["ws"]
        m, kk = x.shape
        n = w.shape[0]
        n_pad = -(-n // 128) * 128
        w_pad = np.zeros((n_pad, kk), dtype=np.int8)
        w_pad[:n] = w
        ws_pad = np.zeros(n_pad, dtype=np.float32)
        ws_pad[:n] = ws
        q = q_buffer(m, kk)
        qs = torch.zeros(m, dtype=torch.float32, device="cuda")
        ops.prepare_plain_i8(dev(x, torch.float16), q, qs, kk, kk)
        c = torch.zeros((m, n_pad), dtype=torch.float16, device="cuda")
        ops.gemm_i8_256(m, q, dev(w_pad), dev(ws_pad), qs, c, kk, kk, n_pad)
        out = kat.f16_from_bits(host(c, np.uint16))[:, :n].astype(np.float64)
        ref = kat.f16_from_bits(g["out"]).astype(np.float64)
        rel_l2 = np.linalg.norm(out - ref) / np.linalg.norm(ref)
        assert rel_l2 < 1e-2, (name, rel_l2)
        assert np.abs(out - ref).max() <= 2e-2 * np.abs(ref).max(), name


@pytest.mark.parametrize("k_size", [2048, 4096])
def test_config0_shape_class_through_prologue_and_gemm(ops, k_size):
    """The single W8A8 linear of the benchmark's first configuration -- 256 tokens, 3072 outputs, f16 activations
    ~N(0,1) with 1 % of the channels scaled by 20, int8 weights uniform in [-127,127], channel scales ~U(1e-3,1e-2)
    -- at the two legal reduction widths on either side of its K = 3072 (the reference's prologues take widths
    that are multiples of 2048, kernels/prepare_plain_i8.loom:10-13): prepare_plain_i8 then gemm_i8_256, every
    code, scale, accumulator and output bit against the oracle."""
    m, n = 256, 3072
    rng = np.random.default_rng(k_size)
    x = rng.standard_normal((m, k_size)).astype(np.float32)
    x[:, rng.choice(k_size, size=k_size // 100, replace=False)] *= 20.0
    x16 = kat.f16_bits(x)
    w = rng.integers(-127, 128, size=(n, k_size), dtype=np.int16).astype(np.int8)
    ws = rng.uniform(1e-3, 1e-2, size=n).astype(np.float32)
    q = q_buffer(m, k_size)
    qs = torch.zeros(m, dtype=torch.float32, device="cuda")
    ops.prepare_plain_i8(dev(x16, torch.float16), q, qs, k_size, k_size)
    want_q, want_s = oracle.prepare_plain_i8(x16, k_size, k_size, fill=0xA5)
    np.testing.assert_array_equal(host(q, np.int8), want_q)
    np.testing.assert_array_equal(host(qs, np.uint32), want_s.view(np.uint32))
    acc = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    ops.gemm_i8_acc(m, q, dev(w), acc, k_size, k_size, n)
    want_acc = oracle.gemm_i8_acc(want_q, w, k_size, k_size, n)
    np.testing.assert_array_equal(host(acc, np.int32), want_acc)
    c = torch.zeros((m, n), dtype=torch.float16, device="cuda")
    ops.gemm_i8_256(m, q, dev(w), dev(ws), qs, c, k_size, k_size, n)
    np.testing.assert_array_equal(host(c, np.uint16), oracle.epilogue_plain(want_acc, ws, want_s))
    # against the real-valued product of the rotated activations (the weights are stored rotated) the error
    # stays at the level of 127-level activation quantisation
    h4 = np.array([[1, 1, 1, -1], [1, 1, -1, 1], [1, -1, 1, 1], [-1, 1, 1, 1]], dtype=np.float64)
    h256 = np.kron(np.kron(h4, h4), np.kron(h4, h4)) / 16.0
    rotated = (kat.f16_from_bits(x16).astype(np.float64).reshape(m, k_size // 256, 256) @ h256.T).reshape(m, k_size)
    exact = rotated @ (w.astype(np.float64) * ws[:, None].astype(np.float64)).T
    got = kat.f16_from_bits(host(c, np.uint16)).astype(np.float64)
    assert np.linalg.norm(got - exact) / np.linalg.norm(exact) < 2e-2


def test_unaligned_buffers_are_refused(ops):
    a = torch.zeros(128 * 128 + 16, dtype=torch.int8, device="cuda")
    w = torch.zeros((128, 128), dtype=torch.int8, device="cuda")
    s = torch.ones(128, dtype=torch.float32, device="cuda")
    c = torch.zeros((1, 128), dtype=torch.float16, device="cuda")
    with pytest.raises(k.InvalidArgument, match="16-byte aligned"):
        ops.gemm_i8_256(1, a[1:129], w, s, s, c, 128, 128, 128)


def test_single_cta_kernel_serves_the_same_shapes():
    """Shapes with whole 256-column tiles and more than 128 rows go to the two-CTA kernel; with
    KREA2_GEMM_PAIR=0 the same cases run on the single-CTA kernel and must give the same bits."""
    import os
    import subprocess
    import sys
    if os.environ.get("KREA2_GEMM_PAIR") == "0":
        pytest.skip("already the single-CTA run")
    env = dict(os.environ, KREA2_GEMM_PAIR="0")
    result = subprocess.run([sys.executable, "-m", "pytest", __file__, "-q", "-x", "-m", "gpu", "-k",
                             "seeded_operands or integer_gemms or full_size"], env=env, capture_output=True, text=True)
    assert result.returncode == 0, result.stdout[-2000:] + result.stderr[-2000:]


@pytest.mark.parametrize("inputs", [6144, 16384])
def test_fused_convrot_call_equals_the_launch_sequence(ops, inputs):
    """krea2_quantized_forward against the four Ops.launch calls and the reference's CPU algebra."""
    weights, scales, x_bf16 = kat.convrot_case(inputs)
    layer = ops.Quantized(torch.from_numpy(weights), torch.from_numpy(scales), weights.shape[0], inputs)
    x = dev(x_bf16, torch.bfloat16)
    stream = torch.cuda.current_stream()
    fused = layer.forward_fused(stream, x)
    np.testing.assert_array_equal(host(fused, np.uint16), kat.convrot_expected(weights, scales, x_bf16))
    np.testing.assert_array_equal(host(fused, np.uint16), host(layer.forward(ops.Ops(), stream, x), np.uint16))
    small = torch.empty(16, dtype=torch.uint8, device="cuda")
    with pytest.raises(k.InvalidArgument, match="workspace"):
        layer.forward_fused(stream, x, small)


def test_the_swiglu_kernel_equals_torchs_silu_product_bit_for_bit(ops):
    """The CUDA gate|up GEMM against tests/golden/swiglu_bf16.npz (`F.silu(g) * u` on bf16 tensors, the statement of
    `Krea2Ref.swiglu`, scripts/quantized_reference.py:222-225): int8 operands are built whose exact products are the
    fixture's accumulators, so the epilogue sees every bf16 gate value with an exponent from -8 to 6."""
    import os
    acc, scale, want, outputs = kat.swiglu_golden_accumulators(os.path.join(os.path.dirname(__file__), "golden", "swiglu_bf16.npz"))
    k_size, got = 512, []
    cut = acc.shape[1] // 512 * 256  # two launches of whole 256-column tiles, each within the 32768-column limit
    for part in (slice(0, cut), slice(cut, acc.shape[1])):
        columns = part.stop - part.start
        assert columns % 256 == 0 and columns <= 32768
        a, w = kat.weights_for_accumulators(acc[0, part], k_size)
        c = torch.zeros((1, columns // 2), dtype=torch.float16, device="cuda")
        ops.gemm_i8_swiglu_256(1, dev(a), dev(w), dev(scale[part]), dev(np.ones(1, np.float32)), c, k_size, k_size, columns)
        torch.cuda.synchronize()
        got.append(c.cpu().numpy().astype(np.float32)[0])
    got = np.concatenate(got)[:outputs]
    normal = np.abs(want) >= 2.0 ** -14
    np.testing.assert_array_equal(got[normal], want[normal])
    assert np.abs(got - want)[~normal].max() <= 2.0 ** -25


@pytest.mark.parametrize("wide", [False, True])
def test_the_residual_kernels_equal_torchs_gated_update_bit_for_bit(ops, wide):
    """Both residual exports against tests/golden/resid_bf16.npz (`x + gate * a` on bf16 tensors, the residual update
    of `Krea2Ref.block`, scripts/quantized_reference.py:262-268), through int8 operands whose exact products are the
    fixture's accumulators."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "resid_bf16.npz"))
    n, k_size = g["acc"].size, 1024
    a, w = kat.weights_for_accumulators(g["acc"], k_size)
    c = dev(g["x"][None, :].view(np.int16), torch.bfloat16)
    gate = dev(oracle.bf16_bits_to_f32(g["gate"]))
    scale, ones = dev(np.full(n, 2.0 ** -12, np.float32)), dev(np.ones(1, np.float32))
    if wide:
        ops.gemm_i8_resid_256x256(1, dev(a), dev(w), scale, ones, c, gate, k_size, k_size, n, schedule_rows=0)
    else:
        ops.gemm_i8_resid_256(1, dev(a), dev(w), scale, ones, c, gate, k_size, k_size, n)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(c.view(torch.int16).cpu().numpy().view(np.uint16)[0], g["out"])
