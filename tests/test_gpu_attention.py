"""QK-norm + RoPE, the V transpose and grouped-query attention (the launches between the
q|k|v|gate GEMM and the gated prologue).  RoPE and the transpose are compared bit for bit with the
oracle and with the reference's own test recipe (tests/quantized.rs:87-169); attention, whose
reference kernel uses approximate exponentials and free re-association, is held to the reference
test's tolerance against a float64 softmax (tests/quantized.rs:309-383: 2e-2 + 2e-2 * |x|)."""
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
    assert k.device_status() == 0


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.view(dtype) if dtype is not None else t).cuda()


def bits(t):
    torch.cuda.synchronize()
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def run_rope(ops, inp, qs, ks, cos, sin, stride, qh, kvh):
    tokens = inp.shape[0]
    q = torch.zeros((tokens, qh * 128), dtype=torch.float16, device="cuda")
    kk = torch.zeros((tokens, kvh * 128), dtype=torch.float16, device="cuda")
    v = torch.zeros((tokens, kvh * 128), dtype=torch.float16, device="cuda")
    ops.rope_qknorm_f16(dev(inp, torch.float16), dev(qs), dev(ks), dev(cos), dev(sin), q, kk, v, stride, qh, kvh, qh * 128,
                        1e-5)
    return bits(q), bits(kk), bits(v)


@pytest.mark.parametrize("tokens,qh,kvh,stride", [(3, 9, 2, 1664), (3, 48, 12, 15360)])
def test_rotary_rounds_normalized_and_rotated_values_to_bf16(ops, tokens, qh, kvh, stride):
    """tests/quantized.rs:87-169."""
    dim = 128
    inp = kat.f16_bits(kat.bf16_round_f32(kat.values(tokens * stride, 0.7))).reshape(tokens, stride)
    qs, ks = kat.values(dim, 0.3), kat.values(dim, -0.2)
    i = np.arange(tokens * dim)
    cos = np.cos((i // 2).astype(np.float32) * np.float32(0.03)).astype(np.float32)
    sin = np.sin((i // 2).astype(np.float32) * np.float32(0.03)).astype(np.float32)
    q, kk, v = run_rope(ops, inp, qs, ks, cos, sin, stride, qh, kvh)
    x = kat.f16_from_bits(inp).astype(np.float64)
    for out, heads, off, scale in [(q, qh, 0, qs), (kk, kvh, qh * dim, ks)]:
        act = kat.f16_from_bits(out).astype(np.float64).reshape(tokens, heads, dim)
        rows = x[:, off:off + heads * dim].reshape(tokens, heads, dim)
        rms = np.sqrt((rows ** 2).sum(-1, keepdims=True) / dim + 1e-5)
        norm = kat.bf16_round_f64(rows / rms * (1 + scale.astype(np.float64)))
        partner = np.empty_like(norm)
        partner[..., 0::2], partner[..., 1::2] = -norm[..., 1::2], norm[..., 0::2]
        c, s = cos.reshape(tokens, 1, dim), sin.reshape(tokens, 1, dim)
        want = kat.bf16_round_f32((norm.astype(np.float32) * c + partner.astype(np.float32) * s).astype(np.float32))
        assert np.all(kat.bf16_round_f64(act) == act)
        kat.close(act, want.astype(np.float64), 1e-3, 4e-3)
    np.testing.assert_array_equal(v, inp[:, (qh + kvh) * dim:(qh + 2 * kvh) * dim])
    oq, ok, ov = oracle.rope_qknorm_f16(inp, qs, ks, cos, sin, stride, qh, kvh, qh * dim)
    np.testing.assert_array_equal(q, oq)
    np.testing.assert_array_equal(kk, ok)
    np.testing.assert_array_equal(v, ov)


def test_rotary_is_bit_exact_on_seeded_rows(ops):
    rng = np.random.default_rng(8)
    tokens, qh, kvh, stride = 77, 48, 12, 15360
    inp = kat.f16_bits(kat.bf16_round_f32((rng.standard_normal((tokens, stride)) * 3).astype(np.float32)))
    qs, ks = (rng.standard_normal(128) * 0.2).astype(np.float32), (rng.standard_normal(128) * 0.2).astype(np.float32)
    ang = rng.uniform(0, 6.28, (tokens, 128)).astype(np.float32)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    got = run_rope(ops, inp, qs, ks, cos, sin, stride, qh, kvh)
    want = oracle.rope_qknorm_f16(inp, qs, ks, cos, sin, stride, qh, kvh, qh * 128)
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)


@pytest.mark.parametrize("rows,width,capacity", [(3, 128, 64), (97, 256, 160), (1043, 1536, 1088)])
def test_v_transpose_matches_and_leaves_the_headroom(ops, rows, width, capacity):
    rng = np.random.default_rng(rows)
    x = rng.integers(0, 65536, size=(rows, width)).astype(np.uint16)
    out = torch.full((width, capacity), 0x1234, dtype=torch.int16, device="cuda").view(torch.float16)
    ops.v_transpose(dev(x, torch.float16), out, width, capacity)
    want = oracle.v_transpose(x, width, capacity, out=np.full((width, capacity), 0x1234, dtype=np.uint16))
    np.testing.assert_array_equal(bits(out), want)


def run_attention(ops, q, kk, v, tokens, qh, kvh, capacity, scale, q32=False):
    vt = np.zeros((kvh * 128, capacity), dtype=np.uint16)
    vt[:, :tokens] = v[:tokens].T
    out = torch.zeros((tokens, qh * 128), dtype=torch.float16, device="cuda")
    ops.attention_gqa(tokens, kvh, dev(q, torch.float16), dev(kk, torch.float16), dev(vt, torch.float16), out, qh * 128,
                      kvh * 128, qh * 128, capacity, scale, q32=q32)
    return bits(out)


@pytest.mark.parametrize("tokens", [16, 17, 31, 32, 33, 63, 64, 65, 97])
def test_production_attention_tiles_match_grouped_cpu_softmax(ops, tokens):
    """tests/quantized.rs:309-383."""
    heads, kv, d = 4, 1, 128
    capacity = -(-(tokens + 79) // 64) * 64
    q = kat.f16_bits(kat.values(capacity * heads * d, 0.5)).reshape(capacity, heads * d)
    kk = kat.f16_bits(kat.values(capacity * kv * d, 0.3)).reshape(capacity, kv * d)
    v = kat.f16_bits(kat.values(capacity * kv * d, 0.7)).reshape(capacity, kv * d)
    q[tokens:], kk[tokens:], v[tokens:] = 0, 0, 0
    scale = 1.0 / np.sqrt(d)
    want = oracle.attention_gqa(q[:tokens], kk[:tokens], v[:tokens], heads, kv, scale)
    out = run_attention(ops, q[:tokens], kk[:tokens], v, tokens, heads, kv, capacity, scale)
    kat.close(kat.f16_from_bits(out).astype(np.float64), want, 2e-2, 2e-2)
    again = run_attention(ops, q[:tokens], kk[:tokens], v, tokens, heads, kv, capacity, scale, q32=True)
    np.testing.assert_array_equal(again, out)


@pytest.mark.parametrize("tokens,qh,kvh", [(300, 8, 2), (1043, 8, 2), (129, 4, 4), (127, 4, 2), (128, 4, 2), (255, 4, 2),
                                           (256, 4, 2), (257, 4, 2), (384, 2, 1), (385, 2, 1), (511, 2, 2), (640, 2, 1)])
def test_attention_on_seeded_heads(ops, tokens, qh, kvh):
    """Several key tiles, a ragged last tile, grouped heads; scores spread enough that the running
    maximum moves between tiles.  Token counts on both sides of the 128-key tile and of the 256 query rows a
    block owns: a second query tile that is empty, one row long, full."""
    from krea2_hrx_b200 import shape
    rng = np.random.default_rng(tokens)
    capacity = shape.capacity(tokens)
    q = kat.f16_bits((rng.standard_normal((tokens, qh * 128)) * 1.5).astype(np.float32))
    kk = kat.f16_bits((rng.standard_normal((tokens, kvh * 128)) * 1.5).astype(np.float32))
    kk_f = kat.f16_from_bits(kk).astype(np.float32)
    kk_f[tokens // 2:] *= 3.0  # later keys score higher: the maximum climbs
    kk = kat.f16_bits(kk_f)
    v = kat.f16_bits(rng.standard_normal((tokens, kvh * 128)).astype(np.float32))
    scale = 1.0 / np.sqrt(128)
    want = oracle.attention_gqa(q, kk, v, qh, kvh, scale)
    out = run_attention(ops, q, kk, v, tokens, qh, kvh, capacity, scale)
    kat.close(kat.f16_from_bits(out).astype(np.float64), want, 2e-2, 2e-2)


def test_attention_at_the_session_shape_on_sampled_rows(ops):
    """4608 tokens, 48 query heads over 12 key/value heads: sampled query rows against float64."""
    from krea2_hrx_b200 import shape
    tokens, qh, kvh = 4608, 48, 12
    capacity = shape.capacity(tokens)
    gen = torch.Generator(device="cuda").manual_seed(3)
    q = torch.randn((tokens, qh * 128), generator=gen, device="cuda").to(torch.float16)
    kk = torch.randn((tokens, kvh * 128), generator=gen, device="cuda").to(torch.float16)
    v = torch.randn((tokens, kvh * 128), generator=gen, device="cuda").to(torch.float16)
    vt = torch.zeros((kvh * 128, capacity), dtype=torch.float16, device="cuda")
    ops.v_transpose(v, vt, kvh * 128, capacity)
    out = torch.zeros((tokens, qh * 128), dtype=torch.float16, device="cuda")
    scale = 1.0 / np.sqrt(128)
    ops.attention_gqa(tokens, kvh, q, kk, vt, out, qh * 128, kvh * 128, qh * 128, capacity, scale)
    rows = [0, 127, 128, 2303, 4480, 4607]
    want = oracle.attention_gqa(bits(q[rows]), bits(kk), bits(v), qh, kvh, scale)
    kat.close(kat.f16_from_bits(bits(out[rows])).astype(np.float64), want, 2e-2, 2e-2)


@pytest.mark.parametrize("tokens", [8192, 8219, 16896])
def test_long_sequences_through_the_q32_export_on_sampled_rows(ops, tokens):
    """The reference switches to its 32-query-row kernel at 8192 tokens (src/kernels/shape.rs:20-31) and serves up
    to 16896 (:8).  The session shape, 48 query heads over 12 key/value heads, through the `_q32` export: sampled
    query rows (first, last, both sides of the 128-key tiles and of the 256 query rows a block owns) against
    float64, and the plain export must give the same bytes."""
    from krea2_hrx_b200 import shape
    assert shape.attention_rows(tokens) == 32
    qh, kvh = 48, 12
    capacity = shape.capacity(tokens)
    gen = torch.Generator(device="cuda").manual_seed(tokens)
    q = (torch.randn((tokens, qh * 128), generator=gen, device="cuda") * 1.2).to(torch.float16)
    kk = (torch.randn((tokens, kvh * 128), generator=gen, device="cuda") * 1.2).to(torch.float16)
    kk[tokens // 3:] *= 1.5  # later keys score higher: the running maximum moves
    v = torch.randn((tokens, kvh * 128), generator=gen, device="cuda").to(torch.float16)
    vt = torch.zeros((kvh * 128, capacity), dtype=torch.float16, device="cuda")
    ops.v_transpose(v, vt, kvh * 128, capacity)
    scale = 1.0 / np.sqrt(128)
    out = torch.zeros((tokens, qh * 128), dtype=torch.float16, device="cuda")
    ops.attention_gqa(tokens, kvh, q, kk, vt, out, qh * 128, kvh * 128, qh * 128, capacity, scale, q32=True)
    rows = [0, 255, 256, tokens // 2 - 1, 8191, tokens - 129, tokens - 1]
    want = oracle.attention_gqa(bits(q[rows]), bits(kk), bits(v), qh, kvh, scale)
    kat.close(kat.f16_from_bits(bits(out[rows])).astype(np.float64), want, 2e-2, 2e-2)
    plain = torch.zeros_like(out)
    ops.attention_gqa(tokens, kvh, q, kk, vt, plain, qh * 128, kvh * 128, qh * 128, capacity, scale)
    assert torch.equal(plain.view(torch.int16), out.view(torch.int16))


def test_attention_repeated_dispatch_is_deterministic(ops):
    """The reference's race check (tests/softmax_repeat.rs) for the attention kernel: the same launch, repeated
    while other work keeps the device busy, gives the same bytes every time.  The kernel orders its products
    and softmax passes through the tensor pipe's issue order; a slip there would show up as run-to-run noise."""
    from krea2_hrx_b200 import shape
    tokens, qh, kvh = 2311, 24, 6
    capacity = shape.capacity(tokens)
    gen = torch.Generator(device="cuda").manual_seed(11)
    q = (torch.randn((tokens, qh * 128), generator=gen, device="cuda") * 1.5).to(torch.float16)
    kk = (torch.randn((tokens, kvh * 128), generator=gen, device="cuda") * 1.5).to(torch.float16)
    v = torch.randn((tokens, kvh * 128), generator=gen, device="cuda").to(torch.float16)
    vt = torch.zeros((kvh * 128, capacity), dtype=torch.float16, device="cuda")
    ops.v_transpose(v, vt, kvh * 128, capacity)
    scale = 1.0 / np.sqrt(128)
    first = None
    busy = torch.empty(64 << 20, dtype=torch.uint8, device="cuda")
    for i in range(8):
        out = torch.zeros((tokens, qh * 128), dtype=torch.float16, device="cuda")
        if i % 2:
            busy.fill_(i)  # a different cache and memory state in front of every other launch
        ops.attention_gqa(tokens, kvh, q, kk, vt, out, qh * 128, kvh * 128, qh * 128, capacity, scale)
        got = bits(out)
        if first is None:
            first = got
            rows = [0, 255, 256, 1155, 2310]
            want = oracle.attention_gqa(bits(q[rows]), bits(kk), bits(v), qh, kvh, scale)
            kat.close(kat.f16_from_bits(got[rows]).astype(np.float64), want, 2e-2, 2e-2)
        else:
            np.testing.assert_array_equal(got, first)


def test_qk_norm_and_rope_equal_the_reference_torch_code_bit_for_bit(ops):
    """The CUDA kernel against tests/golden/rope_qknorm.npz (the reference's own `rms_norm` + `apply_rope` on its own
    rope tables, made by tests/golden/make_rope_golden.py): q and k are the reference's bf16 values exactly."""
    import os
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "rope_qknorm.npz"))
    fused = oracle.bf16_bits_to_f32(g["fused"])
    inp = fused.astype(np.float16).view(np.uint16)
    q, kk, v = run_rope(ops, inp, g["q_scale"], g["k_scale"], g["cos"], g["sin"], 1536, 8, 2)
    np.testing.assert_array_equal(q.view(np.float16).astype(np.float32), oracle.bf16_bits_to_f32(g["q"]))
    np.testing.assert_array_equal(kk.view(np.float16).astype(np.float32), oracle.bf16_bits_to_f32(g["k"]))
    np.testing.assert_array_equal(v.view(np.float16).astype(np.float32), fused[:, 10 * 128:])


def test_attention_tracks_torchs_scaled_dot_product_attention(ops):
    """The CUDA kernel against tests/golden/attention_sdpa.npz (`F.scaled_dot_product_attention` on bf16 tensors with
    repeated key/value heads, `Krea2Ref.attention`, scripts/quantized_reference.py:215-218): 208 tokens, two key tiles
    with the second ragged, eight query heads over two key/value heads.  The tolerance is the reference attention
    test's (tests/quantized.rs:309-383); torch's own bf16 output rounding is most of the difference."""
    import importlib.util
    import os
    from krea2_hrx_b200 import shape
    golden = os.path.join(os.path.dirname(__file__), "golden")
    spec = importlib.util.spec_from_file_location("make_attention_golden", os.path.join(golden, "make_attention_golden.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    q, k, v = module.inputs()
    want = oracle.bf16_bits_to_f32(np.load(os.path.join(golden, "attention_sdpa.npz"))["out"])
    tokens, qh, kvh = module.TOKENS, module.Q_HEADS, module.KV_HEADS
    capacity = shape.capacity(tokens)
    q_d, k_d, v_d = (torch.from_numpy(a.astype(np.float16)).cuda() for a in (q, k, v))
    vt = torch.zeros((kvh * 128, capacity), dtype=torch.float16, device="cuda")
    ops.v_transpose(v_d, vt, kvh * 128, capacity)
    out = torch.zeros((tokens, qh * 128), dtype=torch.float16, device="cuda")
    ops.attention_gqa(tokens, kvh, q_d, k_d, vt, out, qh * 128, kvh * 128, qh * 128, capacity, float(1.0 / np.sqrt(128.0)))
    torch.cuda.synchronize()
    got = out.cpu().numpy().astype(np.float32)
    err = np.abs(got - want)
    assert np.all(err <= 2e-2 + 2e-2 * np.abs(want))
    rel = float(np.sqrt((err ** 2).sum() / (want ** 2).sum()))
    print(f"CUDA attention vs torch SDPA (bf16), 208 tokens: relative RMS {rel:.5f}")
    assert rel < 0.004
