"""The fused hand-off from the gate|up GEMM to the down projection's prologue: gemm_i8_swiglu_rotated_256
followed by prepare_rotated_i8 must write exactly the codes and scales of gemm_i8_swiglu_256 followed by
prepare_plain_i8 (the reference's two launches, src/session/mod.rs:803-826) -- against the CPU oracle at sizes
it finishes quickly, GPU against GPU at the benchmark's size and at ragged row counts."""
import numpy as np
import pytest
import torch

import oracle
import session_oracle as so

pytestmark = pytest.mark.gpu

k = pytest.importorskip("krea2_hrx_b200")
from krea2_hrx_b200 import ops, session, shape  # noqa: E402


@pytest.fixture(autouse=True)
def healthy_device():
    yield
    assert k.device_status() == 0


def operands(m, k_size, n, seed, outliers=True):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    pitch = shape.gemm_pitch(k_size)
    a = torch.randint(-127, 128, (m, pitch), generator=gen, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (n, pitch), generator=gen, device="cuda", dtype=torch.int8)
    ws = torch.rand(n, generator=gen, device="cuda") * 4e-4 + 1e-5
    a_s = torch.rand(m, generator=gen, device="cuda") * 0.05 + 1e-3
    if outliers:
        a_s[m // 2] = 0.0       # a token whose row is all zero
        ws[5] = 0.0             # a dead channel
        a_s[0] *= 400.0         # a row whose outputs reach the top of the f16 range and beyond
    return a, w, ws, a_s, pitch


def both_ways(m, k_size, n, a, w, ws, a_s, pitch, fill=0xA5):
    inter = n // 2
    out_pitch = shape.gemm_pitch(inter)
    results = []
    for fused in (False, True):
        c = torch.zeros((m, inter), dtype=torch.float16, device="cuda")
        q = torch.full((m, out_pitch), fill, dtype=torch.uint8, device="cuda").view(torch.int8)
        qs = torch.zeros(m, dtype=torch.float32, device="cuda")
        if fused:
            ops.gemm_i8_swiglu_rotated_256(m, a, w, ws, a_s, c, k_size, pitch, n)
            ops.prepare_rotated_i8(c, q, qs, inter, out_pitch)
        else:
            ops.gemm_i8_swiglu_256(m, a, w, ws, a_s, c, k_size, pitch, n)
            ops.prepare_plain_i8(c, q, qs, inter, out_pitch)
        torch.cuda.synchronize()
        results.append((q, qs))
    return results


@pytest.mark.parametrize("m,k_size,n", [(17, 2048, 4096), (129, 2048, 4096), (257, 2048, 8192), (300, 6144, 4096), (64, 2048, 32768)])
def test_fused_pair_equals_the_two_launches_and_the_oracle(m, k_size, n):
    a, w, ws, a_s, pitch = operands(m, k_size, n, seed=m + n)
    (q0, s0), (q1, s1) = both_ways(m, k_size, n, a, w, ws, a_s, pitch)
    inter = n // 2
    gu = oracle.gemm_i8_swiglu_256(a.cpu().numpy(), w.cpu().numpy(), ws.cpu().numpy(), a_s.cpu().numpy(), k_size, pitch, n)
    want_q, want_s = oracle.prepare_plain_i8(gu, inter, shape.gemm_pitch(inter), fill=0xA5)
    for name, q, s in (("two launches", q0, s0), ("fused pair", q1, s1)):
        np.testing.assert_array_equal(s.cpu().numpy().view(np.uint32), want_s.view(np.uint32), err_msg=name)
        np.testing.assert_array_equal(q.cpu().numpy(), want_q, err_msg=name)  # padding bytes included


@pytest.mark.parametrize("m", [4608, 4115, 1043])
def test_fused_pair_at_the_benchmark_shape(m):
    """K 6144, gate|up 32768 -> 16384 outputs at pitch 16448: GPU against GPU, every byte."""
    k_size, n = 6144, 32768
    a, w, ws, a_s, pitch = operands(m, k_size, n, seed=m, outliers=True)
    (q0, s0), (q1, s1) = both_ways(m, k_size, n, a, w, ws, a_s, pitch)
    assert torch.equal(s0.view(torch.int32), s1.view(torch.int32))
    assert torch.equal(q0, q1)
    assert int((q0[:, :16384] != 0).sum()) > m * 16384 // 2, "the codes are not trivially zero"


def test_rotated_gemm_refuses_a_width_that_is_not_whole_256_column_tiles():
    a, w, ws, a_s, pitch = operands(32, 2048, 4096 + 128, seed=1, outliers=False)
    c = torch.zeros((32, 2048 + 64), dtype=torch.float16, device="cuda")
    with pytest.raises(k.InvalidArgument, match="256"):
        ops.gemm_i8_swiglu_rotated_256(32, a, w, ws, a_s, c, 2048, pitch, 4096 + 128)


@pytest.mark.parametrize("tokens,attention", [(80, False), (300, True)])
def test_a_session_gives_the_same_bits_with_and_without_the_fused_pair(tokens, attention):
    dims = session.ModelDims(**so.SMALL)
    layers = 2
    stream = torch.cuda.current_stream()
    weights = session.Weights(dims, layers)
    weights.fill_synthetic(23, stream)
    x, mods, cos, sin = so.make_inputs(dims, tokens, layers, seed=tokens)
    s = session.Session(stream, weights, tokens, layers)
    s.set_attention(attention)
    outs = []
    for fused in (False, True, False):
        s.set_fused_rotation(fused)
        assert s.set_fused_rotation(fused) is fused
        x_dev = torch.from_numpy(x.copy()).view(torch.bfloat16).cuda()
        s.run_device(stream, x_dev, torch.from_numpy(mods).cuda(), torch.from_numpy(cos), torch.from_numpy(sin))
        torch.cuda.synchronize()
        outs.append(x_dev.view(torch.int16).cpu())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    if not attention:
        want, _ = so.oracle_forward(dims, so.host_weights(weights, layers), x, mods)
        np.testing.assert_array_equal(outs[1].numpy().view(np.uint16), want)
    s.close()
