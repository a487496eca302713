"""The q|k|v|gate GEMM that also does the QK-norm + RoPE launch's work: krea2_gemm_i8_rope_256 must write exactly
what gemm_i8_256 followed by rope_qknorm_f16 writes (the reference's two launches, src/session/mod.rs:702-734):
q and k normalised and rotated, v copied, the gate columns in the fused buffer -- against the CPU oracle at small
sizes, GPU against GPU at the session's shape and at ragged row counts, and a session with the switch on and off."""
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


def case(m, k_size, q_heads, kv_heads, seed, gate_heads=None):
    gate_heads = q_heads if gate_heads is None else gate_heads
    n = (q_heads + 2 * kv_heads + gate_heads) * 128
    gen = torch.Generator(device="cuda").manual_seed(seed)
    pitch = shape.gemm_pitch(k_size)
    a = torch.randint(-127, 128, (m, pitch), generator=gen, device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (n, pitch), generator=gen, device="cuda", dtype=torch.int8)
    ws = torch.rand(n, generator=gen, device="cuda") * 4e-4 + 1e-5
    a_s = torch.rand(m, generator=gen, device="cuda") * 0.05 + 1e-3
    a_s[m // 3] = 0.0  # a token whose q and k rows are all zero: the norm's eps decides
    qn = torch.randn(128, generator=gen, device="cuda") * 0.2
    kn = torch.randn(128, generator=gen, device="cuda") * 0.2
    angle = torch.rand((m, 128), generator=gen, device="cuda") * 6.28
    return dict(m=m, k=k_size, n=n, pitch=pitch, qh=q_heads, kvh=kv_heads, a=a, w=w, ws=ws, a_s=a_s, qn=qn, kn=kn,
                cos=torch.cos(angle).contiguous(), sin=torch.sin(angle).contiguous())


def two_launches(c):
    m, n, qh, kvh = c["m"], c["n"], c["qh"], c["kvh"]
    fused = torch.full((m, n), 7.0, dtype=torch.float16, device="cuda")
    ops.gemm_i8_256(m, c["a"], c["w"], c["ws"], c["a_s"], fused, c["k"], c["pitch"], n)
    q = torch.zeros((m, qh * 128), dtype=torch.float16, device="cuda")
    kk = torch.zeros((m, kvh * 128), dtype=torch.float16, device="cuda")
    v = torch.zeros((m, kvh * 128), dtype=torch.float16, device="cuda")
    ops.rope_qknorm_f16(fused, c["qn"], c["kn"], c["cos"], c["sin"], q, kk, v, n, qh, kvh, qh * 128)
    torch.cuda.synchronize()
    return fused, q, kk, v


def one_launch(c):
    m, n, qh, kvh = c["m"], c["n"], c["qh"], c["kvh"]
    fused = torch.full((m, n), 7.0, dtype=torch.float16, device="cuda")  # the q, k, v columns must stay untouched
    q = torch.zeros((m, qh * 128), dtype=torch.float16, device="cuda")
    kk = torch.zeros((m, kvh * 128), dtype=torch.float16, device="cuda")
    v = torch.zeros((m, kvh * 128), dtype=torch.float16, device="cuda")
    ops.gemm_i8_rope_256(m, c["a"], c["w"], c["ws"], c["a_s"], fused, c["qn"], c["kn"], c["cos"], c["sin"], q, kk, v, c["k"],
                         c["pitch"], n, qh, kvh)
    torch.cuda.synchronize()
    return fused, q, kk, v


def same(a, b):
    return torch.equal(a.view(torch.int16), b.view(torch.int16))


@pytest.mark.parametrize("m,k_size,qh,kvh", [(17, 2048, 4, 1), (129, 2048, 4, 1), (300, 2048, 16, 2), (257, 6144, 6, 2)])
def test_fused_launch_equals_the_two_launches_and_the_oracle(m, k_size, qh, kvh):
    c = case(m, k_size, qh, kvh, seed=m + qh)
    fused2, q2, k2, v2 = two_launches(c)
    fused1, q1, k1, v1 = one_launch(c)
    assert same(q1, q2) and same(k1, k2) and same(v1, v2)
    gate0 = (qh + 2 * kvh) * 128
    assert same(fused1[:, gate0:], fused2[:, gate0:])
    assert bool((fused1[:, :gate0] == 7.0).all()), "only the gate columns of the fused buffer are written"
    want_fused = oracle.gemm_i8_256(c["a"].cpu().numpy(), c["w"].cpu().numpy(), c["ws"].cpu().numpy(), c["a_s"].cpu().numpy(),
                                    c["k"], c["pitch"], c["n"])
    wq, wk, wv = oracle.rope_qknorm_f16(want_fused, c["qn"].cpu().numpy(), c["kn"].cpu().numpy(), c["cos"].cpu().numpy(),
                                        c["sin"].cpu().numpy(), c["n"], qh, kvh, qh * 128)
    for got, want in ((q1, wq), (k1, wk), (v1, wv)):
        np.testing.assert_array_equal(got.view(torch.int16).cpu().numpy().view(np.uint16), want)


@pytest.mark.parametrize("m", [4608, 4115, 1043])
def test_fused_launch_at_the_session_shape(m):
    """K 6144, 48 query and 12 key/value heads, 48 gate heads (15360 columns): GPU against GPU, every byte."""
    c = case(m, 6144, 48, 12, seed=m)
    fused2, q2, k2, v2 = two_launches(c)
    fused1, q1, k1, v1 = one_launch(c)
    assert same(q1, q2) and same(k1, k2) and same(v1, v2)
    assert same(fused1[:, 9216:], fused2[:, 9216:])
    assert float(q1.float().abs().mean()) > 0.1, "the outputs are not trivially zero"


def test_bad_head_counts_are_refused():
    c = case(32, 2048, 4, 1, seed=1)
    fused, q, kk, v = two_launches(c)
    with pytest.raises(k.InvalidArgument, match="do not fit"):
        ops.gemm_i8_rope_256(32, c["a"], c["w"], c["ws"], c["a_s"], fused, c["qn"], c["kn"], c["cos"], c["sin"], q, kk, v,
                             c["k"], c["pitch"], c["n"], 20, 1)


@pytest.mark.parametrize("tokens", [80, 300])
def test_a_session_gives_the_same_bits_with_and_without_the_fused_launch(tokens):
    dims = session.ModelDims(**so.SMALL)
    layers = 2
    stream = torch.cuda.current_stream()
    weights = session.Weights(dims, layers)
    weights.fill_synthetic(29, stream)
    x, mods, cos, sin = so.make_inputs(dims, tokens, layers, seed=tokens)
    s = session.Session(stream, weights, tokens, layers)
    outs, launches = [], []
    for fused in (False, True, False):
        s.set_fused_rope(fused)
        assert s.set_fused_rope(fused) is fused
        launches.append(s.launches_per_forward())
        x_dev = torch.from_numpy(x.copy()).view(torch.bfloat16).cuda()
        s.run_device(stream, x_dev, torch.from_numpy(mods).cuda(), torch.from_numpy(cos), torch.from_numpy(sin))
        torch.cuda.synchronize()
        outs.append(x_dev.view(torch.int16).cpu())
    assert launches == [layers * 11, layers * 10, layers * 11]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    s.close()
