"""The column-sharded and the token-sharded chains.  On one GPU every rank's buffers live on the same device
and the ranks' launches are interleaved step by step (parallel.run_emulated, run_emulated_rows); on two or
more GPUs a torchrun child process per GPU runs the fused pushes and the NCCL baselines (tests/tp_worker.py).
Either way the residual stream must equal the single-device session's bit for bit."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

import session_oracle as so

pytestmark = pytest.mark.gpu

k = pytest.importorskip("krea2_hrx_b200")


def bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_sharded_chain_on_one_gpu_equals_the_session(world):
    from krea2_hrx_b200 import parallel, session
    # eight shares of whole 128-column tiles need four key/value heads: q|k|v|gate = 5120 columns
    dims = session.ModelDims(**(dict(so.SMALL, kv_heads=4) if world == 8 else so.SMALL))
    layers, tokens = 2, 300
    stream = torch.cuda.current_stream()
    weights = session.Weights(dims, layers)
    weights.fill_synthetic(11, stream)
    x, mods, cos, sin = so.make_inputs(dims, tokens, layers, seed=world)
    single = session.Session(stream, weights, tokens, layers)
    single.set_attention(False)  # the sharded chain is the W8A8 chain
    want = torch.from_numpy(x.copy()).view(torch.bfloat16)
    single.run(stream, want, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    fabric = parallel.LocalFabric(world)
    ranks = [parallel.TensorParallel(fabric, r, dims, parallel.shard_weights(weights, layers, world, r), tokens)
             for r in range(world)]
    x_dev = torch.from_numpy(x.copy()).view(torch.bfloat16).cuda()
    mods_dev = torch.from_numpy(mods).cuda()
    for _ in range(2):  # twice: flags and epochs carry over between forwards
        outs = parallel.run_emulated(ranks, x_dev, mods_dev)
        torch.cuda.synchronize()
        for out in outs:
            np.testing.assert_array_equal(bits(out), bits(want))
    assert ranks[0].launches == 2 * layers * 4
    assert k.device_status() == 0
    single.close()


@pytest.mark.parametrize("world,tokens", [(1, 80), (2, 300), (4, 300), (3, 131), (8, 300), (8, 1043)])
def test_token_sharded_blocks_on_one_gpu_equal_the_session(world, tokens):
    """Rows of the sequence spread over `world` ranks that all live on this GPU: the full block, attention on,
    must give every rank exactly its rows of the single-device session's output."""
    from krea2_hrx_b200 import parallel, session
    dims = session.ModelDims(**so.SMALL)
    layers = 3  # odd: the K/V buffers' parity restarts inside a forward and across forwards
    stream = torch.cuda.current_stream()
    weights = session.Weights(dims, layers)
    weights.fill_synthetic(17, stream)
    x, mods, cos, sin = so.make_inputs(dims, tokens, layers, seed=40 + world)
    single = session.Session(stream, weights, tokens, layers)
    want = torch.from_numpy(x.copy()).view(torch.bfloat16)
    single.run(stream, want, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    fabric = parallel.LocalFabric(world)
    ranks = [parallel.TokenParallel(fabric, r, weights, tokens, layers) for r in range(world)]
    x_dev = torch.from_numpy(x.copy()).view(torch.bfloat16).cuda()
    mods_dev = torch.from_numpy(mods).cuda()
    for _ in range(2):  # twice: flags, epochs and buffer parity carry over between forwards
        outs = parallel.run_emulated_rows(ranks, x_dev, mods_dev, torch.from_numpy(cos), torch.from_numpy(sin))
        torch.cuda.synchronize()
        for rank, out in zip(ranks, outs):
            first, count = rank.rows
            np.testing.assert_array_equal(bits(out), bits(want[first:first + count]))
    assert k.device_status() == 0
    single.close()


def test_attention_of_a_row_range_equals_those_rows_of_the_full_launch():
    from krea2_hrx_b200 import ops, shape
    tokens, qh, kvh = 700, 8, 2
    capacity = shape.capacity(tokens)
    gen = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn((tokens, qh * 128), generator=gen, device="cuda").to(torch.float16)
    kk = torch.randn((tokens, kvh * 128), generator=gen, device="cuda").to(torch.float16)
    v = torch.randn((tokens, kvh * 128), generator=gen, device="cuda").to(torch.float16)
    vt = torch.zeros((kvh * 128, capacity), dtype=torch.float16, device="cuda")
    ops.v_transpose(v, vt, kvh * 128, capacity)
    full = torch.zeros((tokens, qh * 128), dtype=torch.float16, device="cuda")
    ops.attention_gqa(tokens, kvh, q, kk, vt, full, qh * 128, kvh * 128, qh * 128, capacity, 0.0883883)
    for first, count in [(0, 1), (255, 257), (513, 187), (0, 700)]:
        part = torch.full((count, qh * 128), 9.0, dtype=torch.float16, device="cuda")
        ops.attention_gqa_rows(count, tokens, kvh, q[first:first + count].contiguous(), kk, vt, part, qh * 128, kvh * 128,
                               qh * 128, capacity, 0.0883883)
        torch.cuda.synchronize()
        assert torch.equal(part.view(torch.int16), full[first:first + count].view(torch.int16)), (first, count)
    with pytest.raises(k.InvalidArgument):
        ops.attention_gqa_rows(tokens + 1, tokens, kvh, q, kk, vt, full, qh * 128, kvh * 128, qh * 128, capacity, 0.0883883)


def test_a_share_of_the_rows_through_the_one_tile_form_equals_the_two_tile_launch():
    """The launcher takes one query tile per CTA when that saves rounds over the SMs and two otherwise; both forms
    must give the same bits.  2000 tokens of 48 heads fill the SMs for three rounds of two-tile CTAs (the full
    launch); a share of 1152 rows needs two such rounds or three half-length ones, so it goes through the other
    form."""
    from krea2_hrx_b200 import ops, shape
    tokens, qh, kvh = 2000, 48, 12
    capacity = shape.capacity(tokens)
    gen = torch.Generator(device="cuda").manual_seed(8)
    q = torch.randn((tokens, qh * 128), generator=gen, device="cuda").to(torch.float16)
    kk = torch.randn((tokens, kvh * 128), generator=gen, device="cuda").to(torch.float16)
    v = torch.randn((tokens, kvh * 128), generator=gen, device="cuda").to(torch.float16)
    vt = torch.zeros((kvh * 128, capacity), dtype=torch.float16, device="cuda")
    ops.v_transpose(v, vt, kvh * 128, capacity)
    full = torch.zeros((tokens, qh * 128), dtype=torch.float16, device="cuda")
    ops.attention_gqa(tokens, kvh, q, kk, vt, full, qh * 128, kvh * 128, qh * 128, capacity, 0.0883883)
    for first, count in [(300, 1152), (0, 1043), (1700, 300)]:
        part = torch.full((count, qh * 128), 9.0, dtype=torch.float16, device="cuda")
        ops.attention_gqa_rows(count, tokens, kvh, q[first:first + count].contiguous(), kk, vt, part, qh * 128, kvh * 128,
                               qh * 128, capacity, 0.0883883)
        torch.cuda.synchronize()
        assert torch.equal(part.view(torch.int16), full[first:first + count].view(torch.int16)), (first, count)
    assert k.device_status() == 0
    assert k.device_status() == 0


def test_sharded_gemm_refuses_bad_descriptions():
    from krea2_hrx_b200 import _lib
    import ctypes
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    desc = _lib.Shard()
    desc.world, desc.rank, desc.pitch, desc.offset = 2, 0, 256, 128
    desc.dest[0] = p
    desc.dest[1] = p

    def call(kind=0, n=128):
        return k.lib().krea2_gemm_i8_sharded(None, kind, 16, p, p, p, p, p, 128, 128, n, ctypes.byref(desc)), \
            k.lib().krea2_last_error().decode()
    status, message = call(n=256)
    assert status == 1 and "do not fit" in message
    desc.offset = 8
    status, message = call()
    assert status == 1 and "multiples of 16" in message
    desc.offset, desc.world = 0, 9
    status, message = call()
    assert status == 1 and "world" in message
    desc.world = 2
    desc.dest[1] = None
    status, message = call()
    assert status == 1 and "destination 1" in message
    status, message = call(kind=7)
    assert status == 1 and "unknown kind" in message


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_chain_on_two_gpus_fused_and_nccl():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    worker = os.path.join(os.path.dirname(__file__), "tp_worker.py")
    world = min(torch.cuda.device_count(), 4)
    world = 2 if world < 4 else 4
    try:
        result = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                                 "--master-addr", "127.0.0.1", "--master-port", str(port), worker, "--check"],
                                capture_output=True, text=True, timeout=240, env={**os.environ, "NCCL_NVLS_ENABLE": "0"})
    except subprocess.TimeoutExpired as late:
        def text(b):
            return (b.decode(errors="replace") if isinstance(b, bytes) else (b or ""))[-3000:]
        pytest.fail("the sharded worker did not finish: " + text(late.stdout) + text(late.stderr))
    assert result.returncode == 0, result.stdout[-3000:] + result.stderr[-3000:]
    assert "tp check ok" in result.stdout


def test_a_wait_for_a_peer_that_never_publishes_gives_up_and_reports_it():
    """Failure detection without a fault: slot 1 of the flag array is never written (a peer that died between
    steps), so the bounded wait runs out after its two seconds, raises the device status word and returns; the
    context stays usable and the next read of the status is clean."""
    import time
    from krea2_hrx_b200._lib import check, lib
    assert k.device_status() == 0
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    flags[0] = 1  # this rank's own slab has "landed"
    stream = torch.cuda.current_stream()
    began = time.time()
    check(lib().krea2_shard_wait(stream.cuda_stream, flags.data_ptr(), 2, 1, None))
    status = k.device_status()  # synchronises
    waited = time.time() - began
    assert status & 16, f"status word {status}: the wait did not report that it gave up"
    assert 1.5 < waited < 10.0, f"the wait took {waited:.1f} s against a limit of 2 s"
    assert k.device_status() == 0, "the status word is cleared by reading it"
    # the device still computes
    from krea2_hrx_b200 import ops
    a = torch.randint(-127, 128, (64, 128), device="cuda", dtype=torch.int8)
    w = torch.randint(-127, 128, (128, 128), device="cuda", dtype=torch.int8)
    acc = torch.zeros((64, 128), dtype=torch.int32, device="cuda")
    ops.gemm_i8_acc(64, a, w, acc, 128, 128, 128)
    torch.cuda.synchronize()
    want = a.cpu().to(torch.int64) @ w.cpu().to(torch.int64).t()
    assert torch.equal(acc.cpu().to(torch.int64), want)
    # once the peer's slot is set the same wait returns at once
    flags[1] = 1
    check(lib().krea2_shard_wait(stream.cuda_stream, flags.data_ptr(), 2, 1, None))
    assert k.device_status() == 0
