"""The resident session against the oracle chain, and the reference's session invariants
(src/session/mod.rs:843-1065): graph replay equals the eager run after inputs change, a foreign
stream is refused, a block range equals the chain of its parts."""
import numpy as np
import pytest
import torch

import oracle
import session_oracle as so

pytestmark = pytest.mark.gpu

k = pytest.importorskip("krea2_hrx_b200")


def bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.fixture(scope="module")
def small():
    from krea2_hrx_b200 import session
    dims = session.ModelDims(**so.SMALL)
    stream = torch.cuda.current_stream()
    weights = session.Weights(dims, 3)
    weights.fill_synthetic(7, stream)
    return dims, weights, so.host_weights(weights, 3)


@pytest.mark.parametrize("tokens", [16, 275, 1043])
def test_session_run_matches_the_oracle_chain(small, tokens):
    from krea2_hrx_b200 import session
    dims, weights, host = small
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, tokens, 3)
    assert s.set_attention(False) is True  # the W8A8 chain alone is what the oracle reproduces bit for bit
    assert (s.tokens(), s.layers()) == (tokens, 3)
    x, mods, cos, sin = so.make_inputs(dims, tokens, 3, seed=tokens)
    x_t = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, x_t, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    want, trace = so.oracle_forward(dims, host, x, mods)
    np.testing.assert_array_equal(bits(x_t), want)
    # the last block's quantised operand is still in the session's buffers
    ptr, n = s.buffer("a_s")
    assert n >= tokens * 4
    assert k.device_status() == 0
    s.close()


def test_synthetic_weights_follow_the_plan_layout(small):
    """src/checkpoint/plan.rs:135-141: 256-byte aligned spans in name order; rows at the GEMM pitch
    with zero padding; value ranges of the synthetic fill."""
    dims, weights, host = small
    from krea2_hrx_b200 import shape
    names = sorted(f"blocks.{i}.{n}" for i in range(3) for n in
                   ["qkvg.q", "qkvg.s", "wo.q", "wo.s", "gu.q", "gu.s", "down.q", "down.s", "prenorm", "postnorm",
                    "qnorm", "knorm"])
    base, _ = weights.locate(names[0])
    cursor = base
    for name in names:
        ptr, n = weights.locate(name)
        assert ptr == cursor and ptr % 256 == 0, name
        cursor = ptr + -(-n // 256) * 256
    down = host[0]["down.q"].reshape(dims.hidden, shape.gemm_pitch(dims.inter))
    assert down.min() >= -127 and down.max() <= 127 and np.all(down[:, dims.inter:] == 0)
    assert abs(float(down[:, :dims.inter].astype(np.float64).mean())) < 0.5
    s = host[1]["gu.s"]
    assert s.min() >= 1e-3 and s.max() <= 1e-2 + 1e-6
    assert 0.05 < host[2]["prenorm"].std() < 0.2
    with pytest.raises(k.InvalidArgument, match="no span named"):
        weights.locate("blocks.9.qkvg.q")


def test_graph_replay_equals_the_eager_run_after_inputs_change(small):
    """src/session/mod.rs:915-973."""
    from krea2_hrx_b200 import session
    dims, weights, host = small
    tokens = 275
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, tokens, 3)
    assert s.launches_per_forward() == 3 * 11
    for seed in (1, 2, 1):
        x, mods, cos, sin = so.make_inputs(dims, tokens, 3, seed=seed)
        eager = torch.from_numpy(x.copy()).view(torch.bfloat16)
        s.run(stream, eager, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
        # fresh device allocations every time: the graph must not depend on caller addresses
        x_dev = torch.from_numpy(x.copy()).view(torch.bfloat16).cuda()
        mods_dev = torch.from_numpy(mods).cuda()
        s.run_device(stream, x_dev, mods_dev, torch.from_numpy(cos), torch.from_numpy(sin))
        torch.cuda.synchronize()
        np.testing.assert_array_equal(bits(x_dev), bits(eager))
    s.close()


def test_a_block_range_equals_the_chain_of_its_parts(small):
    """src/session/mod.rs:1000-1065: two independent prefixes equal the whole."""
    from krea2_hrx_b200 import session
    dims, weights, host = small
    tokens = 64
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, tokens, 3)
    x, mods, cos, sin = so.make_inputs(dims, tokens, 3, seed=4)
    args = (torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    whole = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, whole, *args)
    parts = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, parts, *args, first_block=0, block_count=2)
    s.run(stream, parts, *args, first_block=2, block_count=1)
    np.testing.assert_array_equal(bits(parts), bits(whole))
    with pytest.raises(k.InvalidArgument, match="block range"):
        s.run(stream, parts, *args, first_block=3)
    with pytest.raises(k.InvalidArgument, match="block range"):
        s.run(stream, parts, *args, first_block=1, block_count=3)
    s.close()


def test_a_session_refuses_a_foreign_stream_and_wrong_sizes(small):
    """src/session/mod.rs:375-380, 975-998, 516-528."""
    from krea2_hrx_b200 import session
    dims, weights, host = small
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, 32, 2)
    x, mods, cos, sin = so.make_inputs(dims, 32, 2, seed=5)
    x_t = torch.from_numpy(x.copy()).view(torch.bfloat16)
    other = torch.cuda.Stream()
    with pytest.raises(k.InvalidArgument, match="stream that created it"):
        s.run(other, x_t, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    with pytest.raises(k.InvalidArgument, match="x has"):
        s.run(stream, x_t[:-1].clone(), torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    with pytest.raises(k.InvalidArgument, match="mods"):
        s.run(stream, x_t, torch.from_numpy(mods[:1].copy()), torch.from_numpy(cos), torch.from_numpy(sin))
    with pytest.raises(k.InvalidArgument, match="cos/sin"):
        s.run(stream, x_t, torch.from_numpy(mods), torch.from_numpy(cos[:1].copy()), torch.from_numpy(sin))
    with pytest.raises(k.InvalidArgument, match="weights hold"):
        session.Session(stream, weights, 32, 4)
    s.close()


def test_run_device_refuses_tensors_of_the_wrong_kind(small):
    """cos and sin are fingerprinted on the host and x and mods are read through raw device pointers, so a tensor on
    the wrong side, of another dtype or non-contiguous must be refused before the library sees its address."""
    from krea2_hrx_b200 import session
    dims, weights, host = small
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, 64, 2)
    x, mods, cos, sin = so.make_inputs(dims, 64, 2, seed=12)
    x_dev = torch.from_numpy(x.copy()).view(torch.bfloat16).cuda()
    mods_dev, cos_t, sin_t = torch.from_numpy(mods).cuda(), torch.from_numpy(cos), torch.from_numpy(sin)
    s.run_device(stream, x_dev, mods_dev, cos_t, sin_t)  # the well-formed call
    with pytest.raises(k.InvalidArgument, match="cos/sin"):
        s.run_device(stream, x_dev, mods_dev, cos_t.cuda(), sin_t)
    with pytest.raises(k.InvalidArgument, match="cos/sin"):
        s.run_device(stream, x_dev, mods_dev, cos_t.double(), sin_t.double())
    with pytest.raises(k.InvalidArgument, match="cos/sin"):
        s.run_device(stream, x_dev, mods_dev, cos_t.t().contiguous().t(), sin_t)
    with pytest.raises(k.InvalidArgument, match="x as a contiguous CUDA bfloat16"):
        s.run_device(stream, x_dev.cpu(), mods_dev, cos_t, sin_t)
    with pytest.raises(k.InvalidArgument, match="x as a contiguous CUDA bfloat16"):
        s.run_device(stream, x_dev.float(), mods_dev, cos_t, sin_t)
    with pytest.raises(k.InvalidArgument, match="mods as a contiguous CUDA float32"):
        s.run_device(stream, x_dev, mods_dev[:1].contiguous(), cos_t, sin_t)
    with pytest.raises(k.InvalidArgument, match="mods as a contiguous CUDA float32"):
        s.run_device(stream, x_dev, mods_dev.cpu(), cos_t, sin_t)
    torch.cuda.synchronize()
    s.close()


@pytest.mark.parametrize("tokens", [97, 700])
def test_dependent_launches_change_no_bit(small, tokens, monkeypatch):
    """With KREA2_DEPENDENT_LAUNCH=1 a session's launches carry the programmatic-stream-serialization attribute: a
    kernel's blocks start under the last blocks of the kernel before it and wait for it before their first global
    access.  Same kernels, same order: the full block (attention on) must give the same bytes, eagerly, replayed from
    the graph and in a profiled forward (which falls back to ordinary launches)."""
    from krea2_hrx_b200 import session
    dims, weights, host = small
    stream = torch.cuda.current_stream()
    layers = 3
    x, mods, cos, sin = so.make_inputs(dims, tokens, layers, seed=33)
    args = (torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    monkeypatch.delenv("KREA2_DEPENDENT_LAUNCH", raising=False)
    plain = session.Session(stream, weights, tokens, layers)
    want = torch.from_numpy(x.copy()).view(torch.bfloat16)
    plain.run(stream, want, *args)
    monkeypatch.setenv("KREA2_DEPENDENT_LAUNCH", "1")
    chained = session.Session(stream, weights, tokens, layers)
    for _ in range(3):  # the first call records the graph, the others replay it
        got = torch.from_numpy(x.copy()).view(torch.bfloat16)
        chained.run(stream, got, *args)
        np.testing.assert_array_equal(bits(got), bits(want))
    x_dev = torch.from_numpy(x.copy()).view(torch.bfloat16).cuda()
    chained.run_device(stream, x_dev, args[0].cuda(), args[1], args[2])
    torch.cuda.synchronize()
    np.testing.assert_array_equal(bits(x_dev.cpu()), bits(want))
    chained.set_profile(True)
    got = torch.from_numpy(x.copy()).view(torch.bfloat16)
    chained.run(stream, got, *args)
    np.testing.assert_array_equal(bits(got), bits(want))
    assert k.device_status() == 0
    plain.close()
    chained.close()


def test_profiled_forward_reports_the_reference_stage_labels(small):
    """src/session/mod.rs:461-494, 627-647."""
    from krea2_hrx_b200 import session
    dims, weights, host = small
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, 128, 3)
    x, mods, cos, sin = so.make_inputs(dims, 128, 3, seed=6)
    plain = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, plain, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    assert s.set_profile(True) is False
    profiled = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, profiled, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    np.testing.assert_array_equal(bits(profiled), bits(plain))
    table = dict(s.stage_profile())
    for label in ["prepare", "gemm qkvg", "qk norm + rope", "V transpose", "f16 attention", "prepare gated",
                  "gemm wo + residual", "gemm gate|up + swiglu", "prepare swiglu", "gemm down + residual"]:
        assert table[label] > 0.0, label
    s.set_attention(False)
    s.set_profile(True)
    s.run(stream, profiled, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    assert "f16 attention" not in dict(s.stage_profile()) and s.launches_per_forward() == 3 * 8
    assert s.set_profile(False) is True
    s.close()


def test_profile_json_appends_the_raw_intervals_of_each_profiled_forward(small, tmp_path, monkeypatch):
    """KREA2_PROFILE_JSON (src/session/mod.rs:438-459): one JSON line per profiled forward with tokens, layers
    and the device interval of every launch; an unwritable path is an invalid-argument error naming the variable."""
    import json
    from krea2_hrx_b200 import session
    dims, weights, host = small
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, 64, 2)
    x, mods, cos, sin = so.make_inputs(dims, 64, 2, seed=8)
    path = tmp_path / "profile.jsonl"
    monkeypatch.setenv("KREA2_PROFILE_JSON", str(path))
    s.set_profile(True)
    for _ in range(2):
        s.run(stream, torch.from_numpy(x.copy()).view(torch.bfloat16), torch.from_numpy(mods), torch.from_numpy(cos),
              torch.from_numpy(sin))
    records = [json.loads(line) for line in path.read_text().splitlines()]
    assert len(records) == 2
    for record in records:
        assert record["tokens"] == 64 and record["layers"] == 2
        intervals = record["profile"]["intervals"]
        assert len(intervals) == 2 * 11 and record["profile"]["frequency_hz"] == 1000000000
        assert [i["label"] for i in intervals[:3]] == ["prepare", "gemm qkvg", "qk norm + rope"]
        assert [i["block"] for i in intervals] == [0] * 11 + [1] * 11
        assert all(i["end_tick"] >= i["start_tick"] for i in intervals)
        assert all(b["start_tick"] >= a["start_tick"] for a, b in zip(intervals, intervals[1:]))
        total_ms = sum(i["end_tick"] - i["start_tick"] for i in intervals) / 1e6
        assert abs(total_ms - sum(ms for _, ms in s.stage_profile())) < 0.05 or record is records[0]
    monkeypatch.setenv("KREA2_PROFILE_JSON", str(tmp_path / "missing" / "profile.jsonl"))
    with pytest.raises(k.InvalidArgument, match="KREA2_PROFILE_JSON"):
        s.run(stream, torch.from_numpy(x.copy()).view(torch.bfloat16), torch.from_numpy(mods), torch.from_numpy(cos),
              torch.from_numpy(sin))
    s.close()


@pytest.mark.parametrize("tokens", [64, 300])
def test_full_block_session_equals_the_oracle_chain_around_the_attention_kernel(small, tokens):
    """With attention on, a block is the reference's eleven launches.  Everything but attention is
    exact on the CPU (RoPE included) and the attention kernel is deterministic, so the session must
    equal, bit for bit, the oracle chain with the standalone attention kernel in attention's place.
    Against the chain with float64 attention the residual stream is only close: random int8
    weights amplify attention's rounding through the following quantisations."""
    from krea2_hrx_b200 import session
    from krea2_hrx_b200.parallel import DeviceView
    dims, weights, host = small
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, tokens, 2)
    x, mods, cos, sin = so.make_inputs(dims, tokens, 2, seed=tokens)
    args = (torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    one = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, one, *args, first_block=0, block_count=1)
    want, trace = so.oracle_forward(dims, host, x, mods, count=1, attention=so.gpu_attention(tokens), cos=cos, sin=sin)
    # q, k, v of the block just run are still in the session's buffers: exact against the oracle's RoPE
    for name, want_bits in zip(("q", "k", "v"), trace["qkv"]):
        ptr, nbytes = s.buffer(name)
        width = want_bits.shape[1]
        got = torch.as_tensor(DeviceView(ptr, nbytes), device="cuda").view(torch.int16)[: tokens * width]
        np.testing.assert_array_equal(got.cpu().numpy().view(np.uint16).reshape(tokens, width), want_bits, err_msg=name)
    np.testing.assert_array_equal(bits(one), want)
    both = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, both, *args)
    want2, _ = so.oracle_forward(dims, host, x, mods, count=2, attention=so.gpu_attention(tokens), cos=cos, sin=sin)
    np.testing.assert_array_equal(bits(both), want2)
    loose, _ = so.oracle_forward(dims, host, x, mods, count=2, attention=True, cos=cos, sin=sin)
    assert so.relative_l2(bits(both), loose) < 6e-2
    assert k.device_status() == 0
    s.close()


@pytest.mark.parametrize("tokens", [4608, 16896])
def test_the_benchmark_sized_chain_matches_the_oracle_on_sampled_tokens(tokens):
    """Reference dimensions at the benchmark's token count and at the largest the session accepts.  The W8A8
    chain treats every token on its own (prologues and GEMM rows are per token), so the oracle chain over a
    sample of rows must equal the same rows of the full forward bit for bit; two forwards must agree in full."""
    from krea2_hrx_b200 import session
    dims, layers = session.ModelDims(), 2
    stream = torch.cuda.current_stream()
    weights = session.Weights(dims, layers)
    weights.fill_synthetic(99, stream)
    s = session.Session(stream, weights, tokens, layers)
    s.set_attention(False)
    x, mods, cos, sin = so.make_inputs(dims, tokens, layers, seed=tokens)
    runs = []
    for _ in range(2):
        x_t = torch.from_numpy(x.copy()).view(torch.bfloat16)
        s.run(stream, x_t, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
        runs.append(bits(x_t).reshape(tokens, dims.hidden))
    np.testing.assert_array_equal(runs[0], runs[1])
    rows = np.unique(np.concatenate([[0, 1, 255, 256, tokens - 257, tokens - 1],
                                     np.random.default_rng(3).integers(0, tokens, 26)]))
    want, _ = so.oracle_forward(dims, so.host_weights(weights, layers), x[rows], mods)
    np.testing.assert_array_equal(runs[0][rows], want)
    s.close()
