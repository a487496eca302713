"""The denoising loop (schedule -> modulation -> blocks -> [guidance] -> Euler) around a resident session,
against the same loop on the CPU oracle, bit for bit.  Small dimensions, the W8A8 chain alone so that every
stage is exact; one case runs the full block with the library's attention kernel as that stage of the oracle
loop."""
import numpy as np
import pytest
import torch

import oracle
import session_oracle as so

pytestmark = pytest.mark.gpu

k = pytest.importorskip("krea2_hrx_b200")
from krea2_hrx_b200 import pipeline, schedule, session  # noqa: E402


def dev16(bits_array):
    return torch.from_numpy(np.ascontiguousarray(bits_array).view(np.int16)).cuda().view(torch.bfloat16)


def host16(t):
    torch.cuda.synchronize()
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def make_case(layers, text_tokens, image_tokens, steps, seed):
    dims = session.ModelDims(**so.SMALL)
    rng = np.random.default_rng(seed)
    tokens = text_tokens + image_tokens
    bf = lambda a: oracle.f32_to_bf16_bits(np.asarray(a, dtype=np.float32))
    case = dict(dims=dims, tokens=tokens,
                text=bf(rng.standard_normal((text_tokens, dims.hidden))),
                uncond=bf(rng.standard_normal((text_tokens, dims.hidden))),
                sample=bf(rng.standard_normal((image_tokens, dims.hidden))),
                tables=bf(rng.standard_normal((layers, 6, dims.hidden)) * 0.3),
                vectors=[bf(rng.standard_normal(6 * dims.hidden) * 0.2) for _ in range(steps)])
    case["cos"] = np.cos(rng.uniform(0, 6.28, (tokens, dims.head_dim))).astype(np.float32)
    case["sin"] = np.sin(rng.uniform(0, 6.28, (tokens, dims.head_dim))).astype(np.float32)
    return case


def oracle_loop(case, blocks, steps, mu, guidance, last=None, attention=False):
    last = steps if last is None else last
    sample = case["sample"].copy()
    text_tokens = case["text"].shape[0]
    deltas = []
    for step in range(last):
        sigma = np.float32(oracle.sigma(step, steps, mu))
        delta = np.float32(oracle.next_sigma(step, last, steps, mu)) - sigma
        deltas.append(float(delta))
        mods = oracle.modulation(case["vectors"][step], case["tables"])

        def forward(text):
            x = np.concatenate([text, sample], axis=0)
            out, _ = so.oracle_forward(case["dims"], blocks, x, mods, attention=attention, cos=case["cos"], sin=case["sin"])
            return np.ascontiguousarray(out[text_tokens:])
        velocity = forward(case["text"])
        if guidance > 0:
            velocity = oracle.guidance(velocity, forward(case["uncond"]), guidance)
        sample = oracle.euler(sample, velocity, float(delta))
    return sample, deltas


def build(case, layers, steps, mu, guidance, attention):
    stream = torch.cuda.current_stream()
    weights = session.Weights(case["dims"], layers)
    weights.fill_synthetic(31, stream)
    s = session.Session(stream, weights, case["tokens"], layers)
    s.set_attention(attention)
    d = pipeline.Denoiser(s, dev16(case["tables"]), torch.from_numpy(case["cos"]), torch.from_numpy(case["sin"]),
                          dev16(case["text"]), steps=steps, mu=mu, guidance=guidance,
                          uncond_text=dev16(case["uncond"]) if guidance > 0 else None)
    return s, d, so.host_weights(weights, layers)


def test_eight_turbo_steps_equal_the_oracle_loop():
    """Config: 8 steps, the Turbo shift 1.15, no guidance (src/pipeline/mod.rs:306-308, 338)."""
    layers, steps = 2, 8
    case = make_case(layers, 16, 64, steps, seed=5)
    s, d, blocks = build(case, layers, steps, schedule.TURBO_MU, 0.0, attention=False)
    sample = dev16(case["sample"])
    seen = []
    d.generate(sample, [dev16(v) for v in case["vectors"]], progress=lambda step, last: seen.append((step, last)) or pipeline.CONTINUE)
    want, deltas = oracle_loop(case, blocks, steps, schedule.TURBO_MU, 0.0)
    np.testing.assert_array_equal(host16(sample), want)
    assert seen == [(i + 1, steps) for i in range(steps)]
    assert abs(sum(deltas) + schedule.sigma(0, steps, schedule.TURBO_MU)) < 1e-6, "the deltas walk sigma down to zero"
    assert k.device_status() == 0
    s.close()


def test_guided_steps_with_the_dynamic_shift_and_an_early_finish():
    """Raw's loop: two forwards per step combined by guidance, mu from the image's token count, and a progress
    callback that ends the run early, whose last step lands on sigma zero (schedule.rs:33-35)."""
    layers, steps = 1, 6
    case = make_case(layers, 16, 48, steps, seed=9)
    s, d, blocks = build(case, layers, steps, None, 3.5, attention=False)
    assert d.mu == schedule.dynamic_mu(48)
    sample = dev16(case["sample"])
    d.generate(sample, [dev16(v) for v in case["vectors"]],
               progress=lambda step, last: pipeline.FINISH if step == 2 else pipeline.CONTINUE)
    want, deltas = oracle_loop(case, blocks, steps, schedule.dynamic_mu(48), 3.5, last=3)
    np.testing.assert_array_equal(host16(sample), want)
    assert len(deltas) == 3
    with pytest.raises(k.Cancelled):
        d.generate(sample, [dev16(v) for v in case["vectors"]], progress=lambda step, last: pipeline.CANCEL)
    s.close()


def test_steps_of_the_full_block_equal_the_oracle_loop_around_the_attention_kernel():
    layers, steps = 2, 3
    case = make_case(layers, 16, 64, steps, seed=13)
    s, d, blocks = build(case, layers, steps, schedule.TURBO_MU, 0.0, attention=True)
    sample = dev16(case["sample"])
    d.generate(sample, [dev16(v) for v in case["vectors"]])
    want, _ = oracle_loop(case, blocks, steps, schedule.TURBO_MU, 0.0, attention=so.gpu_attention(case["tokens"]))
    np.testing.assert_array_equal(host16(sample), want)
    s.close()


def test_bad_arguments_are_refused():
    case = make_case(1, 16, 48, 2, seed=1)
    s, d, _ = build(case, 1, 2, schedule.TURBO_MU, 0.0, attention=False)
    with pytest.raises(k.InvalidArgument):
        pipeline.Denoiser(s, dev16(case["tables"]), torch.from_numpy(case["cos"]), torch.from_numpy(case["sin"]),
                          dev16(case["text"]), steps=0)
    with pytest.raises(k.InvalidArgument):
        pipeline.Denoiser(s, dev16(case["tables"]), torch.from_numpy(case["cos"]), torch.from_numpy(case["sin"]),
                          dev16(case["text"]), guidance=3.5)  # no negative prompt
    with pytest.raises(k.InvalidArgument):
        d.generate(dev16(case["sample"]), [dev16(case["vectors"][0])])  # one vector for two steps
    s.close()


@pytest.mark.parametrize("world,text_tokens,image_tokens", [(2, 16, 120), (4, 40, 91), (3, 70, 61), (8, 50, 206)])
def test_the_token_sharded_loop_equals_the_loop_on_one_device(world, text_tokens, image_tokens):
    """Every rank keeps to its rows of [text; image] through all steps (ranks emulated on this GPU, their launches
    interleaved stage by stage); the rows each rank owns must equal the single-device loop's, full block with
    attention.  The shares cut through the text/image boundary in different places: a rank of text rows only
    (world 3), one of both, ranks of image rows only."""
    from krea2_hrx_b200 import parallel
    layers, steps = 3, 4
    case = make_case(layers, text_tokens, image_tokens, steps, seed=20 + world)
    s, d, _ = build(case, layers, steps, schedule.TURBO_MU, 0.0, attention=True)
    vectors = [dev16(v) for v in case["vectors"]]
    want = dev16(case["sample"])
    d.generate(want, vectors)
    fabric = parallel.LocalFabric(world)
    runners = [parallel.TokenParallel(fabric, r, s.weights, case["tokens"], layers) for r in range(world)]
    loops = [pipeline.ShardedDenoiser(run, dev16(case["tables"]), torch.from_numpy(case["cos"]), torch.from_numpy(case["sin"]),
                                      dev16(case["text"]), steps=steps, graph=False) for run in runners]
    assert sum(loop.image_rows[1] for loop in loops) == image_tokens
    if world == 3:
        assert loops[0].image_rows[1] == 0  # 44 rows of the 70 text tokens and nothing else
    samples = [dev16(case["sample"]) for _ in range(world)]
    for index in range(steps):
        for loop, sample in zip(loops, samples):
            loop.begin_step(index, sample, vectors[index])
        generators = [run.stages("push") for run in runners]
        while generators:
            alive = []
            for g in generators:
                try:
                    next(g)
                    alive.append(g)
                except StopIteration:
                    pass
            generators = alive
        for loop, sample in zip(loops, samples):
            loop.finish_step(sample)
    got = dev16(case["sample"])  # rows no rank owns would stay as they started; every row has an owner
    for loop, sample in zip(loops, samples):
        first, count = loop.image_rows
        got[first:first + count] = sample[first:first + count]
        others = torch.ones(image_tokens, dtype=torch.bool)
        others[first:first + count] = False
        assert torch.equal(sample[others.cuda()].view(torch.int16), dev16(case["sample"])[others.cuda()].view(torch.int16))
    np.testing.assert_array_equal(host16(got), host16(want))
    assert k.device_status() == 0
    with pytest.raises(k.InvalidArgument):
        loops[0].begin_step(0, samples[0][:-1], vectors[0])
    s.close()
