"""The sampler's pointwise kernels through the C ABI against the CPU oracle, bit for bit."""
import numpy as np
import pytest
import torch

import kat
import oracle

pytestmark = pytest.mark.gpu

k = pytest.importorskip("krea2_hrx_b200")
from krea2_hrx_b200 import kernels, ops  # noqa: E402


def dev(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda().view(torch.bfloat16)


def host(t: torch.Tensor) -> np.ndarray:
    torch.cuda.synchronize()
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def random_bits(rng, n, scale=1.0):
    x = rng.standard_normal(n).astype(np.float32) * np.float32(scale)
    x[rng.integers(0, n, max(1, n // 50))] *= 40.0
    x[rng.integers(0, n, max(1, n // 200))] = 0.0
    return kat.bf16_bits_from_f32(x)


def test_the_euler_step_rounds_where_the_sampler_rounds():
    """tests/arithmetic.rs:38-62, on the device."""
    i = np.arange(1000, dtype=np.float32)
    samples = kat.bf16_bits_from_f32((i - 500.0) / np.float32(97.0))
    velocity = kat.bf16_bits_from_f32(np.sin(i).astype(np.float32) * np.float32(3.0))
    sample = dev(samples).view(1, 1000)
    ops.euler_step(sample, dev(velocity).view(1, 1000), -0.1234)
    np.testing.assert_array_equal(host(sample).ravel(), oracle.euler(samples, velocity, -0.1234))


def test_guidance_combines_as_krea_defines_it():
    """tests/arithmetic.rs:64-84, on the device."""
    i = np.arange(512, dtype=np.float32)
    cond = kat.bf16_bits_from_f32(np.cos(i * np.float32(0.017)).astype(np.float32))
    uncond = kat.bf16_bits_from_f32(np.sin(i * np.float32(0.023)).astype(np.float32))
    c = dev(cond).view(1, 512)
    ops.guidance(c, dev(uncond).view(1, 512), 3.5)
    np.testing.assert_array_equal(host(c).ravel(), oracle.guidance(cond, uncond, 3.5))


@pytest.mark.parametrize("count", [1, 7, 8, 9, 255, 4096 * 64, 4096 * 64 + 3])
@pytest.mark.parametrize("offset", [0, 1])
def test_in_place_updates_are_bit_exact_at_ragged_sizes_and_alignments(count, offset):
    """Vector path, its ragged tail, and the element path an odd element offset forces."""
    rng = np.random.default_rng(count * 2 + offset)
    a, b = random_bits(rng, count + offset), random_bits(rng, count + offset, 3.0)
    for delta in (-0.1234, 0.0625, -1.0):
        target, other = dev(a), dev(b)
        ops.euler_step(target[offset:], other[offset:], delta)
        got = host(target)
        np.testing.assert_array_equal(got[offset:], oracle.euler(a[offset:], b[offset:], delta))
        np.testing.assert_array_equal(got[:offset], a[:offset])
    target, other = dev(a), dev(b)
    ops.guidance(target[offset:], other[offset:], 3.5)
    np.testing.assert_array_equal(host(target)[offset:], oracle.guidance(a[offset:], b[offset:], 3.5))


def test_a_zero_delta_leaves_the_latents_alone():
    """Idempotence at the largest latent grid the reference generates (16384 tokens x 64 channels)."""
    rng = np.random.default_rng(5)
    a, b = random_bits(rng, 16384 * 64), random_bits(rng, 16384 * 64)
    target = dev(a)
    ops.euler_step(target, dev(b), 0.0)
    np.testing.assert_array_equal(host(target), a)


@pytest.mark.parametrize("layers,width", [(28, 6144), (3, 6 * 50), (1, 7)])
def test_modulation_tables_are_bit_exact(layers, width):
    """Models::modulation (src/models/graph.rs:405-425) at the reference's size [28][6][6144] and at ragged ones."""
    rng = np.random.default_rng(layers)
    xsize = 6 * width
    x, tables = random_bits(rng, xsize), random_bits(rng, layers * xsize, 0.3)
    out = torch.empty(layers * xsize, dtype=torch.float32, device="cuda")
    ops.modulation(dev(x), dev(tables), out)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy().view(np.uint32), oracle.modulation(x, tables).view(np.uint32))


def test_generic_launch_reaches_the_sampler_kernels():
    """Ops::launch_1d with the reference's kernel names; the float scalar rides in the config."""
    rng = np.random.default_rng(9)
    n = 2048
    a, b = random_bits(rng, n), random_bits(rng, n)
    target, other = dev(a), dev(b)
    one = kernels.Scalars()
    ops.Ops().launch_1d(None, "euler", kernels.config([]), one.index(n).float(-0.25), [target, other], n)
    np.testing.assert_array_equal(host(target), oracle.euler(a, b, -0.25))
    with pytest.raises(k.InvalidArgument):
        ops.Ops().launch_1d(None, "euler", kernels.config([]), kernels.Scalars().index(n), [target, other], n)


def test_mismatched_shapes_are_refused():
    a, b = torch.zeros(4, 8, dtype=torch.bfloat16, device="cuda"), torch.zeros(8, 4, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(k.InvalidArgument):
        ops.euler_step(a, b, 0.1)
    with pytest.raises(k.InvalidArgument):
        ops.guidance(a, b, 0.1)
