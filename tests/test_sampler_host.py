"""The pointwise sampler arithmetic and the sigma schedule: the CPU oracle against the reference's own
known-answer tests (tests/arithmetic.rs, tests/schedule.rs) and recorded scheduler bits, and the library's
host-side schedule functions against the same (they run without a GPU)."""
import hashlib
import os

import numpy as np
import pytest

import kat
import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "schedule_sigmas.npz")
TOKENS = [0, 16, 256, 589, 4096, 6400, 16384]


def bf(x):
    return kat.bf16_round_f32(np.asarray(x, dtype=np.float32))


def test_the_euler_step_rounds_where_the_sampler_rounds():
    """tests/arithmetic.rs:38-62."""
    i = np.arange(1000, dtype=np.float32)
    samples, velocity = (i - 500.0) / np.float32(97.0), np.sin(i).astype(np.float32) * np.float32(3.0)
    delta = np.float32(-0.1234)
    product = bf(bf(delta) * bf(velocity))
    want = kat.bf16_bits_from_f32(bf(samples) + product)
    got = oracle.euler(kat.bf16_bits_from_f32(samples), kat.bf16_bits_from_f32(velocity), float(delta))
    np.testing.assert_array_equal(got, want)


def test_guidance_combines_as_krea_defines_it():
    """tests/arithmetic.rs:64-84."""
    i = np.arange(512, dtype=np.float32)
    cond, uncond = np.cos(i * np.float32(0.017)).astype(np.float32), np.sin(i * np.float32(0.023)).astype(np.float32)
    scale = np.float32(3.5)
    c, u = bf(cond), bf(uncond)
    want = kat.bf16_bits_from_f32(c + bf(scale * bf(c - u)))
    got = oracle.guidance(kat.bf16_bits_from_f32(cond), kat.bf16_bits_from_f32(uncond), float(scale))
    np.testing.assert_array_equal(got, want)


def test_modulation_adds_the_vector_to_every_table_row():
    """kernels/native/modulation.loom:33-42: bf16 of the sum, widened to f32, x repeating with period xsize."""
    rng = np.random.default_rng(11)
    xsize, rows = 6 * 64, 5
    x = kat.bf16_bits_from_f32(rng.standard_normal(xsize).astype(np.float32))
    tables = kat.bf16_bits_from_f32(rng.standard_normal((rows, xsize)).astype(np.float32) * 0.3)
    want = bf(kat.bf16_to_f32(x)[None, :] + kat.bf16_to_f32(tables))
    np.testing.assert_array_equal(oracle.modulation(x, tables).view(np.uint32), want.view(np.uint32))


def sigma_stream(sigma, dynamic_mu):
    out = []
    for tokens in TOKENS:
        mu = 1.15 if tokens == 0 else dynamic_mu(tokens)
        for steps in range(1, 101):
            out.extend(sigma(step, steps, mu) for step in range(steps + 1))
    return np.array(out, dtype="<f4")


def check_against_recorded_scheduler(sigma, dynamic_mu):
    """tests/schedule.rs:4-22: all 36,050 recorded scheduler sigmas, bit for bit (by the hash of the whole
    stream, and value by value on the stored subset of grids)."""
    golden = np.load(GOLDEN)
    stream = sigma_stream(sigma, dynamic_mu)
    assert stream.size == int(golden["count"][0])
    for key in golden.files:
        if not (key.startswith("t") and "_s" in key):
            continue
        tokens, steps = (int(v[1:]) for v in key.split("_"))
        mu = 1.15 if tokens == 0 else dynamic_mu(tokens)
        got = np.array([sigma(step, steps, mu) for step in range(steps + 1)], dtype="<f4").view(np.uint32)
        np.testing.assert_array_equal(got, golden[key], err_msg=key)
    assert hashlib.sha256(stream.tobytes()).digest() == golden["sha256"].tobytes()


def check_schedule_properties(sigma, next_sigma, dynamic_mu):
    """The unit tests of src/pipeline/schedule.rs:39-69."""
    for step in range(8):
        assert next_sigma(step, 8, 8, 1.15) == sigma(step + 1, 8, 1.15)
    assert next_sigma(2, 4, 8, 1.15) == sigma(3, 8, 1.15)
    assert next_sigma(3, 4, 8, 1.15) == 0.0
    assert sigma(0, 8, 1.15) == 1.0 and sigma(8, 8, 1.15) == 0.0
    for step in range(8):
        assert sigma(step, 8, 1.15) > sigma(step + 1, 8, 1.15), step
    assert abs(dynamic_mu(256) - 0.5) < 1e-12
    assert abs(dynamic_mu(6400) - 1.15) < 1e-12
    assert abs(dynamic_mu(4096) - 0.906) < 1e-3


def test_oracle_schedule_matches_the_recorded_scheduler_bits():
    check_against_recorded_scheduler(oracle.sigma, oracle.dynamic_mu)
    check_schedule_properties(oracle.sigma, oracle.next_sigma, oracle.dynamic_mu)


def test_library_schedule_matches_the_recorded_scheduler_bits():
    schedule = pytest.importorskip("krea2_hrx_b200.schedule")
    check_against_recorded_scheduler(schedule.sigma, schedule.dynamic_mu)
    check_schedule_properties(schedule.sigma, schedule.next_sigma, schedule.dynamic_mu)
    assert schedule.TURBO_MU == 1.15
