"""The oracle's block chain against the reference's own torch block.

tests/golden/block_w8a8.npz holds what `Krea2Ref.block` of scripts/quantized_reference.py (:262-268,
imported unmodified by tests/golden/make_block_golden.py) returns for one and two transformer blocks
at the reference's dimensions, `quant="w8a8"`, over the seeded weights of tests/block_case.py.  The
torch code rotates with a dense matrix, quantises by division and rounds to bf16 only where its
tensors are bf16, so the comparison is by relative RMS, the measure the reference itself uses
between its kernels and this code: 0.0117 over a 28-block forward (docs/testing.md:226).
"""
import os

import numpy as np
import pytest

import block_case
import oracle
import session_oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "block_w8a8.npz")
# relative RMS bounds per block count; the reference's own 28-block figure is the ceiling
BOUNDS = {1: 0.008, 2: 0.0117}


@pytest.fixture(scope="module")
def case():
    golden = np.load(GOLDEN)
    blocks = block_case.oracle_blocks(block_case.block_tensors())
    return golden, blocks


def test_the_fixture_inputs_are_the_seeded_ones(case):
    golden, _ = case
    x, mods = block_case.block_inputs()
    np.testing.assert_array_equal(golden["x"], oracle.f32_to_bf16_bits(x))
    np.testing.assert_array_equal(golden["mods"], mods)
    assert golden["cos"].shape == (block_case.TOKENS, block_case.HEAD_DIM)


@pytest.mark.parametrize("count", [1, 2])
def test_the_oracle_chain_with_float64_attention_tracks_the_reference_block(case, count):
    from krea2_hrx_b200 import session
    golden, blocks = case
    got, _ = session_oracle.oracle_forward(session.ModelDims(), blocks, golden["x"], golden["mods"], count=count,
                                           attention=True, cos=golden["cos"], sin=golden["sin"])
    want = golden[f"after_block_{count - 1}"]
    rel = session_oracle.relative_l2(got, want)
    print(f"oracle chain vs Krea2Ref, {count} block(s): relative RMS {rel:.5f} (reference kernels vs the same code "
          f"over 28 blocks: 0.0117)")
    assert rel < BOUNDS[count]
    # the update itself (not only the residual it rides on) must agree
    x0 = oracle.bf16_bits_to_f32(golden["x"]).astype(np.float64)
    delta_got = oracle.bf16_bits_to_f32(got).astype(np.float64) - x0
    delta_want = oracle.bf16_bits_to_f32(want).astype(np.float64) - x0
    assert np.linalg.norm(delta_got - delta_want) / np.linalg.norm(delta_want) < 0.04


def test_the_oracle_chain_tracks_the_reference_block_over_several_key_tiles(case):
    """208 tokens: the attention spans two 128-key tiles, the second ragged.  tests/golden/block_w8a8_long.npz holds
    the reference block's output rows `rows`; x and the modulation are regenerated from the seed."""
    from krea2_hrx_b200 import session
    _, blocks = case
    golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "block_w8a8_long.npz"))
    x, mods = block_case.long_inputs()
    assert list(golden["rows"]) == block_case.LONG_ROWS and golden["cos"].shape == (block_case.LONG_TOKENS, block_case.HEAD_DIM)
    got, _ = session_oracle.oracle_forward(session.ModelDims(), blocks, oracle.f32_to_bf16_bits(x), mods, count=1,
                                           attention=True, cos=golden["cos"], sin=golden["sin"])
    rel = session_oracle.relative_l2(got[golden["rows"]], golden["after_block_0_rows"])
    print(f"oracle chain vs Krea2Ref, 208 tokens, 1 block: relative RMS {rel:.5f}")
    assert rel < BOUNDS[1]
    x0 = x[golden["rows"]].astype(np.float64)
    delta_got = oracle.bf16_bits_to_f32(got[golden["rows"]]).astype(np.float64) - x0
    delta_want = oracle.bf16_bits_to_f32(golden["after_block_0_rows"]).astype(np.float64) - x0
    assert np.linalg.norm(delta_got - delta_want) / np.linalg.norm(delta_want) < 0.04


def test_modulation_and_two_blocks_track_the_reference_blocks_forward(case):
    """tests/golden/blocks_forward_w8a8.npz: `Krea2Ref.blocks_forward` (scripts/quantized_reference.py:270-273) -- per
    block `block_modulation` (the shared vector plus the block's `mod.lin` table, :257-259) and `block` -- over the
    48-token inputs.  Here: the oracle's modulation kernel feeds the oracle chain."""
    from krea2_hrx_b200 import session
    golden, blocks = case
    want = np.load(os.path.join(os.path.dirname(__file__), "golden", "blocks_forward_w8a8.npz"))["out"]
    vector, tables = block_case.modulation_inputs()
    mods = oracle.modulation(oracle.f32_to_bf16_bits(vector), oracle.f32_to_bf16_bits(tables)).reshape(block_case.LAYERS, 6, -1)
    got, _ = session_oracle.oracle_forward(session.ModelDims(), blocks, golden["x"], mods, count=block_case.LAYERS,
                                           attention=True, cos=golden["cos"], sin=golden["sin"])
    rel = session_oracle.relative_l2(got, want)
    print(f"oracle modulation + chain vs Krea2Ref.blocks_forward, 2 blocks: relative RMS {rel:.5f}")
    assert rel < BOUNDS[2]
