"""The CUDA session, attention on, against the reference's own torch block (tests/golden/block_w8a8.npz,
made by tests/golden/make_block_golden.py from `Krea2Ref.block`, scripts/quantized_reference.py:262-268).

The seeded weights of tests/block_case.py are written as a checkpoint file under the checkpoint's own
tensor names, loaded through the library's checkpoint path at the reference's dimensions, and one and
two blocks are run from host buffers.  Relative RMS is the reference's measure between its kernels and
this torch code: 0.0117 over 28 blocks (docs/testing.md:226)."""
import os

import numpy as np
import pytest
import torch

import block_case
import session_oracle
from oracle import plan as plan_oracle

pytestmark = pytest.mark.gpu

k = pytest.importorskip("krea2_hrx_b200")
from krea2_hrx_b200 import session  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "block_w8a8.npz")
BOUNDS = {1: 0.008, 2: 0.0117}


@pytest.fixture(scope="module")
def loaded(tmp_path_factory):
    tensors = block_case.block_tensors()
    path = tmp_path_factory.mktemp("block") / "krea2_block_case.safetensors"
    plan_oracle.write_safetensors(str(path), tensors, metadata={"format": "pt"})
    weights = session.Weights.load(path, torch.cuda.current_stream())
    torch.cuda.synchronize()
    os.remove(path)
    return weights, np.load(GOLDEN)


@pytest.mark.parametrize("count", [1, 2])
def test_the_session_with_attention_tracks_the_reference_block(loaded, count):
    weights, golden = loaded
    assert weights.dims == session.ModelDims() and weights.layers == block_case.LAYERS
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, block_case.TOKENS, count)
    s.set_attention(True)
    x = torch.from_numpy(golden["x"].copy()).view(torch.bfloat16)
    s.run(stream, x, torch.from_numpy(golden["mods"][:count].copy()), torch.from_numpy(golden["cos"]),
          torch.from_numpy(golden["sin"]))
    got = x.view(torch.int16).numpy().view(np.uint16)
    want = golden[f"after_block_{count - 1}"]
    rel = session_oracle.relative_l2(got, want)
    print(f"CUDA session vs Krea2Ref, {count} block(s): relative RMS {rel:.5f} (reference kernels vs the same code "
          f"over 28 blocks: 0.0117)")
    assert rel < BOUNDS[count]
    assert k.device_status() == 0
    s.close()


def test_the_session_tracks_the_reference_block_over_several_key_tiles(loaded):
    """208 tokens, one block: the attention kernel walks two key tiles, the second ragged, against the reference
    block's own softmax (tests/golden/block_w8a8_long.npz: the rope tables and a sample of the output rows)."""
    import oracle
    weights, _ = loaded
    golden = np.load(os.path.join(os.path.dirname(__file__), "golden", "block_w8a8_long.npz"))
    x32, mods = block_case.long_inputs()
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, block_case.LONG_TOKENS, 1)
    s.set_attention(True)
    x = torch.from_numpy(oracle.f32_to_bf16_bits(x32).view(np.int16).copy()).view(torch.bfloat16)
    s.run(stream, x, torch.from_numpy(mods.copy()), torch.from_numpy(golden["cos"]), torch.from_numpy(golden["sin"]))
    got = x.view(torch.int16).numpy().view(np.uint16)[golden["rows"]]
    rel = session_oracle.relative_l2(got, golden["after_block_0_rows"])
    print(f"CUDA session vs Krea2Ref, 208 tokens, 1 block: relative RMS {rel:.5f}")
    assert rel < BOUNDS[1]
    assert k.device_status() == 0
    s.close()


def test_modulation_and_the_session_track_the_reference_blocks_forward(loaded):
    """`krea2_modulation` (the shared vector plus each block's table) feeding a two-block session, against
    `Krea2Ref.blocks_forward` (scripts/quantized_reference.py:257-259, 270-273; tests/golden/blocks_forward_w8a8.npz)."""
    import oracle
    from krea2_hrx_b200 import ops
    weights, golden = loaded
    want = np.load(os.path.join(os.path.dirname(__file__), "golden", "blocks_forward_w8a8.npz"))["out"]
    vector, tables = block_case.modulation_inputs()
    as_bf16 = lambda a: torch.from_numpy(oracle.f32_to_bf16_bits(a).view(np.int16).copy()).view(torch.bfloat16).cuda()
    stream = torch.cuda.current_stream()
    mods = torch.empty((block_case.LAYERS, 6, block_case.HIDDEN), dtype=torch.float32, device="cuda")
    ops.modulation(as_bf16(vector), as_bf16(tables), mods, stream)
    s = session.Session(stream, weights, block_case.TOKENS, block_case.LAYERS)
    s.set_attention(True)
    x = torch.from_numpy(golden["x"].copy()).view(torch.bfloat16).cuda()
    s.run_device(stream, x, mods, torch.from_numpy(golden["cos"]), torch.from_numpy(golden["sin"]))
    torch.cuda.synchronize()
    got = x.cpu().view(torch.int16).numpy().view(np.uint16)
    rel = session_oracle.relative_l2(got, want)
    print(f"CUDA modulation + session vs Krea2Ref.blocks_forward, 2 blocks: relative RMS {rel:.5f}")
    assert rel < BOUNDS[2]
    assert k.device_status() == 0
    s.close()
