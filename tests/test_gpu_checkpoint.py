"""Loading a checkpoint file onto the device: every span bit for bit, and a session over the loaded
weights against the CPU oracle chain fed from the file's own tensors."""
import numpy as np
import pytest
import torch

import session_oracle
from oracle import plan as plan_oracle

pytestmark = pytest.mark.gpu

k = pytest.importorskip("krea2_hrx_b200")
from krea2_hrx_b200 import session  # noqa: E402
from krea2_hrx_b200.checkpoint import Checkpoint  # noqa: E402

LAYERS = 2


@pytest.fixture(scope="module")
def loaded(tmp_path_factory):
    tensors = plan_oracle.synthetic_blocks(np.random.default_rng(21), layers=LAYERS, bf16_norms=False, **session_oracle.SMALL)
    path = tmp_path_factory.mktemp("ckpt") / "krea2_small.safetensors"
    plan_oracle.write_safetensors(str(path), tensors, metadata={"format": "pt"}, prefix="model.diffusion_model.")
    weights = session.Weights.load(path, torch.cuda.current_stream())
    torch.cuda.synchronize()
    return weights, tensors


def test_every_span_lands_where_the_plan_says(loaded):
    weights, tensors = loaded
    assert weights.layers == LAYERS
    assert (weights.dims.hidden, weights.dims.kv_heads, weights.dims.head_dim, weights.dims.inter) == (2048, 2, 128, 4096)
    want, total = plan_oracle.plan(tensors, LAYERS)
    assert session.Weights.plan_bytes(weights.dims, LAYERS) == total
    base, _ = weights.locate(next(iter(want)))
    for name, expect in want.items():
        ptr, nbytes = weights.locate(name)
        assert ptr - base == expect["offset"] and nbytes == expect["image"].size, name
        np.testing.assert_array_equal(weights.read(name, torch.uint8).numpy(), expect["image"], err_msg=name)


def test_a_session_over_the_loaded_weights_matches_the_oracle_chain(loaded):
    weights, _ = loaded
    dims, tokens = weights.dims, 80
    stream = torch.cuda.current_stream()
    s = session.Session(stream, weights, tokens, LAYERS)
    s.set_attention(False)
    x, mods, cos, sin = session_oracle.make_inputs(dims, tokens, LAYERS, seed=5)
    x_t = torch.from_numpy(x.copy()).view(torch.bfloat16)
    s.run(stream, x_t, torch.from_numpy(mods), torch.from_numpy(cos), torch.from_numpy(sin))
    want, _ = session_oracle.oracle_forward(dims, session_oracle.host_weights(weights, LAYERS), x, mods)
    np.testing.assert_array_equal(x_t.view(torch.int16).numpy().view(np.uint16), want)
    s.close()


def test_a_checkpoint_of_another_block_shape_is_refused(tmp_path):
    """The file plans fine, but its fused row count is not what the kernels' block shape implies."""
    shape = dict(layers=1, hidden=2048, kv_heads=1, head_dim=128, inter=2048)
    tensors = plan_oracle.synthetic_blocks(np.random.default_rng(2), **shape)
    tensors["blocks.0.attn.wv.weight"] = np.concatenate([tensors["blocks.0.attn.wv.weight"]] * 2)
    tensors["blocks.0.attn.wv.weight_scale"] = np.concatenate([tensors["blocks.0.attn.wv.weight_scale"]] * 2)
    path = tmp_path / "odd.safetensors"
    plan_oracle.write_safetensors(str(path), tensors)
    assert Checkpoint(path).plan().layers == 1
    with pytest.raises(k.InvalidArgument):
        session.Weights.load(path)
