"""Generates tests/golden/rope_qknorm.npz from the reference's own torch QK-norm and rotary embedding.

Run once in a checkout that has the krea2-hrx sources beside it:
    python tests/golden/make_rope_golden.py /path/to/krea2-hrx

It imports `rms_norm`, `apply_rope`, `rope_tables` and `position_ids` from scripts/quantized_reference.py
unmodified and applies them as `Krea2Ref.attention` does (:211-214): q and k of a fused q|k|v row, bf16,
per-head zero-centred RMSNorm, then the interleaved-pair rotation, each returning bf16.  Eight query heads
and two key/value heads over 8 text + 4 x 6 image tokens keep the fixture small; the inputs are bf16 values
that f16 holds exactly, since the kernel reads the f16 output of the q|k|v|gate GEMM.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
Q_HEADS, KV_HEADS, HEAD_DIM, TEXT, GRID_H, GRID_W, SEED = 8, 2, 128, 8, 4, 6, 424242


def load(reference_root):
    path = os.path.join(reference_root, "scripts", "quantized_reference.py")
    spec = importlib.util.spec_from_file_location("quantized_reference", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules["quantized_reference"] = module
    spec.loader.exec_module(module)
    return module


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    ref = load(sys.argv[1])
    assert ref.HEAD_DIM == HEAD_DIM
    tokens = TEXT + GRID_H * GRID_W
    gen = torch.Generator().manual_seed(SEED)
    heads = Q_HEADS + 2 * KV_HEADS
    # magnitudes from 1/8 to 8 across heads so that the norm has something to do; exact in bf16 and in f16
    spread = torch.exp2(torch.randint(-3, 4, (1, heads, 1), generator=gen).float())
    fused = (torch.randn((tokens, heads, HEAD_DIM), generator=gen) * spread).to(torch.bfloat16)
    assert torch.equal(fused.float(), fused.float().to(torch.float16).float())
    q_scale = torch.randn(HEAD_DIM, generator=gen) * 0.1
    k_scale = torch.randn(HEAD_DIM, generator=gen) * 0.1
    cos, sin = ref.rope_tables(ref.position_ids(TEXT, GRID_H, GRID_W, "cpu"))
    q = fused[None, :, :Q_HEADS]
    k = fused[None, :, Q_HEADS:Q_HEADS + KV_HEADS]
    with torch.no_grad():
        q = ref.apply_rope(ref.rms_norm(q, q_scale), cos, sin)
        k = ref.apply_rope(ref.rms_norm(k, k_scale), cos, sin)
    out = {"fused": bits(fused.reshape(tokens, heads * HEAD_DIM)), "q_scale": q_scale.numpy(), "k_scale": k_scale.numpy(),
           "cos": cos.numpy(), "sin": sin.numpy(), "q": bits(q[0].reshape(tokens, -1)), "k": bits(k[0].reshape(tokens, -1))}
    np.savez_compressed(os.path.join(HERE, "rope_qknorm.npz"), **out)
    print({name: value.shape for name, value in out.items()})


if __name__ == "__main__":
    main()
