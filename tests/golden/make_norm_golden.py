"""Generates tests/golden/norm_modulate.npz from the reference's own torch statement of RMSNorm + adaLN.

Run once in a checkout that has the krea2-hrx sources beside it:
    python tests/golden/make_norm_golden.py /path/to/krea2-hrx

It imports `rms_norm` from scripts/quantized_reference.py unmodified and evaluates the argument `Krea2Ref.block`
hands to its attention and its MLP (:265, :267): `(1.0 + prescale) * rms_norm(x, scale) + preshift` on bf16
tensors, the norm scale in f32.  Twelve rows of 6144 values with per-row magnitudes from 2^-6 to 2^5, one of them
all zero.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROWS, WIDTH = 12, 6144


def load(reference_root):
    path = os.path.join(reference_root, "scripts", "quantized_reference.py")
    spec = importlib.util.spec_from_file_location("quantized_reference", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules["quantized_reference"] = module
    spec.loader.exec_module(module)
    return module


def bits(t):
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    ref = load(sys.argv[1])
    gen = torch.Generator().manual_seed(31337)
    spread = torch.exp2(torch.arange(-6, 6).float())[:, None]
    x = (torch.randn((ROWS, WIDTH), generator=gen) * spread).to(torch.bfloat16)
    x[7] = 0
    scale = torch.randn(WIDTH, generator=gen) * 0.1
    prescale = (torch.randn(WIDTH, generator=gen) * 0.3).to(torch.bfloat16)
    preshift = (torch.randn(WIDTH, generator=gen) * 0.3).to(torch.bfloat16)
    with torch.no_grad():
        out = (1.0 + prescale) * ref.rms_norm(x, scale) + preshift
    np.savez_compressed(os.path.join(HERE, "norm_modulate.npz"), x=bits(x), scale=scale.numpy(), prescale=bits(prescale),
                        preshift=bits(preshift), out=bits(out))
    print(out.shape, out.dtype)


if __name__ == "__main__":
    main()
