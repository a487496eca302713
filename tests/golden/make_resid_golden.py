"""Generates tests/golden/resid_bf16.npz: the reference's own statement of the gated residual update.

Run once where torch is installed:
    python tests/golden/make_resid_golden.py

`Krea2Ref.block` (scripts/quantized_reference.py:262-268) updates the residual stream as `x + pregate * a` and
`x + postgate * f` on bf16 tensors: torch rounds the product to bf16 and the sum to bf16.  The fixture holds integer
accumulators whose dequantised values (channel scale 2^-12, token scale 1) are exactly the bf16 projection
outputs, seeded bf16 gates and prior residuals of mixed magnitudes (so that sums cancel, absorb and carry), and
torch's result as bf16 bits.
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
COLUMNS = 8192


def main():
    rng = np.random.Generator(np.random.PCG64(99))
    acc = ((rng.integers(128, 256, COLUMNS) << rng.integers(0, 16, COLUMNS)) * rng.choice([-1, 1], COLUMNS)).astype(np.int32)
    acc[:16] = 0
    a = torch.from_numpy(acc.astype(np.float32) / 4096).to(torch.bfloat16)
    assert torch.equal(a.float() * 4096, torch.from_numpy(acc.astype(np.float32)))
    gate = (torch.from_numpy(rng.standard_normal(COLUMNS).astype(np.float32)) * 0.5).to(torch.bfloat16)
    spread = torch.from_numpy(np.exp2(rng.integers(-6, 5, COLUMNS)).astype(np.float32))
    x = (torch.from_numpy(rng.standard_normal(COLUMNS).astype(np.float32)) * spread).to(torch.bfloat16)
    x[16:48] = -(gate[16:48] * a[16:48])  # exact cancellation
    out = x + gate * a
    bits = lambda t: t.view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "resid_bf16.npz"), acc=acc, gate=bits(gate), x=bits(x), out=bits(out))
    print(acc.shape, out.dtype)


if __name__ == "__main__":
    main()
