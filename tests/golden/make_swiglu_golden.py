"""Generates tests/golden/swiglu_bf16.npz: the reference's own statement of the SwiGLU product.

Run once where torch is installed:
    python tests/golden/make_swiglu_golden.py

`Krea2Ref.swiglu` (scripts/quantized_reference.py:222-225) computes `F.silu(g) * u` on the bf16 outputs of the
gate and up projections: torch rounds the SiLU to bf16 and the product to bf16.  The fixture holds integer
accumulators whose dequantised values (channel scale 2^-15 for gate and 2^-8 for up columns, token scale 1)
are exactly the bf16 gate and up values -- every bf16 gate value with an exponent from -8 to 6, each paired with eight seeded up values below 128
in magnitude -- and torch's result as bf16 bits.
"""
import os

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    mantissas = np.arange(128, 256, dtype=np.int64)              # 8 significant bits: exact in bf16
    shifts = np.arange(0, 15, dtype=np.int64)                    # acc = m << s; value = acc / 2^15 -> exponents -8..6
    magnitudes = (mantissas[None, :] << shifts[:, None]).reshape(-1)
    gate_acc = np.concatenate([magnitudes, -magnitudes, [0]]).astype(np.int32)
    rng = np.random.Generator(np.random.PCG64(77))
    up_m = rng.integers(128, 256, size=(gate_acc.size, 8))
    up_s = rng.integers(0, 8, size=(gate_acc.size, 8))  # |u| < 128: products stay inside f16's range
    up_acc = ((up_m << up_s) * rng.choice([-1, 1], size=up_m.shape)).astype(np.int32)
    gate_acc = np.repeat(gate_acc[:, None], 8, axis=1)
    g = torch.from_numpy(gate_acc.astype(np.float32) / 32768).to(torch.bfloat16)
    u = torch.from_numpy(up_acc.astype(np.float32) / 256).to(torch.bfloat16)
    assert torch.equal(g.float() * 32768, torch.from_numpy(gate_acc.astype(np.float32)))
    assert torch.equal(u.float() * 256, torch.from_numpy(up_acc.astype(np.float32)))
    out = F.silu(g) * u
    np.savez_compressed(os.path.join(HERE, "swiglu_bf16.npz"), gate_acc=gate_acc, up_acc=up_acc,
                        product=out.view(torch.int16).numpy().view(np.uint16))
    print(gate_acc.shape, out.shape)


if __name__ == "__main__":
    main()
