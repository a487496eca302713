"""Generates tests/golden/gate_attention.npz: the reference's own statement of the attention output gate.

Run once where torch is installed:
    python tests/golden/make_gate_golden.py

`Krea2Ref.attention` (scripts/quantized_reference.py:219) computes `o * torch.sigmoid(gate)` on bf16 tensors: torch
rounds the sigmoid to bf16 and the product to bf16.  The fixture holds every bf16 gate value with an exponent from
-8 to 6 (and zero), each against four seeded bf16 attention values; all inputs are exact in f16, which is what the
kernel reads.
"""
import os

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    mantissas = np.arange(128, 256, dtype=np.float64)
    magnitudes = (mantissas[None, :] * np.exp2(np.arange(-15, 0, dtype=np.float64))[:, None]).reshape(-1)  # 2^-8 .. 127.5
    gate = np.repeat(np.concatenate([magnitudes, -magnitudes, [0.0]])[:, None], 4, axis=1).astype(np.float32)
    rng = np.random.Generator(np.random.PCG64(55))
    attn = (rng.standard_normal(gate.shape) * np.exp2(rng.integers(-4, 3, gate.shape))).astype(np.float32)
    g, o = torch.from_numpy(gate).to(torch.bfloat16), torch.from_numpy(attn).to(torch.bfloat16)
    assert torch.equal(g.float(), torch.from_numpy(gate)) and torch.equal(g.float(), g.float().to(torch.float16).float())
    assert torch.equal(o.float(), o.float().to(torch.float16).float())
    out = o * torch.sigmoid(g)
    bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "gate_attention.npz"), gate=bits(g), attn=bits(o), out=bits(out))
    print(out.shape)


if __name__ == "__main__":
    main()
