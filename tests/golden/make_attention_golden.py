"""Generates tests/golden/attention_sdpa.npz: the reference's own statement of grouped-query attention.

Run once where torch is installed:
    python tests/golden/make_attention_golden.py

`Krea2Ref.attention` (scripts/quantized_reference.py:215-218) repeats each key/value head over its group of query
heads and calls `F.scaled_dot_product_attention` on bf16 tensors.  The inputs are seeded (numpy PCG64, so the tests
regenerate them): 208 tokens -- two 128-key tiles of the kernel, the second ragged -- eight query heads over two
key/value heads, values rounded to bf16 of a magnitude f16 holds exactly.  The fixture keeps torch's bf16 output.
"""
import os

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
TOKENS, Q_HEADS, KV_HEADS, HEAD_DIM, SEED = 208, 8, 2, 128, 909


def inputs():
    """q [tokens][q_heads*128], k, v [tokens][kv_heads*128] as f32 holding bf16 values."""
    rng = np.random.Generator(np.random.PCG64(SEED))

    def bf16(a):
        bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(np.float32)
        return np.where(np.abs(rounded) < 2.0 ** -10, np.float32(0), rounded)  # what is left is exact in f16
    q = bf16(rng.standard_normal((TOKENS, Q_HEADS * HEAD_DIM)) * 1.5)
    k = bf16(rng.standard_normal((TOKENS, KV_HEADS * HEAD_DIM)) * 1.5)
    v = bf16(rng.standard_normal((TOKENS, KV_HEADS * HEAD_DIM)))
    return q, k, v


def main():
    q, k, v = (torch.from_numpy(a).to(torch.bfloat16) for a in inputs())
    q = q.view(1, TOKENS, Q_HEADS, HEAD_DIM)
    k = k.view(1, TOKENS, KV_HEADS, HEAD_DIM).repeat_interleave(Q_HEADS // KV_HEADS, dim=2)
    v = v.view(1, TOKENS, KV_HEADS, HEAD_DIM).repeat_interleave(Q_HEADS // KV_HEADS, dim=2)
    with torch.no_grad():
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
    out = o.reshape(TOKENS, Q_HEADS * HEAD_DIM).contiguous().view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(os.path.join(HERE, "attention_sdpa.npz"), out=out)
    print(out.shape)


if __name__ == "__main__":
    main()
