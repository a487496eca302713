"""The seeded synthetic transformer blocks behind tests/golden/block_w8a8.npz.

The weights (435 MB of int8 per block at the reference's dimensions) are too large to commit, so
the fixture holds only the inputs and the reference's outputs; the weights are regenerated from the
seed here, by the script that made the fixture and by the tests that use it alike.  numpy's PCG64
streams are the same on every platform.

Tensor names and shapes are the checkpoint's own (src/checkpoint/plan.rs:96-131,
scripts/quantized_reference.py:205-268): int8 rows `[N][K]` with f32 `weight_scale[N]`, zero-centred
norm scales.  Channel scales are drawn so that every linear layer's output has roughly unit
variance for unit-variance input, which keeps all branches of the block (attention, gate, SwiGLU,
residual adds) at comparable magnitudes, as in a trained model.
"""
from __future__ import annotations

from collections import OrderedDict

import numpy as np

HIDDEN, KV_HEADS, HEAD_DIM, INTER = 6144, 12, 128, 16384  # src/session/mod.rs:35-45
SEED, LAYERS = 20240611, 2
TEXT_TOKENS, GRID_H, GRID_W = 16, 4, 8
TOKENS = TEXT_TOKENS + GRID_H * GRID_W  # 48
# A second case over the same weights whose sequence spans several 128-key tiles of the attention kernel, the
# last one ragged: one block, and the fixture keeps a sample of the output rows.
LONG_GRID_H, LONG_GRID_W = 12, 16
LONG_TOKENS = TEXT_TOKENS + LONG_GRID_H * LONG_GRID_W  # 208
LONG_ROWS = sorted(set(range(0, LONG_TOKENS, 4)) | set(range(LONG_TOKENS - 8, LONG_TOKENS)) | {1, 15, 16, 17, 127, 129})


def block_tensors(layers: int = LAYERS, seed: int = SEED) -> "OrderedDict[str, np.ndarray]":
    tensors: "OrderedDict[str, np.ndarray]" = OrderedDict()
    kv = KV_HEADS * HEAD_DIM
    for block in range(layers):
        rng = np.random.Generator(np.random.PCG64([seed, block]))
        p = f"blocks.{block}"

        def linear(name, rows, k):
            tensors[f"{name}.weight"] = rng.integers(-127, 128, size=(rows, k), dtype=np.int8)
            unit = 1.0 / (np.sqrt(k) * 73.3)  # uniform codes in [-127, 127] have a standard deviation of 73.3
            tensors[f"{name}.weight_scale"] = (rng.uniform(0.5, 1.5, size=rows) * unit).astype(np.float32)

        def norm(name, n):
            tensors[name] = (rng.standard_normal(n) * 0.1).astype(np.float32)

        linear(f"{p}.attn.wq", HIDDEN, HIDDEN)
        linear(f"{p}.attn.wk", kv, HIDDEN)
        linear(f"{p}.attn.wv", kv, HIDDEN)
        linear(f"{p}.attn.gate", HIDDEN, HIDDEN)
        linear(f"{p}.attn.wo", HIDDEN, HIDDEN)
        linear(f"{p}.mlp.gate", INTER, HIDDEN)
        linear(f"{p}.mlp.up", INTER, HIDDEN)
        linear(f"{p}.mlp.down", HIDDEN, INTER)
        norm(f"{p}.prenorm.scale", HIDDEN)
        norm(f"{p}.postnorm.scale", HIDDEN)
        norm(f"{p}.attn.qknorm.qnorm.scale", HEAD_DIM)
        norm(f"{p}.attn.qknorm.knorm.scale", HEAD_DIM)
    return tensors


def bf16_round(values: np.ndarray) -> np.ndarray:
    """f32 values rounded to the nearest bf16 (ties to even), still as f32."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return rounded.astype(np.uint32).view(np.float32)


def block_inputs(layers: int = LAYERS, seed: int = SEED, tokens: int = TOKENS, stream: int = 1000):
    """x (f32 holding bf16 values, [tokens][HIDDEN]) and the per-block modulation (f32 holding bf16
    values, [layers][6][HIDDEN]: prescale, preshift, pregate, postscale, postshift, postgate)."""
    rng = np.random.Generator(np.random.PCG64([seed, stream]))
    x = bf16_round(rng.standard_normal((tokens, HIDDEN)).astype(np.float32))
    mods = (rng.standard_normal((layers, 6, HIDDEN)) * 0.3).astype(np.float32)
    return x, bf16_round(mods)


def oracle_blocks(tensors, layers: int = LAYERS):
    """The tensors laid out as the device holds them (oracle/plan.py), keyed as session_oracle.oracle_forward
    reads them."""
    from oracle import plan as plan_oracle
    spans, _ = plan_oracle.plan(tensors, layers)
    out = []
    for block in range(layers):
        p = f"blocks.{block}."
        entry = {}
        for name in ("qkvg", "wo", "gu", "down"):
            entry[f"{name}.q"] = spans[f"{p}{name}.q"]["image"].view(np.int8)
            entry[f"{name}.s"] = spans[f"{p}{name}.s"]["image"].view(np.float32)
        for name in ("prenorm", "postnorm", "qnorm", "knorm"):
            entry[name] = spans[f"{p}{name}"]["image"].view(np.float32)
        out.append(entry)
    return out


def long_inputs():
    """The inputs of the several-tile case: 208 tokens, one block."""
    return block_inputs(layers=1, tokens=LONG_TOKENS, stream=1001)


def modulation_inputs(layers: int = LAYERS, seed: int = SEED):
    """The time model's modulation vector (f32 holding bf16 values, [6 * HIDDEN]) and the blocks' tables
    `blocks.N.mod.lin` ([layers][6 * HIDDEN]) that `Krea2Ref.block_modulation` adds to it."""
    rng = np.random.Generator(np.random.PCG64([seed, 1002]))
    vector = bf16_round((rng.standard_normal(6 * HIDDEN) * 0.2).astype(np.float32))
    tables = bf16_round((rng.standard_normal((layers, 6 * HIDDEN)) * 0.2).astype(np.float32))
    return vector, tables
