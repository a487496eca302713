"""numpy restatement of the checkpoint's device layout (src/checkpoint/plan.rs), and a writer for
small synthetic `.safetensors` files to feed it.

TEST INFRASTRUCTURE ONLY: used by tests/ to check the library's checkpoint reader and loader.
"""
from __future__ import annotations

import json
from collections import OrderedDict
from typing import Dict, List, Tuple

import numpy as np

DTYPES = {np.dtype(np.int8): "I8", np.dtype(np.float32): "F32", np.dtype(np.uint16): "BF16"}


def gemm_pitch(k: int) -> int:
    """src/kernels/shape.rs:24-30: rows whose bytes are a multiple of 8192 take 64 bytes of padding."""
    return k + 64 if k % 8192 == 0 else k


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], metadata=None, prefix: str = "") -> None:
    """The public container format: u64 little-endian header length, JSON header, tensor bytes.
    uint16 arrays are stored as BF16."""
    header, payload, cursor = OrderedDict(), [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, array in tensors.items():
        raw = np.ascontiguousarray(array).tobytes()
        header[prefix + name] = {"dtype": DTYPES[array.dtype], "shape": list(array.shape), "data_offsets": [cursor, cursor + len(raw)]}
        payload.append(raw)
        cursor += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(len(text).to_bytes(8, "little"))
        f.write(text)
        for raw in payload:
            f.write(raw)


def synthetic_blocks(rng, layers: int, hidden: int, kv_heads: int, head_dim: int, inter: int, bf16_norms=False):
    """Seeded tensors under the checkpoint's own names (plan.rs:96-131), int8 rows with f32 row scales."""
    tensors: "OrderedDict[str, np.ndarray]" = OrderedDict()

    def linear(name, rows, k):
        tensors[f"{name}.weight"] = rng.integers(-127, 128, size=(rows, k), dtype=np.int8)
        tensors[f"{name}.weight_scale"] = rng.uniform(1e-3, 1e-2, size=rows).astype(np.float32)

    def norm(name, n):
        v = (rng.standard_normal(n) * 0.1).astype(np.float32)
        tensors[name] = (v.view(np.uint32) >> 16).astype(np.uint16) if bf16_norms else v

    kv = kv_heads * head_dim
    for block in range(layers):
        p = f"blocks.{block}"
        linear(f"{p}.attn.wq", hidden, hidden)
        linear(f"{p}.attn.wk", kv, hidden)
        linear(f"{p}.attn.wv", kv, hidden)
        linear(f"{p}.attn.gate", hidden, hidden)
        linear(f"{p}.attn.wo", hidden, hidden)
        linear(f"{p}.mlp.gate", inter, hidden)
        linear(f"{p}.mlp.up", inter, hidden)
        linear(f"{p}.mlp.down", hidden, inter)
        norm(f"{p}.prenorm.scale", hidden)
        norm(f"{p}.postnorm.scale", hidden)
        norm(f"{p}.attn.qknorm.qnorm.scale", head_dim)
        norm(f"{p}.attn.qknorm.knorm.scale", head_dim)
    return tensors


def operand(tensors, parts: List[str], group: int) -> Tuple[np.ndarray, np.ndarray, List[Tuple[str, int, int]]]:
    """plan.rs:150-232: (device image of the rows, gathered scales, segments)."""
    weights = [tensors[f"{part}.weight"] for part in parts]
    scales = [tensors[f"{part}.weight_scale"] for part in parts]
    k = weights[0].shape[1]
    pieces, scale_pieces, segments = [], [], []
    if group == 0:
        for part, w, s in zip(parts, weights, scales):
            pieces.append(w)
            scale_pieces.append(s)
            segments.append((f"{part}.weight", 0, w.shape[0]))
    else:
        for start in range(0, weights[0].shape[0], group):
            for part, w, s in zip(parts, weights, scales):
                pieces.append(w[start:start + group])
                scale_pieces.append(s[start:start + group])
                segments.append((f"{part}.weight", start, start + group))
    rows = np.concatenate(pieces, axis=0)
    image = np.zeros((rows.shape[0], gemm_pitch(k)), dtype=np.int8)
    image[:, :k] = rows
    return image, np.concatenate(scale_pieces).astype(np.float32), segments


def vector(tensors, name: str) -> np.ndarray:
    """plan.rs:234-268: f32 as stored, bf16 widened exactly."""
    v = tensors[name]
    return (v.astype(np.uint32) << 16).view(np.float32) if v.dtype == np.uint16 else v


def plan(tensors, layers: int):
    """plan.rs:85-144 -> (OrderedDict name -> dict(offset, image bytes, segments, rows, row_bytes, pitch), total)."""
    spans = {}
    for block in range(layers):
        p = f"blocks.{block}"
        for out, parts, group in ((f"{p}.qkvg", [f"{p}.attn.wq", f"{p}.attn.wk", f"{p}.attn.wv", f"{p}.attn.gate"], 0),
                                  (f"{p}.wo", [f"{p}.attn.wo"], 0), (f"{p}.down", [f"{p}.mlp.down"], 0),
                                  (f"{p}.gu", [f"{p}.mlp.gate", f"{p}.mlp.up"], 16)):
            image, scales, segments = operand(tensors, parts, group)
            k = tensors[f"{parts[0]}.weight"].shape[1]
            spans[f"{out}.q"] = dict(image=image.view(np.uint8).ravel(), segments=segments, rows=image.shape[0], row_bytes=k,
                                     pitch=image.shape[1])
            spans[f"{out}.s"] = dict(image=scales.view(np.uint8).ravel(), segments=[], rows=0, row_bytes=0, pitch=0)
        for out, name in (("prenorm", f"{p}.prenorm.scale"), ("postnorm", f"{p}.postnorm.scale"),
                          ("qnorm", f"{p}.attn.qknorm.qnorm.scale"), ("knorm", f"{p}.attn.qknorm.knorm.scale")):
            v = vector(tensors, name)
            host = tensors[name].dtype == np.uint16
            spans[f"{p}.{out}"] = dict(image=v.view(np.uint8).ravel(), segments=[] if host else [(name, 0, 1)],
                                       rows=0 if host else 1, row_bytes=0 if host else v.nbytes, pitch=0 if host else v.nbytes)
    ordered, total = OrderedDict(), 0
    for name in sorted(spans, key=lambda n: n.encode()):
        span = spans[name]
        span["offset"] = total
        total += -(-span["image"].size // 256) * 256
        ordered[name] = span
    return ordered, total
