"""Generates tests/golden/quantlinear_*.npz from the reference's own torch W8A8 scheme.

Run once in a checkout that has the krea2-hrx sources beside it:
    python tests/golden/make_quantlinear_golden.py /path/to/krea2-hrx

It imports `hadamard`, `rotate_groups`, `quant_rows` and `QuantLinear` from
scripts/quantized_reference.py (:76-125) unmodified and records, for seeded inputs,
the rotated activations, the per-token codes and scales, the f32 accumulator and the
f16 output.  The scheme rotates with a dense normalised matrix in f32 and has no bf16
rounding points, so it is a TOLERANCE reference for the kernels (the reference measures
0.0117 relative RMS between the two over a forward), not a bit reference.
"""
import importlib.util
import os
import sys

import numpy as np
import torch


def load(reference_root):
    path = os.path.join(reference_root, "scripts", "quantized_reference.py")
    spec = importlib.util.spec_from_file_location("quantized_reference", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules["quantized_reference"] = module
    spec.loader.exec_module(module)
    return module


def case(ref, seed, m, k, n):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((m, k)).astype(np.float32)
    outliers = rng.choice(k, size=max(1, k // 100), replace=False)
    x[:, outliers] *= 20.0
    x16 = torch.from_numpy(x).to(torch.float16)
    w = torch.from_numpy(rng.integers(-127, 128, size=(n, k), dtype=np.int64).astype(np.int8))
    ws = torch.from_numpy(rng.uniform(1e-3, 1e-2, size=(n, 1)).astype(np.float32))
    h = ref.hadamard(ref.HADAMARD_GROUP)
    layer = ref.QuantLinear(w, ws, h, 127)
    rotated = ref.rotate_groups(x16.float(), h)
    codes, scales = ref.quant_rows(rotated, 127)
    out = layer(x16)
    return dict(x=x16.numpy().view(np.uint16), w=w.numpy(), ws=ws.numpy().reshape(-1),
                hadamard=h.numpy(), codes=codes.numpy().astype(np.int8), scales=scales.numpy().reshape(-1),
                out=out.numpy().view(np.uint16))


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    ref = load(sys.argv[1])
    here = os.path.dirname(os.path.abspath(__file__))
    torch.manual_seed(0)
    for name, (seed, m, k, n) in {"small": (11, 8, 2048, 64), "hidden": (12, 4, 6144, 32)}.items():
        np.savez_compressed(os.path.join(here, f"quantlinear_{name}.npz"), **case(ref, seed, m, k, n))


if __name__ == "__main__":
    main()
