"""Records the reference's scheduler oracle for the sigma-schedule tests.

Run once in a checkout that has the krea2-hrx sources beside it:

    python tests/golden/make_schedule_golden.py /path/to/krea2-hrx

The reference holds 36,050 recorded scheduler sigmas (tests/fixtures/sigmas.f32le; layout in
tests/fixtures/README.md and tests/schedule.rs:6-20: image-token counts 0 (the fixed shift 1.15), 16,
256, 589, 4096, 6400, 16384, then step counts 1..100, each grid with its terminal zero).  This script
stores the SHA-256 of that whole stream, so a test can hold every one of the values bit for bit by
regenerating the stream, and a readable subset of the grids (the step counts in SUBSET_STEPS).
"""
import hashlib
import os
import sys

import numpy as np

TOKENS = [0, 16, 256, 589, 4096, 6400, 16384]
SUBSET_STEPS = [1, 2, 3, 4, 8, 20, 28, 50, 52, 100]


def main() -> None:
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    root = sys.argv[1]
    raw = open(os.path.join(root, "tests", "fixtures", "sigmas.f32le"), "rb").read()
    bits = np.frombuffer(raw, dtype="<u4")
    subset, cursor = {}, 0
    for tokens in TOKENS:
        for steps in range(1, 101):
            grid = bits[cursor:cursor + steps + 1]
            cursor += steps + 1
            if steps in SUBSET_STEPS:
                subset[f"t{tokens}_s{steps}"] = grid.copy()
    assert cursor == bits.size == 36050
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "schedule_sigmas.npz")
    np.savez_compressed(out, sha256=np.frombuffer(hashlib.sha256(raw).digest(), dtype=np.uint8),
                        count=np.array([bits.size]), tokens=np.array(TOKENS), **subset)
    print(out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
