"""Builds libkrea2_b200.so from csrc/ with nvcc for sm_100a, in-tree."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libkrea2_b200.so")
SOURCES = ["api.cu", "prepare.cu", "gemm_i8.cu", "session.cu", "quantized.cu", "attention.cu", "sampler.cu", "checkpoint.cu"]
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-O2,-Wall", "--expt-relaxed-constexpr",
]


def nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise RuntimeError("nvcc not found; it is needed to build libkrea2_b200.so")


def stale() -> bool:
    if not os.path.exists(LIB):
        return True
    built = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)] + [os.path.join(HERE, "..", "include", "krea2_b200.h")]
    return any(os.path.getmtime(d) > built for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compiles every .cu of csrc/ (one object each, in parallel) and links the shared library."""
    if not force and not stale():
        return LIB
    out = os.path.join(HERE, "build")
    os.makedirs(out, exist_ok=True)
    compiler = nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []
    jobs = []
    for src in SOURCES:
        obj = os.path.join(out, src.replace(".cu", ".o"))
        cmd = [compiler, *FLAGS, *extra, "-c", os.path.join(CSRC, src), "-o", obj]
        jobs.append((src, obj, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    objects = []
    for src, obj, proc in jobs:
        log, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(log)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        objects.append(obj)
    subprocess.run([compiler, "-shared", "-o", LIB, *objects, "-lcudart"], check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
