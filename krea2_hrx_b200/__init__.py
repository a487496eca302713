"""krea2_hrx_b200: the W8A8 linear-layer path of krea2-hrx, hand-written for NVIDIA B200 (sm_100a).

The compute lives in libkrea2_b200.so (CUDA, built from csrc/ by build.py) behind the C ABI of
include/krea2_b200.h.  The modules here mirror the reference crate's host interface for this path:
`shape` (kernels::shape), `kernels` (Config, Scalars, Shape), `ops` (Ops::launch, Quantized, the pointwise
sampler kernels), `session` (Session, Weights), `schedule` (pipeline::schedule), `checkpoint` (Checkpoint, Plan)
`pipeline` (the denoising loop of Pipeline::generate around a session) and `parallel` (weights or tokens
sharded over several devices, which the reference does not have).
"""
from . import kernels, shape  # noqa: F401
from ._lib import (Cancelled, Error, Internal, InvalidArgument, Poisoned, Runtime, device_status, lib)  # noqa: F401

__all__ = ["kernels", "shape", "ops", "session", "schedule", "checkpoint", "parallel", "pipeline", "lib", "device_status", "Error", "InvalidArgument", "Cancelled",
           "Poisoned", "Runtime", "Internal"]


def __getattr__(name):
    # ops and session import torch; keep `import krea2_hrx_b200` light for the shape rules.
    if name in ("ops", "session", "schedule", "checkpoint", "parallel", "pipeline"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
