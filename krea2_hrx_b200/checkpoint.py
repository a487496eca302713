"""checkpoint::{Checkpoint, Plan} (src/checkpoint/file.rs, plan.rs) over the library's C entry points.

Everything here is host work: a checkpoint can be opened, planned and assembled without a GPU.
`session.Weights.load` uploads it.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import List, Tuple

import numpy as np

from ._lib import Dims, SpanInfo, check, lib


@dataclass(frozen=True)
class Segment:
    """Rows to copy from one checkpoint tensor (plan.rs:14-21)."""
    tensor: str
    rows: range


@dataclass(frozen=True)
class Span:
    """One destination on the device (plan.rs:23-43)."""
    device_offset: int
    device_bytes: int
    rows: int
    row_bytes: int
    device_row_bytes: int
    segments: Tuple[Segment, ...]
    file_bytes: int


class Checkpoint:
    """A mapped `.safetensors` file indexed under the transformer's tensor names."""

    def __init__(self, path: str):
        handle = ctypes.c_void_p()
        check(lib().krea2_checkpoint_open(str(path).encode(), ctypes.byref(handle)))
        self._handle, self.path = handle, str(path)

    def has(self, name: str) -> bool:
        return bool(lib().krea2_checkpoint_has(self._handle, name.encode()))

    def block_count(self) -> int:
        return int(lib().krea2_checkpoint_block_count(self._handle))

    def names(self) -> List[str]:
        count = lib().krea2_checkpoint_names(self._handle, None, 0)
        out = (ctypes.c_char_p * max(1, count))()
        lib().krea2_checkpoint_names(self._handle, out, count)
        return [out[i].decode() for i in range(count)]

    def get(self, name: str) -> Tuple[str, Tuple[int, ...], bytes]:
        """(dtype, shape, raw bytes) of a tensor (file.rs:103-109)."""
        dtype, shape, rank = ctypes.c_char_p(), ctypes.POINTER(ctypes.c_size_t)(), ctypes.c_size_t()
        data, count = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().krea2_checkpoint_tensor(self._handle, name.encode(), ctypes.byref(dtype), ctypes.byref(shape),
                                            ctypes.byref(rank), ctypes.byref(data), ctypes.byref(count)))
        return dtype.value.decode(), tuple(shape[i] for i in range(rank.value)), ctypes.string_at(data.value, count.value)

    def dims(self):
        """(ModelDims-like tuple, layers): the block shape the tensors declare."""
        dims, layers = Dims(), ctypes.c_size_t()
        check(lib().krea2_checkpoint_dims(self._handle, ctypes.byref(dims), ctypes.byref(layers)))
        return (dims.hidden, dims.kv_heads, dims.head_dim, dims.inter), layers.value

    def plan(self) -> "Plan":
        return Plan(self)

    def close(self) -> None:
        if getattr(self, "_handle", None):
            lib().krea2_checkpoint_close(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except TypeError:  # interpreter shutdown: the module globals are already gone
            pass


class Plan:
    """Plan::for_checkpoint (plan.rs:85-144): named spans in device order and the allocation they need."""

    def __init__(self, checkpoint: Checkpoint):
        total, layers, count = ctypes.c_size_t(), ctypes.c_size_t(), ctypes.c_size_t()
        check(lib().krea2_checkpoint_plan(checkpoint._handle, ctypes.byref(total), ctypes.byref(layers), ctypes.byref(count)))
        self._checkpoint = checkpoint
        self.total_bytes, self.layers = total.value, layers.value
        self.names = []
        for i in range(count.value):
            name = ctypes.c_char_p()
            check(lib().krea2_checkpoint_span_name(checkpoint._handle, i, ctypes.byref(name)))
            self.names.append(name.value.decode())

    def span(self, name: str) -> Span:
        info = SpanInfo()
        check(lib().krea2_checkpoint_span(self._checkpoint._handle, name.encode(), ctypes.byref(info)))
        segments = []
        for i in range(info.segments):
            tensor, begin, end = ctypes.c_char_p(), ctypes.c_size_t(), ctypes.c_size_t()
            check(lib().krea2_checkpoint_segment(self._checkpoint._handle, name.encode(), i, ctypes.byref(tensor),
                                                 ctypes.byref(begin), ctypes.byref(end)))
            segments.append(Segment(tensor.value.decode(), range(begin.value, end.value)))
        return Span(info.device_offset, info.device_bytes, info.rows, info.row_bytes, info.device_row_bytes,
                    tuple(segments), info.file_bytes)

    def assemble(self, name: str) -> np.ndarray:
        """The span as it lies on the device: rows at the device pitch, padding zero."""
        span = self.span(name)
        out = np.empty(span.device_bytes, dtype=np.uint8)
        check(lib().krea2_checkpoint_assemble(self._checkpoint._handle, name.encode(), out.ctypes.data, out.size))
        return out
