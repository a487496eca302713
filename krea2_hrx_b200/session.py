"""krea2::session (src/session/mod.rs, weights.rs): the resident block session, over the C ABI."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ._lib import Dims, InvalidArgument, check, lib

# src/session/mod.rs:35-45
HIDDEN, KV_HEADS, HEAD_DIM, INTER = 6144, 12, 128, 16384
QKVG = HIDDEN + 2 * KV_HEADS * HEAD_DIM + HIDDEN
GATE_OFFSET = HIDDEN + 2 * KV_HEADS * HEAD_DIM


@dataclass(frozen=True)
class ModelDims:
    hidden: int = HIDDEN
    kv_heads: int = KV_HEADS
    head_dim: int = HEAD_DIM
    inter: int = INTER

    @property
    def qkvg(self) -> int:
        return 2 * self.hidden + 2 * self.kv_heads * self.head_dim

    @property
    def gate_offset(self) -> int:
        return self.hidden + 2 * self.kv_heads * self.head_dim

    def c(self) -> Dims:
        return Dims(self.hidden, self.kv_heads, self.head_dim, self.inter)


def _stream_ptr(stream) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


class Weights:
    """session::Weights (src/session/weights.rs:17-126): one device allocation, spans by name."""

    def __init__(self, dims: ModelDims = ModelDims(), layers: int = 28):
        self.dims, self.layers = dims, layers
        handle = ctypes.c_void_p()
        c_dims = dims.c()
        check(lib().krea2_weights_create(ctypes.byref(c_dims), layers, ctypes.byref(handle)))
        self._handle = handle

    @classmethod
    def load(cls, path, stream=None) -> "Weights":
        """Weights::load (src/session/weights.rs:40-44): reads the checkpoint, derives the layout, uploads it."""
        from .checkpoint import Checkpoint
        checkpoint = Checkpoint(path)
        try:
            (hidden, kv_heads, head_dim, inter), layers = checkpoint.dims()
            handle = ctypes.c_void_p()
            check(lib().krea2_weights_load_checkpoint(checkpoint._handle, _stream_ptr(stream), ctypes.byref(handle)))
        finally:
            checkpoint.close()
        self = cls.__new__(cls)
        self.dims, self.layers = ModelDims(hidden=hidden, kv_heads=kv_heads, head_dim=head_dim, inter=inter), layers
        self._handle = handle
        return self

    @staticmethod
    def plan_bytes(dims: ModelDims, layers: int) -> int:
        n = ctypes.c_size_t()
        c_dims = dims.c()
        check(lib().krea2_weights_plan_bytes(ctypes.byref(c_dims), layers, ctypes.byref(n)))
        return n.value

    def fill_synthetic(self, seed: int, stream=None) -> None:
        check(lib().krea2_weights_fill_synthetic(self._handle, seed, _stream_ptr(stream)))

    def locate(self, name: str) -> Tuple[int, int]:
        """(device address, bytes) of a span such as "blocks.3.qkvg.q" (weights.rs:112-125)."""
        ptr, n = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().krea2_weights_locate(self._handle, name.encode(), ctypes.byref(ptr), ctypes.byref(n)))
        return ptr.value, n.value

    def read(self, name: str, dtype: torch.dtype) -> torch.Tensor:
        """A host copy of one span (for tests that feed the same weights to the CPU oracle)."""
        ptr, n = self.locate(name)
        out = torch.empty(n // torch.empty((), dtype=dtype).element_size(), dtype=dtype)
        check(lib().krea2_weights_download(self._handle, name.encode(), out.data_ptr(), n, _stream_ptr(None)))
        return out

    def upload(self, name: str, host: torch.Tensor, stream=None) -> None:
        host = host.contiguous()
        check(lib().krea2_weights_upload(self._handle, name.encode(), host.data_ptr(),
                                         host.numel() * host.element_size(), _stream_ptr(stream)))

    def __del__(self):
        try:
            if getattr(self, "_handle", None):
                lib().krea2_weights_release(self._handle)
                self._handle = None
        except TypeError:  # interpreter shutdown: the module globals are already gone
            pass


def validate(checkpoint_path, tokens: int, layers: int) -> None:
    """Session::validate (src/session/mod.rs:249-261): raises InvalidArgument for dimensions this build cannot
    serve or a checkpoint that cannot be laid out, without touching a device."""
    check(lib().krea2_session_validate(str(checkpoint_path).encode(), tokens, layers))


class Session:
    """session::Session: buffers sized by shape::capacity, bound to its creating stream."""

    def __init__(self, stream: Optional[torch.cuda.Stream], weights: Weights, tokens: int, layers: int):
        self.stream = stream or torch.cuda.current_stream()
        self.weights = weights
        handle = ctypes.c_void_p()
        check(lib().krea2_session_create(self.stream.cuda_stream, weights._handle, tokens, layers,
                                         ctypes.byref(handle)))
        self._handle = handle

    @staticmethod
    def validate_dimensions(tokens: int, layers: int) -> None:
        """Session::validate_dimensions (mod.rs:278-287): touches no device."""
        check(lib().krea2_session_validate_dimensions(tokens, layers))

    @classmethod
    def with_weights(cls, stream, weights: Weights, tokens: int, layers: int) -> "Session":
        return cls(stream, weights, tokens, layers)

    def tokens(self) -> int:
        return lib().krea2_session_tokens(self._handle)

    def layers(self) -> int:
        return lib().krea2_session_layers(self._handle)

    def set_profile(self, enable: bool) -> bool:
        return bool(lib().krea2_session_set_profile(self._handle, int(enable)))

    def set_attention(self, enable: bool) -> bool:
        """Full block (True) or the W8A8 chain alone, the query columns in the attention output's place (False)."""
        return bool(lib().krea2_session_set_attention(self._handle, int(enable)))

    def set_fused_rotation(self, enable: bool) -> bool:
        """The SwiGLU output's hand-off to the down projection: the reference's two launches (False) or the fused
        pair whose GEMM epilogue starts the prologue's rotation (True); the same bits either way."""
        return bool(lib().krea2_session_set_fused_rotation(self._handle, int(enable)))

    def set_fused_rope(self, enable: bool) -> bool:
        """Whether the q|k|v|gate GEMM also does the QK-norm + RoPE launch's work (ten launches per block instead
        of eleven, attention on only); the same bits either way."""
        return bool(lib().krea2_session_set_fused_rope(self._handle, int(enable)))

    def stage_profile(self) -> List[Tuple[str, float]]:
        labels = (ctypes.c_char_p * 16)()
        millis = (ctypes.c_double * 16)()
        n = lib().krea2_session_stage_profile(self._handle, labels, millis, 16)
        return [(labels[i].decode(), millis[i]) for i in range(n)]

    def launches_per_forward(self) -> int:
        return lib().krea2_session_launches_per_forward(self._handle)

    def run(self, stream, x: torch.Tensor, mods: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
            first_block: int = 0, block_count: Optional[int] = None) -> None:
        """Session::run (mod.rs:502-540): HOST tensors; x (bf16 [tokens][hidden]) is updated in place."""
        for t in (x, mods, cos, sin):
            if t.is_cuda or not t.is_contiguous():
                raise InvalidArgument("Session.run takes contiguous host tensors")
        if x.numel() != self.tokens() * self.weights.dims.hidden:
            raise InvalidArgument(f"x has {x.numel()} elements, expected {self.tokens() * self.weights.dims.hidden}")
        if mods.numel() != self.layers() * 6 * self.weights.dims.hidden:
            raise InvalidArgument("mods has the wrong element count")
        if cos.numel() != self.tokens() * self.weights.dims.head_dim or sin.numel() != cos.numel():
            raise InvalidArgument("cos/sin have the wrong element count")
        check(lib().krea2_session_run(self._handle, (stream or self.stream).cuda_stream, x.data_ptr(), mods.data_ptr(),
                                      cos.data_ptr(), sin.data_ptr(), first_block, block_count or 0))

    def run_device(self, stream, x: torch.Tensor, mods: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> None:
        """Session::run_device (mod.rs:553-588): DEVICE x (bf16 [tokens][hidden], updated in place) and mods (f32
        [layers][6][hidden]), HOST cos/sin (f32 [tokens][head_dim]; the library fingerprints them on the host and
        uploads them only when they change); graph replay, asynchronous."""
        dims = self.weights.dims
        for t in (cos, sin):
            if t.is_cuda or not t.is_contiguous() or t.dtype != torch.float32:
                raise InvalidArgument("Session.run_device takes cos/sin as contiguous float32 host tensors")
        if cos.numel() != self.tokens() * dims.head_dim or sin.numel() != cos.numel():
            raise InvalidArgument("cos/sin have the wrong element count")
        if not x.is_cuda or not x.is_contiguous() or x.dtype != torch.bfloat16 or x.numel() != self.tokens() * dims.hidden:
            raise InvalidArgument("Session.run_device takes x as a contiguous CUDA bfloat16 [tokens][hidden] tensor")
        if not mods.is_cuda or not mods.is_contiguous() or mods.dtype != torch.float32 \
                or mods.numel() != self.layers() * 6 * dims.hidden:
            raise InvalidArgument("Session.run_device takes mods as a contiguous CUDA float32 [layers][6][hidden] tensor")
        check(lib().krea2_session_run_device(self._handle, (stream or self.stream).cuda_stream, x.data_ptr(),
                                             x.numel() * x.element_size(), mods.data_ptr(),
                                             mods.numel() * mods.element_size(), cos.data_ptr(), sin.data_ptr()))

    def buffer(self, name: str) -> Tuple[int, int]:
        ptr, n = ctypes.c_void_p(), ctypes.c_size_t()
        check(lib().krea2_session_buffer(self._handle, name.encode(), ctypes.byref(ptr), ctypes.byref(n)))
        return ptr.value, n.value

    def close(self) -> None:
        if getattr(self, "_handle", None):
            lib().krea2_session_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except TypeError:  # interpreter shutdown: the module globals are already gone
            pass
