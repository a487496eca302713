"""krea2::ops::Ops::launch / launch_1d (src/ops/mod.rs:673-713) and the typed kernel calls.

Buffers are torch CUDA tensors (device memory and streams are torch's; the arithmetic is not):
each call passes raw device pointers through the C ABI of libkrea2_b200.so.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import kernels, shape
from ._lib import Binding, ConfigEntry, InvalidArgument, check, lib


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def _ptr(t: torch.Tensor) -> int:
    if not t.is_cuda:
        raise InvalidArgument("buffers must live on a CUDA device")
    if not t.is_contiguous():
        raise InvalidArgument("buffers must be contiguous")
    return t.data_ptr()


def _bytes(t: torch.Tensor) -> int:
    return t.numel() * t.element_size()


FLOAT_SCALARS = {"euler": "delta", "guidance": "scale"}


class Ops:
    """The generic dispatcher: kernel by name, config by key, scalars, buffers in binding order."""

    def launch(self, stream, name: str, config: kernels.Config, scalars: kernels.Scalars,
               bindings: Sequence[torch.Tensor], grid_x: int, grid_y: int, threads: int) -> None:
        kernels.grid(name, grid_x, grid_y)
        if scalars.floats and name in FLOAT_SCALARS:  # Scalars::float: the C ABI carries it as a config float
            config = {**config, FLOAT_SCALARS[name]: float(scalars.floats[0])}
        entries = (ConfigEntry * max(1, len(config)))()
        for i, (key, value) in enumerate(config.items()):
            entries[i].key = key.encode()
            if isinstance(value, float):
                entries[i].fvalue = value
            else:
                entries[i].value = int(value)
                entries[i].fvalue = float(value)
        indices = (ctypes.c_uint64 * max(1, len(scalars.indices)))(*scalars.indices)
        binds = (Binding * max(1, len(bindings)))()
        for i, t in enumerate(bindings):
            binds[i].ptr = _ptr(t)
            binds[i].bytes = _bytes(t)
        check(lib().krea2_launch(_stream_ptr(stream), name.encode(), entries, len(config), indices,
                                 len(scalars.indices), binds, len(bindings), grid_x, grid_y, threads))

    def launch_1d(self, stream, name, config, scalars, bindings, elements: int) -> None:
        """One 256-thread workgroup per 256 elements (src/ops/mod.rs:701-713)."""
        self.launch(stream, name, config, scalars, bindings, -(-elements // 256), 1, 256)


# ------------------------------------------------------------------ typed calls (C ABI order)
def prepare_norm_i8(h, norm_scale, mod_scale, mod_shift, q, q_scale, width, out_stride, eps=1e-5, stream=None):
    check(lib().krea2_prepare_norm_i8(_stream_ptr(stream), h.shape[0], _ptr(h), _ptr(norm_scale), _ptr(mod_scale),
                                      _ptr(mod_shift), _ptr(q), _ptr(q_scale), width, out_stride, eps))


def prepare_gated_i8(attn, gate, q, q_scale, width, out_stride, gate_stride, stream=None, tokens=None):
    tokens = attn.shape[0] if tokens is None else tokens
    check(lib().krea2_prepare_gated_i8(_stream_ptr(stream), tokens, _ptr(attn), gate.data_ptr(), _ptr(q),
                                       _ptr(q_scale), width, out_stride, gate_stride))


def prepare_plain_i8(h, q, q_scale, width, out_stride, stream=None):
    check(lib().krea2_prepare_plain_i8(_stream_ptr(stream), h.shape[0], _ptr(h), _ptr(q), _ptr(q_scale), width,
                                       out_stride))


def gemm_i8_256(m, a, w, scale, a_scale, c, k_size, k_stride, n_size, m_group=4, stream=None):
    check(lib().krea2_gemm_i8_256(_stream_ptr(stream), m, _ptr(a), _ptr(w), _ptr(scale), _ptr(a_scale), _ptr(c),
                                  k_size, k_stride, n_size, m_group))


def gemm_i8_resid_256(m, a, w, scale, a_scale, c, gate, k_size, k_stride, n_size, m_group=4, stream=None):
    check(lib().krea2_gemm_i8_resid_256(_stream_ptr(stream), m, _ptr(a), _ptr(w), _ptr(scale), _ptr(a_scale),
                                        _ptr(c), _ptr(gate), k_size, k_stride, n_size, m_group))


def gemm_i8_resid_256x256(m, a, w, scale, a_scale, c, gate, k_size, k_stride, n_size, m_group=4, schedule_rows=0,
                          stream=None):
    check(lib().krea2_gemm_i8_resid_256x256(_stream_ptr(stream), m, _ptr(a), _ptr(w), _ptr(scale), _ptr(a_scale),
                                            _ptr(c), _ptr(gate), k_size, k_stride, n_size, m_group,
                                            int(schedule_rows)))


def gemm_i8_swiglu_256(m, a, w, scale, a_scale, c, k_size, k_stride, n_size, m_group=4, stream=None):
    check(lib().krea2_gemm_i8_swiglu_256(_stream_ptr(stream), m, _ptr(a), _ptr(w), _ptr(scale), _ptr(a_scale),
                                         _ptr(c), k_size, k_stride, n_size, m_group))


def gemm_i8_swiglu_rotated_256(m, a, w, scale, a_scale, c, k_size, k_stride, n_size, m_group=4, stream=None):
    """gemm_i8_swiglu_256 whose epilogue also applies the first three rotation stages of prepare_plain_i8."""
    check(lib().krea2_gemm_i8_swiglu_rotated_256(_stream_ptr(stream), m, _ptr(a), _ptr(w), _ptr(scale), _ptr(a_scale),
                                                 _ptr(c), k_size, k_stride, n_size, m_group))


def prepare_rotated_i8(h, q, q_scale, width, out_stride, stream=None):
    """The rest of prepare_plain_i8 (last stage, row maximum, codes) on a row gemm_i8_swiglu_rotated_256 wrote."""
    check(lib().krea2_prepare_rotated_i8(_stream_ptr(stream), h.shape[0], _ptr(h), _ptr(q), _ptr(q_scale), width,
                                         out_stride))


def gemm_i8_rope_256(m, a, w, scale, a_scale, c, q_norm, k_norm, cos, sin, q_out, k_out, v_out, k_size, k_stride, n_size,
                     q_heads, kv_heads, eps=1e-5, m_group=4, stream=None):
    """gemm_i8_256 over q|k|v|gate columns whose epilogue also does rope_qknorm_f16's work: q, k normalised and
    rotated, v copied, only the gate columns written to `c`."""
    check(lib().krea2_gemm_i8_rope_256(_stream_ptr(stream), m, _ptr(a), _ptr(w), _ptr(scale), _ptr(a_scale), _ptr(c),
                                       _ptr(q_norm), _ptr(k_norm), _ptr(cos), _ptr(sin), _ptr(q_out), _ptr(k_out), _ptr(v_out),
                                       k_size, k_stride, n_size, m_group, q_heads, kv_heads, eps))


def gemm_i8_acc(m, a, w, acc, k_size, k_stride, n_size, stream=None):
    check(lib().krea2_gemm_i8_acc(_stream_ptr(stream), m, _ptr(a), _ptr(w), _ptr(acc), k_size, k_stride, n_size))


def lora_transport(src, dst, reverse: int, stream=None):
    check(lib().krea2_lora_transport(_stream_ptr(stream), src.numel(), _ptr(src), _ptr(dst), reverse))


class Quantized:
    """training::quantized::Quantized (src/training/quantized.rs:8-112): one W8A8 projection on
    bf16 tensors -- bf16 -> f16 transport, prepare_plain_i8, gemm_i8_256, f16 -> bf16."""

    def __init__(self, weight: torch.Tensor, scales: torch.Tensor, outputs: int, inputs: int):
        """`weight` int8 [outputs][inputs] and `scales` f32 [outputs], on the host or the device;
        rows are re-pitched to shape::gemm_pitch(inputs) as Quantized::load does (:34-47)."""
        if weight.dtype != torch.int8 or tuple(weight.shape) != (outputs, inputs) or scales.dtype != torch.float32 \
                or scales.numel() != outputs:
            raise InvalidArgument("invalid ConvRot projection")
        self.inputs, self.outputs = inputs, outputs
        self.pitch = shape.gemm_pitch(inputs)
        device = torch.device("cuda", torch.cuda.current_device())
        self.weight = torch.zeros((outputs, self.pitch), dtype=torch.int8, device=device)
        self.weight[:, :inputs] = weight.to(device)
        self.scales = scales.to(device).contiguous()

    def forward_fused(self, stream, x: torch.Tensor, workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The same projection through krea2_quantized_forward: one C call, intermediates in a
        caller-owned workspace (allocated here when none is passed)."""
        if x.shape[-1] != self.inputs or x.dtype != torch.bfloat16:
            raise InvalidArgument("ConvRot projection dimensions")
        rows = x.shape[0]
        need = lib().krea2_quantized_workspace_bytes(rows, self.inputs, self.outputs)
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.uint8, device=x.device)
        out = torch.empty((rows, self.outputs), dtype=torch.bfloat16, device=x.device)
        check(lib().krea2_quantized_forward(_stream_ptr(stream), rows, _ptr(x), _ptr(self.weight), _ptr(self.scales),
                                            _ptr(out), self.inputs, self.outputs, _ptr(workspace), _bytes(workspace)))
        return out

    def forward(self, ops: Ops, stream, x: torch.Tensor) -> torch.Tensor:
        if x.shape[-1] != self.inputs or x.dtype != torch.bfloat16:
            raise InvalidArgument("ConvRot projection dimensions")
        rows = x.shape[0]
        dev = x.device
        transport = torch.empty((rows, self.inputs), dtype=torch.float16, device=dev)
        quantized = torch.empty((rows, self.pitch), dtype=torch.int8, device=dev)
        scales = torch.empty((rows,), dtype=torch.float32, device=dev)
        out_f16 = torch.empty((rows, self.outputs), dtype=torch.float16, device=dev)
        out = torch.empty((rows, self.outputs), dtype=torch.bfloat16, device=dev)
        one = kernels.Scalars()
        ops.launch_1d(stream, "lora_transport", kernels.config([("reverse", 1)]), one.index(x.numel()),
                      [x, transport], x.numel())
        ops.launch(stream, "prepare_plain_i8", kernels.config([("width", self.inputs), ("out_stride", self.pitch)]),
                   one.index(rows), [transport, quantized, scales], rows, 1, 256)
        ops.launch(stream, "gemm_i8_256",
                   kernels.config([("k_size", self.inputs), ("k_stride", self.pitch), ("n_size", self.outputs),
                                   ("m_group", shape.gemm_m_group())]),
                   one.index(rows), [quantized, self.weight, self.scales, scales, out_f16], self.outputs // 128,
                   shape.gemm_grid_rows(rows), 256)
        ops.launch_1d(stream, "lora_transport", kernels.config([("reverse", 2)]), one.index(out.numel()),
                      [out_f16, out], out.numel())
        return out


# ------------------------------------------------------------------ the rest of a block
def rope_qknorm_f16(qkv, q_scale, k_scale, cos, sin, q_out, k_out, v_out, row_stride, q_heads, kv_heads, k_offset,
                    eps=1e-5, stream=None, tokens=None):
    tokens = q_out.shape[0] if tokens is None else tokens
    check(lib().krea2_rope_qknorm_f16(_stream_ptr(stream), tokens, qkv.data_ptr(), _ptr(q_scale), _ptr(k_scale), _ptr(cos),
                                      _ptr(sin), _ptr(q_out), _ptr(k_out), _ptr(v_out), row_stride, q_heads, kv_heads,
                                      k_offset, eps))


def v_transpose(x, out, width, row_capacity, stream=None, rows=None):
    rows = x.shape[0] if rows is None else rows
    check(lib().krea2_v_transpose(_stream_ptr(stream), rows, _ptr(x), _ptr(out), width, row_capacity))


def attention_gqa(tokens, kv_heads, q, k, v_transposed, out, q_stride, kv_stride, out_stride, token_capacity, scale,
                  stream=None, q32=False):
    fn = lib().krea2_attention_gqa_lds_f16_wmma_q32 if q32 else lib().krea2_attention_gqa_lds_f16_wmma
    check(fn(_stream_ptr(stream), tokens, kv_heads, _ptr(q), _ptr(k), _ptr(v_transposed), _ptr(out), q_stride, kv_stride,
             out_stride, token_capacity, scale))


def attention_gqa_rows(q_rows, tokens, kv_heads, q, k, v_transposed, out, q_stride, kv_stride, out_stride, token_capacity,
                       scale, stream=None):
    """`q_rows` query rows (q and out hold just those) against all `tokens` keys and values."""
    check(lib().krea2_attention_gqa_f16_rows(_stream_ptr(stream), q_rows, tokens, kv_heads, _ptr(q), _ptr(k),
                                             _ptr(v_transposed), _ptr(out), q_stride, kv_stride, out_stride,
                                             token_capacity, scale))


def rope_qknorm_f16_sharded(tokens, qkv, q_scale, k_scale, cos, sin, q_out, row_stride, q_heads, kv_heads, k_offset,
                            shard, eps=1e-5, stream=None):
    """QK-norm + RoPE of this device's rows; K and V rows go to every device's full-length tensors (`shard`:
    a `_lib.RowShard`)."""
    check(lib().krea2_rope_qknorm_f16_sharded(_stream_ptr(stream), tokens, qkv.data_ptr(), _ptr(q_scale), _ptr(k_scale),
                                              _ptr(cos), _ptr(sin), _ptr(q_out), row_stride, q_heads, kv_heads, k_offset,
                                              eps, ctypes.byref(shard)))


def shard_signal(shard, stream=None):
    check(lib().krea2_shard_signal(_stream_ptr(stream), ctypes.byref(shard)))


# ------------------------------------------------------------------ around the block chain
def modulation(vector, tables, out, stream=None):
    """Models::modulation (src/models/graph.rs:405-425): `out` f32 = bf16(vector[i % len] + tables[i])."""
    if out.numel() != tables.numel():
        raise InvalidArgument("modulation dimensions")
    check(lib().krea2_modulation(_stream_ptr(stream), tables.numel(), _ptr(vector), _ptr(tables), _ptr(out),
                                 vector.numel()))


def euler_step(sample, velocity, delta, stream=None):
    """Ops::euler_step (src/ops/mod.rs:373-390): `sample += delta * velocity` in place with the sampler's
    bf16 rounding at the delta, the product and the sum."""
    if tuple(sample.shape) != tuple(velocity.shape):
        raise InvalidArgument("scheduler tensor dimensions")
    check(lib().krea2_euler(_stream_ptr(stream), sample.numel(), float(delta), _ptr(sample), _ptr(velocity)))


def guidance(cond, uncond, scale, stream=None):
    """Ops::guidance (src/ops/mod.rs:392-410): `cond += scale * (cond - uncond)` in place, bf16 at each step."""
    if tuple(cond.shape) != tuple(uncond.shape):
        raise InvalidArgument("guidance tensor dimensions")
    check(lib().krea2_guidance(_stream_ptr(stream), cond.numel(), float(scale), _ptr(cond), _ptr(uncond)))
