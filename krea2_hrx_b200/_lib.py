"""ctypes binding of libkrea2_b200.so (declared in include/krea2_b200.h).

The library is the product; there is no other implementation behind these calls.  A
missing library is an ImportError-grade failure, never a fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int, c_size_t, c_uint16, c_uint32, c_uint64, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
# KREA2_B200_LIB names another build of the same library (e.g. one compiled with other build-time choices).
LIB_PATH = os.environ.get("KREA2_B200_LIB") or os.path.join(HERE, "libkrea2_b200.so")


class Error(RuntimeError):
    """krea2::Error (src/error.rs:10-29): one class per variant."""
    status = 5


class InvalidArgument(Error, ValueError):
    status = 1


class Cancelled(Error):
    status = 2


class Poisoned(Error):
    status = 3


class Runtime(Error):
    status = 4


class Internal(Error):
    status = 5


_BY_STATUS = {1: InvalidArgument, 2: Cancelled, 3: Poisoned, 4: Runtime, 5: Internal}


class ConfigEntry(ctypes.Structure):
    _fields_ = [("key", c_char_p), ("value", c_uint64), ("fvalue", c_float)]


class Binding(ctypes.Structure):
    _fields_ = [("ptr", c_void_p), ("bytes", c_size_t)]


class Shard(ctypes.Structure):
    _fields_ = [("world", c_uint32), ("rank", c_uint32), ("dest", c_void_p * 8), ("pitch", c_size_t),
                ("offset", c_size_t), ("flags", c_void_p * 8), ("epoch", c_uint32), ("counter", c_void_p), ("epoch_base", c_void_p)]


class RowShard(ctypes.Structure):
    _fields_ = [("world", c_uint32), ("rank", c_uint32), ("k_dest", c_void_p * 8), ("v_dest", c_void_p * 8),
                ("first_row", c_size_t), ("flags", c_void_p * 8), ("epoch", c_uint32), ("counter", c_void_p),
                ("epoch_base", c_void_p)]


class SpanInfo(ctypes.Structure):
    _fields_ = [(name, c_size_t) for name in ("device_offset", "device_bytes", "rows", "row_bytes",
                                               "device_row_bytes", "segments", "file_bytes")]


class Dims(ctypes.Structure):
    _fields_ = [("hidden", c_size_t), ("kv_heads", c_size_t), ("head_dim", c_size_t), ("inter", c_size_t)]


# name -> (restype, argtypes); every symbol include/krea2_b200.h declares.
SIGNATURES = {
    "krea2_last_error": (c_char_p, []),
    "krea2_version": (c_char_p, []),
    "krea2_device_status": (c_int, [POINTER(c_int)]),
    "krea2_prepare_norm_i8": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_size_t, c_size_t, c_float]),
    "krea2_prepare_gated_i8": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t,
                                       c_size_t]),
    "krea2_prepare_plain_i8": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t]),
    "krea2_gemm_i8_256": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                  c_size_t, c_size_t, c_size_t]),
    "krea2_gemm_i8_resid_256": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_size_t, c_size_t, c_size_t, c_size_t]),
    "krea2_gemm_i8_resid_256x256": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                            c_void_p, c_size_t, c_size_t, c_size_t, c_size_t, c_size_t]),
    "krea2_gemm_i8_swiglu_256": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                         c_size_t, c_size_t, c_size_t]),
    "krea2_gemm_i8_swiglu_rotated_256": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                                 c_size_t, c_size_t, c_size_t]),
    "krea2_prepare_rotated_i8": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t]),
    "krea2_gemm_i8_rope_256": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_size_t,
                                       c_size_t, c_size_t, c_float]),
    "krea2_gemm_i8_acc": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t]),
    "krea2_rope_qknorm_f16": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_size_t, c_size_t, c_size_t, c_size_t, c_float]),
    "krea2_v_transpose": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_size_t, c_size_t]),
    "krea2_modulation": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_size_t]),
    "krea2_euler": (c_int, [c_void_p, c_size_t, c_float, c_void_p, c_void_p]),
    "krea2_guidance": (c_int, [c_void_p, c_size_t, c_float, c_void_p, c_void_p]),
    "krea2_schedule_dynamic_mu": (c_double, [c_size_t]),
    "krea2_schedule_sigma": (c_float, [c_size_t, c_size_t, c_double]),
    "krea2_schedule_next_sigma": (c_float, [c_size_t, c_size_t, c_size_t, c_double]),
    "krea2_attention_gqa_lds_f16_wmma": (c_int, [c_void_p, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_size_t, c_float]),
    "krea2_attention_gqa_lds_f16_wmma_q32": (c_int, [c_void_p, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t, c_size_t, c_size_t, c_float]),
    "krea2_gemm_i8_sharded": (c_int, [c_void_p, c_int, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                      c_size_t, c_size_t, POINTER(Shard)]),
    "krea2_shard_wait": (c_int, [c_void_p, c_void_p, c_uint32, c_uint32, c_void_p]),
    "krea2_rope_qknorm_f16_sharded": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                              c_size_t, c_size_t, c_size_t, c_size_t, c_float, POINTER(RowShard)]),
    "krea2_shard_signal": (c_int, [c_void_p, POINTER(RowShard)]),
    "krea2_attention_gqa_f16_rows": (c_int, [c_void_p, c_size_t, c_size_t, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p,
                                             c_size_t, c_size_t, c_size_t, c_size_t, c_float]),
    "krea2_shard_advance": (c_int, [c_void_p, c_void_p, c_uint32]),
    "krea2_lora_transport": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_int]),
    "krea2_quantized_workspace_bytes": (c_size_t, [c_size_t, c_size_t, c_size_t]),
    "krea2_quantized_forward": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t,
                                        c_void_p, c_size_t]),
    "krea2_quantized_static_workspace_bytes": (c_size_t, []),
    "krea2_quantized_forward_static": (c_int, [c_void_p, c_size_t, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t,
                                               c_size_t]),
    "krea2_launch": (c_int, [c_void_p, c_char_p, POINTER(ConfigEntry), c_size_t, POINTER(c_uint64), c_size_t,
                             POINTER(Binding), c_size_t, c_size_t, c_size_t, c_uint32]),
    "krea2_shape_tokens_min": (c_size_t, []),
    "krea2_shape_tokens_max": (c_size_t, []),
    "krea2_shape_capacity": (c_size_t, [c_size_t]),
    "krea2_shape_gemm_pitch": (c_size_t, [c_size_t]),
    "krea2_shape_gemm_grid_rows": (c_size_t, [c_size_t]),
    "krea2_shape_gemm_m_group": (c_size_t, []),
    "krea2_shape_gemm_schedule_rows": (c_int, [c_size_t]),
    "krea2_shape_attention_rows": (c_size_t, [c_size_t]),
    "krea2_shape_gemm_tile_columns": (c_size_t, [c_char_p]),
    "krea2_shape_gemm_tile_threads": (c_uint32, [c_char_p]),
    "krea2_shape_gemm_source": (c_char_p, [c_char_p, c_char_p]),
    "krea2_session_validate_dimensions": (c_int, [c_size_t, c_size_t]),
    "krea2_weights_plan_bytes": (c_int, [POINTER(Dims), c_size_t, POINTER(c_size_t)]),
    "krea2_weights_create": (c_int, [POINTER(Dims), c_size_t, POINTER(c_void_p)]),
    "krea2_weights_locate": (c_int, [c_void_p, c_char_p, POINTER(c_void_p), POINTER(c_size_t)]),
    "krea2_weights_fill_synthetic": (c_int, [c_void_p, c_uint64, c_void_p]),
    "krea2_weights_upload": (c_int, [c_void_p, c_char_p, c_void_p, c_size_t, c_void_p]),
    "krea2_weights_download": (c_int, [c_void_p, c_char_p, c_void_p, c_size_t, c_void_p]),
    "krea2_weights_retain": (None, [c_void_p]),
    "krea2_weights_release": (None, [c_void_p]),
    "krea2_checkpoint_open": (c_int, [c_char_p, POINTER(c_void_p)]),
    "krea2_checkpoint_close": (None, [c_void_p]),
    "krea2_checkpoint_has": (c_int, [c_void_p, c_char_p]),
    "krea2_checkpoint_block_count": (c_size_t, [c_void_p]),
    "krea2_checkpoint_names": (c_size_t, [c_void_p, POINTER(c_char_p), c_size_t]),
    "krea2_checkpoint_tensor": (c_int, [c_void_p, c_char_p, POINTER(c_char_p), POINTER(POINTER(c_size_t)),
                                        POINTER(c_size_t), POINTER(c_void_p), POINTER(c_size_t)]),
    "krea2_checkpoint_plan": (c_int, [c_void_p, POINTER(c_size_t), POINTER(c_size_t), POINTER(c_size_t)]),
    "krea2_checkpoint_span_name": (c_int, [c_void_p, c_size_t, POINTER(c_char_p)]),
    "krea2_checkpoint_span": (c_int, [c_void_p, c_char_p, POINTER(SpanInfo)]),
    "krea2_checkpoint_segment": (c_int, [c_void_p, c_char_p, c_size_t, POINTER(c_char_p), POINTER(c_size_t),
                                         POINTER(c_size_t)]),
    "krea2_checkpoint_assemble": (c_int, [c_void_p, c_char_p, c_void_p, c_size_t]),
    "krea2_checkpoint_dims": (c_int, [c_void_p, POINTER(Dims), POINTER(c_size_t)]),
    "krea2_session_validate": (c_int, [c_char_p, c_size_t, c_size_t]),
    "krea2_weights_load_checkpoint": (c_int, [c_void_p, c_void_p, POINTER(c_void_p)]),
    "krea2_session_create": (c_int, [c_void_p, c_void_p, c_size_t, c_size_t, POINTER(c_void_p)]),
    "krea2_session_destroy": (None, [c_void_p]),
    "krea2_session_tokens": (c_size_t, [c_void_p]),
    "krea2_session_layers": (c_size_t, [c_void_p]),
    "krea2_session_set_profile": (c_int, [c_void_p, c_int]),
    "krea2_session_set_attention": (c_int, [c_void_p, c_int]),
    "krea2_session_set_fused_rotation": (c_int, [c_void_p, c_int]),
    "krea2_session_set_fused_rope": (c_int, [c_void_p, c_int]),
    "krea2_session_stage_profile": (c_size_t, [c_void_p, POINTER(c_char_p), POINTER(c_double), c_size_t]),
    "krea2_session_run": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_size_t]),
    "krea2_session_run_device": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_size_t, c_void_p,
                                         c_void_p]),
    "krea2_session_buffer": (c_int, [c_void_p, c_char_p, POINTER(c_void_p), POINTER(c_size_t)]),
    "krea2_session_launches_per_forward": (c_size_t, [c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises if it was never built (run krea2_hrx_b200/build.py)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m krea2_hrx_b200.build` "
                              "(nvcc, sm_100a); there is no fallback implementation")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int) -> None:
    """Raises the exception class of a non-zero krea2_status with the library's message."""
    if status != 0:
        message = lib().krea2_last_error().decode("utf-8", "replace")
        raise _BY_STATUS.get(status, Internal)(message)


def device_status() -> int:
    value = c_int(0)
    check(lib().krea2_device_status(ctypes.byref(value)))
    return value.value
