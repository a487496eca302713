//! Raw bindings to `libkrea2_b200`, the B200 (sm_100a) implementation of krea2-hrx's W8A8 linear-layer path.
//!
//! UNCOMPILED: this crate was written in an environment without a Rust toolchain.  The `extern "C"` block below
//! is held to `include/krea2_b200.h` by a test of the repository (names, arities and parameter types of every
//! function), but no `cargo build` has ever run on it.
//!
//! One function per exported Loom symbol of the reference (`krea2_<stem>`, the buffers in the order of the
//! kernel's `launch(...)` line, the `config` keys as trailing integers), plus the shape rules of
//! `kernels::shape`, the resident `session::Session` and `session::Weights`, the checkpoint plan and the
//! sampler's pointwise kernels.  `build.rs` compiles the `.cu` sources with nvcc for sm_100a and links them.
//!
//! Where the reference binds this: `Session::launch` (src/session/mod.rs:386-421) and `Ops::launch`
//! (src/ops/mod.rs:673-693) hand a kernel, a grid, a scalar block and an ordered buffer list to
//! `hrx::Stream::dispatch`; with this crate the same call sites pass the same buffers (as device pointers)
//! to the function named after the kernel.
#![allow(non_camel_case_types)]

use core::ffi::{c_char, c_int, c_void};

/// `cudaStream_t`.
pub type krea2_stream = *mut c_void;

/// `krea2::Error` classes (src/error.rs:10-29) as the status every call returns.
pub const KREA2_OK: c_int = 0;
pub const KREA2_INVALID_ARGUMENT: c_int = 1;
pub const KREA2_CANCELLED: c_int = 2;
pub const KREA2_POISONED: c_int = 3;
pub const KREA2_RUNTIME: c_int = 4;
pub const KREA2_INTERNAL: c_int = 5;

pub const KREA2_SHARD_PLAIN: c_int = 0;
pub const KREA2_SHARD_RESID: c_int = 1;
pub const KREA2_SHARD_SWIGLU: c_int = 2;

/// One `config` key of a name-keyed launch (`Ops::launch`, src/ops/mod.rs:673-693).
#[repr(C)]
pub struct krea2_config_entry {
    pub key: *const c_char,
    pub value: u64,
    pub fvalue: f32,
}

/// One buffer binding: device pointer and the extent the kernel may touch.
#[repr(C)]
pub struct krea2_binding {
    pub ptr: *mut c_void,
    pub bytes: usize,
}

/// A column-sharded GEMM launch (no counterpart in the reference).
#[repr(C)]
pub struct krea2_shard {
    pub world: u32,
    pub rank: u32,
    pub dest: [*mut c_void; 8],
    pub pitch: usize,
    pub offset: usize,
    pub flags: [*mut u32; 8],
    pub epoch: u32,
    pub counter: *mut u32,
    pub epoch_base: *const u32,
}

/// A token-sharded QK-norm + RoPE launch (no counterpart in the reference).
#[repr(C)]
pub struct krea2_row_shard {
    pub world: u32,
    pub rank: u32,
    pub k_dest: [*mut c_void; 8],
    pub v_dest: [*mut c_void; 8],
    pub first_row: usize,
    pub flags: [*mut u32; 8],
    pub epoch: u32,
    pub counter: *mut u32,
    pub epoch_base: *const u32,
}

/// The block shape (src/session/mod.rs:35-45).
#[repr(C)]
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub struct krea2_dims {
    pub hidden: usize,
    pub kv_heads: usize,
    pub head_dim: usize,
    pub inter: usize,
}

/// `Plan::span` (src/checkpoint/plan.rs:23-43).
#[repr(C)]
#[derive(Clone, Copy, Debug, Default)]
pub struct krea2_span_info {
    pub device_offset: usize,
    pub device_bytes: usize,
    pub rows: usize,
    pub row_bytes: usize,
    pub device_row_bytes: usize,
    pub segments: usize,
    pub file_bytes: usize,
}

#[repr(C)]
pub struct krea2_weights {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct krea2_session {
    _opaque: [u8; 0],
}
#[repr(C)]
pub struct krea2_checkpoint {
    _opaque: [u8; 0],
}

extern "C" {
    pub fn krea2_last_error() -> *const c_char;
    pub fn krea2_version() -> *const c_char;
    pub fn krea2_device_status(host_status: *mut c_int) -> c_int;
    pub fn krea2_prepare_norm_i8(stream: krea2_stream, tokens: usize, h: *const c_void, norm_scale: *const f32, mod_scale: *const f32, mod_shift: *const f32, q: *mut c_void, q_scale: *mut f32, width: usize, out_stride: usize, eps: f32) -> c_int;
    pub fn krea2_prepare_gated_i8(stream: krea2_stream, tokens: usize, attn: *const c_void, gate: *const c_void, q: *mut c_void, q_scale: *mut f32, width: usize, out_stride: usize, gate_stride: usize) -> c_int;
    pub fn krea2_prepare_plain_i8(stream: krea2_stream, tokens: usize, h: *const c_void, q: *mut c_void, q_scale: *mut f32, width: usize, out_stride: usize) -> c_int;
    pub fn krea2_gemm_i8_256(stream: krea2_stream, m: usize, a: *const c_void, w: *const c_void, scale: *const f32, a_scale: *const f32, c: *mut c_void, k_size: usize, k_stride: usize, n_size: usize, m_group: usize) -> c_int;
    pub fn krea2_gemm_i8_resid_256(stream: krea2_stream, m: usize, a: *const c_void, w: *const c_void, scale: *const f32, a_scale: *const f32, c: *mut c_void, gate: *const f32, k_size: usize, k_stride: usize, n_size: usize, m_group: usize) -> c_int;
    pub fn krea2_gemm_i8_resid_256x256(stream: krea2_stream, m: usize, a: *const c_void, w: *const c_void, scale: *const f32, a_scale: *const f32, c: *mut c_void, gate: *const f32, k_size: usize, k_stride: usize, n_size: usize, m_group: usize, schedule_rows: usize) -> c_int;
    pub fn krea2_gemm_i8_swiglu_256(stream: krea2_stream, m: usize, a: *const c_void, w: *const c_void, scale: *const f32, a_scale: *const f32, c: *mut c_void, k_size: usize, k_stride: usize, n_size: usize, m_group: usize) -> c_int;
    pub fn krea2_gemm_i8_swiglu_rotated_256(stream: krea2_stream, m: usize, a: *const c_void, w: *const c_void, scale: *const f32, a_scale: *const f32, c: *mut c_void, k_size: usize, k_stride: usize, n_size: usize, m_group: usize) -> c_int;
    pub fn krea2_prepare_rotated_i8(stream: krea2_stream, tokens: usize, h: *const c_void, q: *mut c_void, q_scale: *mut f32, width: usize, out_stride: usize) -> c_int;
    pub fn krea2_gemm_i8_rope_256(stream: krea2_stream, m: usize, a: *const c_void, w: *const c_void, scale: *const f32, a_scale: *const f32, c: *mut c_void, q_norm: *const f32, k_norm: *const f32, cos_table: *const f32, sin_table: *const f32, q_out: *mut c_void, k_out: *mut c_void, v_out: *mut c_void, k_size: usize, k_stride: usize, n_size: usize, m_group: usize, q_heads: usize, kv_heads: usize, eps: f32) -> c_int;
    pub fn krea2_gemm_i8_acc(stream: krea2_stream, m: usize, a: *const c_void, w: *const c_void, acc: *mut i32, k_size: usize, k_stride: usize, n_size: usize) -> c_int;
    pub fn krea2_rope_qknorm_f16(stream: krea2_stream, tokens: usize, qkv: *const c_void, q_scale: *const f32, k_scale: *const f32, cos_table: *const f32, sin_table: *const f32, q_out: *mut c_void, k_out: *mut c_void, v_out: *mut c_void, row_stride: usize, q_heads: usize, kv_heads: usize, k_offset: usize, eps: f32) -> c_int;
    pub fn krea2_v_transpose(stream: krea2_stream, rows: usize, x: *const c_void, out: *mut c_void, width: usize, row_capacity: usize) -> c_int;
    pub fn krea2_modulation(stream: krea2_stream, count: usize, x: *const c_void, tables: *const c_void, y: *mut f32, xsize: usize) -> c_int;
    pub fn krea2_euler(stream: krea2_stream, count: usize, delta: f32, sample: *mut c_void, velocity: *const c_void) -> c_int;
    pub fn krea2_guidance(stream: krea2_stream, count: usize, scale: f32, cond: *mut c_void, uncond: *const c_void) -> c_int;
    pub fn krea2_schedule_dynamic_mu(image_tokens: usize) -> f64;
    pub fn krea2_schedule_sigma(step: usize, steps: usize, mu: f64) -> f32;
    pub fn krea2_schedule_next_sigma(step: usize, last: usize, steps: usize, mu: f64) -> f32;
    pub fn krea2_attention_gqa_lds_f16_wmma(stream: krea2_stream, tokens: usize, kv_heads: usize, q: *const c_void, k: *const c_void, v_transposed: *const c_void, out: *mut c_void, q_stride: usize, kv_stride: usize, out_stride: usize, token_capacity: usize, scale: f32) -> c_int;
    pub fn krea2_attention_gqa_lds_f16_wmma_q32(stream: krea2_stream, tokens: usize, kv_heads: usize, q: *const c_void, k: *const c_void, v_transposed: *const c_void, out: *mut c_void, q_stride: usize, kv_stride: usize, out_stride: usize, token_capacity: usize, scale: f32) -> c_int;
    pub fn krea2_gemm_i8_sharded(stream: krea2_stream, kind: c_int, m: usize, a: *const c_void, w: *const c_void, scale: *const f32, a_scale: *const f32, gate: *const f32, k_size: usize, k_stride: usize, n_size: usize, shard: *const krea2_shard) -> c_int;
    pub fn krea2_shard_wait(stream: krea2_stream, flags: *const u32, world: u32, epoch: u32, epoch_base: *const u32) -> c_int;
    pub fn krea2_shard_advance(stream: krea2_stream, epoch_base: *mut u32, delta: u32) -> c_int;
    pub fn krea2_rope_qknorm_f16_sharded(stream: krea2_stream, tokens: usize, qkv: *const c_void, q_scale: *const f32, k_scale: *const f32, cos_table: *const f32, sin_table: *const f32, q_out: *mut c_void, row_stride: usize, q_heads: usize, kv_heads: usize, k_offset: usize, eps: f32, shard: *const krea2_row_shard) -> c_int;
    pub fn krea2_shard_signal(stream: krea2_stream, shard: *const krea2_row_shard) -> c_int;
    pub fn krea2_attention_gqa_f16_rows(stream: krea2_stream, q_rows: usize, tokens: usize, kv_heads: usize, q: *const c_void, k: *const c_void, v_transposed: *const c_void, out: *mut c_void, q_stride: usize, kv_stride: usize, out_stride: usize, token_capacity: usize, scale: f32) -> c_int;
    pub fn krea2_lora_transport(stream: krea2_stream, elements: usize, src: *const c_void, dst: *mut c_void, reverse: c_int) -> c_int;
    pub fn krea2_quantized_workspace_bytes(rows: usize, inputs: usize, outputs: usize) -> usize;
    pub fn krea2_quantized_forward(stream: krea2_stream, rows: usize, x: *const c_void, weight: *const c_void, scales: *const f32, out: *mut c_void, inputs: usize, outputs: usize, workspace: *mut c_void, workspace_bytes: usize) -> c_int;
    pub fn krea2_quantized_static_workspace_bytes() -> usize;
    pub fn krea2_quantized_forward_static(stream: krea2_stream, rows: usize, x: *const c_void, weight: *const c_void, scales: *const f32, out: *mut c_void, inputs: usize, outputs: usize) -> c_int;
    pub fn krea2_launch(stream: krea2_stream, name: *const c_char, config: *const krea2_config_entry, config_count: usize, indices: *const u64, index_count: usize, bindings: *const krea2_binding, binding_count: usize, grid_x: usize, grid_y: usize, threads: u32) -> c_int;
    pub fn krea2_shape_tokens_min() -> usize;
    pub fn krea2_shape_tokens_max() -> usize;
    pub fn krea2_shape_capacity(tokens: usize) -> usize;
    pub fn krea2_shape_gemm_pitch(k: usize) -> usize;
    pub fn krea2_shape_gemm_grid_rows(tokens: usize) -> usize;
    pub fn krea2_shape_gemm_m_group() -> usize;
    pub fn krea2_shape_gemm_schedule_rows(tokens: usize) -> c_int;
    pub fn krea2_shape_attention_rows(tokens: usize) -> usize;
    pub fn krea2_shape_gemm_tile_columns(stem: *const c_char) -> usize;
    pub fn krea2_shape_gemm_tile_threads(stem: *const c_char) -> u32;
    pub fn krea2_shape_gemm_source(family: *const c_char, stem: *const c_char) -> *const c_char;
    pub fn krea2_session_validate_dimensions(tokens: usize, layers: usize) -> c_int;
    pub fn krea2_weights_plan_bytes(dims: *const krea2_dims, layers: usize, bytes: *mut usize) -> c_int;
    pub fn krea2_weights_create(dims: *const krea2_dims, layers: usize, out: *mut *mut krea2_weights) -> c_int;
    pub fn krea2_weights_locate(weights: *const krea2_weights, name: *const c_char, ptr: *mut *mut c_void, bytes: *mut usize) -> c_int;
    pub fn krea2_weights_fill_synthetic(weights: *mut krea2_weights, seed: u64, stream: krea2_stream) -> c_int;
    pub fn krea2_weights_upload(weights: *mut krea2_weights, name: *const c_char, host_bytes: *const c_void, bytes: usize, stream: krea2_stream) -> c_int;
    pub fn krea2_weights_download(weights: *const krea2_weights, name: *const c_char, host_bytes: *mut c_void, bytes: usize, stream: krea2_stream) -> c_int;
    pub fn krea2_weights_retain(weights: *mut krea2_weights);
    pub fn krea2_weights_release(weights: *mut krea2_weights);
    pub fn krea2_checkpoint_open(path: *const c_char, out: *mut *mut krea2_checkpoint) -> c_int;
    pub fn krea2_checkpoint_close(checkpoint: *mut krea2_checkpoint);
    pub fn krea2_checkpoint_has(checkpoint: *const krea2_checkpoint, name: *const c_char) -> c_int;
    pub fn krea2_checkpoint_block_count(checkpoint: *const krea2_checkpoint) -> usize;
    pub fn krea2_checkpoint_names(checkpoint: *const krea2_checkpoint, names: *mut *const c_char, capacity: usize) -> usize;
    pub fn krea2_checkpoint_tensor(checkpoint: *const krea2_checkpoint, name: *const c_char, dtype: *mut *const c_char, shape: *mut *const usize, rank: *mut usize, bytes: *mut *const c_void, byte_count: *mut usize) -> c_int;
    pub fn krea2_checkpoint_plan(checkpoint: *mut krea2_checkpoint, total_bytes: *mut usize, layers: *mut usize, span_count: *mut usize) -> c_int;
    pub fn krea2_checkpoint_span_name(checkpoint: *mut krea2_checkpoint, index: usize, name: *mut *const c_char) -> c_int;
    pub fn krea2_checkpoint_span(checkpoint: *mut krea2_checkpoint, name: *const c_char, info: *mut krea2_span_info) -> c_int;
    pub fn krea2_checkpoint_segment(checkpoint: *mut krea2_checkpoint, span: *const c_char, index: usize, tensor: *mut *const c_char, row_begin: *mut usize, row_end: *mut usize) -> c_int;
    pub fn krea2_checkpoint_assemble(checkpoint: *mut krea2_checkpoint, span: *const c_char, host_bytes: *mut c_void, bytes: usize) -> c_int;
    pub fn krea2_checkpoint_dims(checkpoint: *mut krea2_checkpoint, dims: *mut krea2_dims, layers: *mut usize) -> c_int;
    pub fn krea2_session_validate(checkpoint_path: *const c_char, tokens: usize, layers: usize) -> c_int;
    pub fn krea2_weights_load_checkpoint(checkpoint: *mut krea2_checkpoint, stream: krea2_stream, out: *mut *mut krea2_weights) -> c_int;
    pub fn krea2_session_create(stream: krea2_stream, weights: *mut krea2_weights, tokens: usize, layers: usize, out: *mut *mut krea2_session) -> c_int;
    pub fn krea2_session_destroy(session: *mut krea2_session);
    pub fn krea2_session_tokens(session: *const krea2_session) -> usize;
    pub fn krea2_session_layers(session: *const krea2_session) -> usize;
    pub fn krea2_session_set_profile(session: *mut krea2_session, enable: c_int) -> c_int;
    pub fn krea2_session_stage_profile(session: *const krea2_session, labels: *mut *const c_char, millis: *mut f64, capacity: usize) -> usize;
    pub fn krea2_session_run(session: *mut krea2_session, stream: krea2_stream, host_x: *mut u16, host_mods: *const f32, host_cos: *const f32, host_sin: *const f32, first_block: usize, block_count: usize) -> c_int;
    pub fn krea2_session_run_device(session: *mut krea2_session, stream: krea2_stream, x: *mut c_void, x_bytes: usize, mods: *const c_void, mods_bytes: usize, host_cos: *const f32, host_sin: *const f32) -> c_int;
    pub fn krea2_session_buffer(session: *const krea2_session, name: *const c_char, ptr: *mut *mut c_void, bytes: *mut usize) -> c_int;
    pub fn krea2_session_set_attention(session: *mut krea2_session, enable: c_int) -> c_int;
    pub fn krea2_session_set_fused_rotation(session: *mut krea2_session, enable: c_int) -> c_int;
    pub fn krea2_session_set_fused_rope(session: *mut krea2_session, enable: c_int) -> c_int;
    pub fn krea2_session_launches_per_forward(session: *const krea2_session) -> usize;
}

/// The message of the last failing call on this thread.
pub fn last_error() -> String {
    // SAFETY: the library returns a pointer to a NUL-terminated thread-local buffer that stays valid until the
    // next call on this thread.
    unsafe { std::ffi::CStr::from_ptr(krea2_last_error()) }.to_string_lossy().into_owned()
}

/// Maps a status to `Result`, carrying the library's message.
pub fn check(status: c_int) -> Result<(), (c_int, String)> {
    if status == KREA2_OK {
        Ok(())
    } else {
        Err((status, last_error()))
    }
}
