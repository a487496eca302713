/*
 * krea2_b200 -- C ABI of the B200 (sm_100a) implementation of krea2-hrx's W8A8
 * linear-layer path.
 *
 * The reference has no C ABI of its own: its boundary is the kernel launch ABI that
 * `Session::launch` (src/session/mod.rs:386-421) and `Ops::launch` (src/ops/mod.rs:673-693)
 * hand to the runtime -- an exported symbol `krea2_<stem>`, one packed scalar (the row
 * count) and the buffers in the order of each kernel's `launch(...)` signature, with the
 * shape constants supplied as compile-time `config` keys.  Each function below keeps one
 * such symbol: same name, same buffer order, and the config keys as trailing integers.
 *
 * Conventions
 *  - Every pointer is a DEVICE pointer unless a parameter is named host_*; `stream` is a
 *    `cudaStream_t` (passed as void* so that this header needs no CUDA include).
 *  - The caller owns every buffer; kernels allocate nothing.  Bytes of a row beyond
 *    `width` / `k_size` are never read (GEMM operands) and never written (prologues).
 *  - bf16 and f16 tensors are raw 16-bit patterns, row-major.
 *  - Every function returns a krea2_status; on failure krea2_last_error() returns a
 *    thread-local description.  Invalid arguments are refused before any device work
 *    (the reference's rule, tests/constructor.rs).
 */
#ifndef KREA2_B200_H
#define KREA2_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error classes of krea2::Error (src/error.rs:10-29). */
typedef enum krea2_status {
    KREA2_OK = 0,
    KREA2_INVALID_ARGUMENT = 1,
    KREA2_CANCELLED = 2,
    KREA2_POISONED = 3,
    KREA2_RUNTIME = 4, /* a CUDA call failed, or a kernel reported a bounded wait that ran out */
    KREA2_INTERNAL = 5
} krea2_status;

typedef void *krea2_stream; /* cudaStream_t */

/* Thread-local message of the last failing call on this thread ("" when none). */
const char *krea2_last_error(void);
/* Library version string. */
const char *krea2_version(void);
/* Reads and clears the device-side status word the GEMM sets when one of its bounded
 * waits gives up (0 = healthy).  Synchronises the device. */
int krea2_device_status(int *host_status);

/* ---------------------------------------------------------------- activation prologues */

/* kernels/prepare_norm_i8.loom:11-22.  h bf16 [tokens][width]; norm_scale, mod_scale,
 * mod_shift f32 [width]; q int8 [tokens][out_stride]; q_scale f32 [tokens].
 * width in 2048..32768 step 2048; out_stride multiple of 64, >= width. */
int krea2_prepare_norm_i8(krea2_stream stream, size_t tokens, const void *h, const float *norm_scale,
                          const float *mod_scale, const float *mod_shift, void *q, float *q_scale,
                          size_t width, size_t out_stride, float eps);

/* kernels/prepare_gated_i8.loom:11-22.  attn f16 [tokens][width]; gate f16 rows of pitch
 * gate_stride (multiple of 256, >= width) whose first `width` columns are used. */
int krea2_prepare_gated_i8(krea2_stream stream, size_t tokens, const void *attn, const void *gate, void *q,
                           float *q_scale, size_t width, size_t out_stride, size_t gate_stride);

/* kernels/prepare_plain_i8.loom:10-19.  h f16 [tokens][width]. */
int krea2_prepare_plain_i8(krea2_stream stream, size_t tokens, const void *h, void *q, float *q_scale,
                           size_t width, size_t out_stride);

/* ---------------------------------------------------------------- int8 GEMMs
 * a int8 [m][k_stride], w int8 [n_size][k_stride] (both K-contiguous), scale f32 [n_size]
 * (per output channel), a_scale f32 [m] (per token).  k_size multiple of 128 (64 for the
 * 256x256 export), n_size multiple of 128 (256), k_stride multiple of 64 and >= k_size,
 * m in 1..2^24.  m_group (1..4) and schedule_rows (0/1) are the reference's scheduling
 * hints: range-checked, without numerical effect. */

/* kernels/gemm_i8_256.loom:14-36.  c f16 [m][n_size] = f16(bf16((acc*scale[n])*a_scale[m])). */
int krea2_gemm_i8_256(krea2_stream stream, size_t m, const void *a, const void *w, const float *scale,
                      const float *a_scale, void *c, size_t k_size, size_t k_stride, size_t n_size,
                      size_t m_group);

/* kernels/gemm_i8_resid_256.loom:14-36.  c bf16 [m][n_size] in/out:
 * c = bf16(c + bf16(gate[n] * bf16((acc*scale[n])*a_scale[m]))); gate f32 [n_size]. */
int krea2_gemm_i8_resid_256(krea2_stream stream, size_t m, const void *a, const void *w, const float *scale,
                            const float *a_scale, void *c, const float *gate, size_t k_size, size_t k_stride,
                            size_t n_size, size_t m_group);

/* kernels/gemm_i8_resid_256x256.loom:16-42.  Same arithmetic on the wide tile's constraints. */
int krea2_gemm_i8_resid_256x256(krea2_stream stream, size_t m, const void *a, const void *w,
                                const float *scale, const float *a_scale, void *c, const float *gate,
                                size_t k_size, size_t k_stride, size_t n_size, size_t m_group,
                                size_t schedule_rows);

/* kernels/gemm_i8_swiglu_256.loom:16-38.  w rows interleaved [gate o..o+15 | up o..o+15];
 * c f16 [m][n_size/2] = f16(bf16(bf16(silu(g)) * u)). */
int krea2_gemm_i8_swiglu_256(krea2_stream stream, size_t m, const void *a, const void *w, const float *scale,
                             const float *a_scale, void *c, size_t k_size, size_t k_stride, size_t n_size,
                             size_t m_group);

/* The hand-off between the gate|up GEMM and the down projection's prologue, fused (the reference launches
 * gemm_i8_swiglu_256 then prepare_plain_i8, src/session/mod.rs:803-826; it has no fused form).
 * krea2_gemm_i8_swiglu_rotated_256 is krea2_gemm_i8_swiglu_256 whose epilogue also applies the first three of
 * prepare_plain_i8's four rotation stages (strides 1, 4, 16; each with its quarter and f16 rounding,
 * kernels/prepare_plain_i8.loom:112-232) to the 64 consecutive outputs a thread owns, under the next tile's main
 * loop; c then holds the f16 row after three stages.  krea2_prepare_rotated_i8 takes such a row through the last
 * stage (stride 64, :259-278), the row maximum and the codes (:294-313).  Together they write exactly the q and
 * q_scale that krea2_gemm_i8_swiglu_256 followed by krea2_prepare_plain_i8 writes.  n_size must be a multiple
 * of 256. */
int krea2_gemm_i8_swiglu_rotated_256(krea2_stream stream, size_t m, const void *a, const void *w, const float *scale,
                                     const float *a_scale, void *c, size_t k_size, size_t k_stride, size_t n_size,
                                     size_t m_group);
int krea2_prepare_rotated_i8(krea2_stream stream, size_t tokens, const void *h, void *q, float *q_scale, size_t width,
                             size_t out_stride);

/* The q|k|v|gate product and the QK-norm + RoPE launch that follows it, fused (the reference launches gemm_i8_256
 * then rope_qknorm_f16, src/session/mod.rs:702-734; it has no fused form).  The columns are heads of 128
 * channels: q_heads query heads, kv_heads key heads, kv_heads value heads, then whatever is left (the attention
 * gate).  An epilogue thread owns one row of one head, so the head's RMS norm (1 + scale, bf16), the rotation by
 * the token's angles (bf16) and the f16 store happen on the values gemm_i8_256 would have written, in the
 * standalone kernel's order of operations: q_out f16 [m][q_heads*128], k_out and v_out f16 [m][kv_heads*128]
 * receive exactly what krea2_rope_qknorm_f16 writes from gemm_i8_256's output, and only the columns past the
 * value heads are written to c (f16 [m][n_size]).  q_norm, k_norm f32 [128]; cos_table, sin_table f32 [m][128].
 * n_size must be a multiple of 256. */
int krea2_gemm_i8_rope_256(krea2_stream stream, size_t m, const void *a, const void *w, const float *scale,
                           const float *a_scale, void *c, const float *q_norm, const float *k_norm,
                           const float *cos_table, const float *sin_table, void *q_out, void *k_out, void *v_out,
                           size_t k_size, size_t k_stride, size_t n_size, size_t m_group, size_t q_heads,
                           size_t kv_heads, float eps);

/* The raw i32 accumulators acc [m][n_size] of the same contraction, for parity checks
 * (the reference's tests recompute them on the CPU, tests/quantized.rs:203-211). */
int krea2_gemm_i8_acc(krea2_stream stream, size_t m, const void *a, const void *w, int32_t *acc,
                      size_t k_size, size_t k_stride, size_t n_size);

/* ---------------------------------------------------------------- the rest of a block
 * The three launches between the q|k|v|gate GEMM and the gated prologue
 * (src/session/mod.rs:714-755).  Not W8A8 products; they make a session forward a real block. */

/* kernels/rope_qknorm_f16.loom:13-27.  qkv f16 [tokens][row_stride] (q heads at column 0, k heads
 * at k_offset, v heads right after k); q_scale, k_scale f32 [128]; cos, sin f32 [tokens][128];
 * q_out f16 [tokens][q_heads*128], k_out and v_out f16 [tokens][kv_heads*128]. */
int krea2_rope_qknorm_f16(krea2_stream stream, size_t tokens, const void *qkv, const float *q_scale,
                          const float *k_scale, const float *cos_table, const float *sin_table, void *q_out,
                          void *k_out, void *v_out, size_t row_stride, size_t q_heads, size_t kv_heads,
                          size_t k_offset, float eps);

/* kernels/native/v_transpose.loom.  x f16 [rows][width] -> out f16 [width][row_capacity]; columns
 * rows..row_capacity of `out` are left as they are except inside the last 32-row tile, where
 * they are written as zero. */
int krea2_v_transpose(krea2_stream stream, size_t rows, const void *x, void *out, size_t width, size_t row_capacity);

/* ---------------------------------------------------------------- around the block chain
 * The pointwise kernels of the sampler loop and its sigma schedule (src/pipeline/mod.rs:340-357). */

/* kernels/native/modulation.loom (launched at src/models/graph.rs:405-425): y[i] = bf16(x[i % xsize] +
 * tables[i]) as f32, i < count - the f32 [layers][6][width] table a session reads, from this
 * timestep's bf16 vector x [xsize] and the bf16 block tables [count]. */
int krea2_modulation(krea2_stream stream, size_t count, const void *x, const void *tables, float *y, size_t xsize);

/* kernels/native/euler.loom (src/ops/mod.rs:373-390): sample = bf16(sample + bf16(bf16(delta) * velocity))
 * in place; sample, velocity bf16 [count]. */
int krea2_euler(krea2_stream stream, size_t count, float delta, void *sample, const void *velocity);

/* kernels/native/guidance.loom (src/ops/mod.rs:392-410): cond = bf16(cond + bf16(scale * bf16(cond - uncond)))
 * in place; cond, uncond bf16 [count]. */
int krea2_guidance(krea2_stream stream, size_t count, float scale, void *cond, const void *uncond);

/* src/pipeline/schedule.rs:11-35: the shift of an image with that many tokens; the sigma at `step` of
 * `steps` (zero at step == steps); the sigma a step lands on when the run ends after step `last`. */
double krea2_schedule_dynamic_mu(size_t image_tokens);
float krea2_schedule_sigma(size_t step, size_t steps, double mu);
float krea2_schedule_next_sigma(size_t step, size_t last, size_t steps, double mu);

/* kernels/attention_gqa_lds_f16_wmma.loom:18-41 (and the _q32 sibling, the same function on
 * 32-row groups).  q f16 [tokens][q_stride], k f16 [tokens][kv_stride], v_transposed f16
 * [kv_stride][token_capacity] with finite (zero) headroom past `tokens`, out f16
 * [tokens][out_stride]; query head h reads key/value head h / (q_stride / kv_stride). */
int krea2_attention_gqa_lds_f16_wmma(krea2_stream stream, size_t tokens, size_t kv_heads, const void *q,
                                     const void *k, const void *v_transposed, void *out, size_t q_stride,
                                     size_t kv_stride, size_t out_stride, size_t token_capacity, float scale);
int krea2_attention_gqa_lds_f16_wmma_q32(krea2_stream stream, size_t tokens, size_t kv_heads, const void *q,
                                         const void *k, const void *v_transposed, void *out, size_t q_stride,
                                         size_t kv_stride, size_t out_stride, size_t token_capacity, float scale);

/* ---------------------------------------------------------------- column-sharded GEMMs
 * New with this library (the reference runs on one device).  Device r of `world` holds rows
 * [r*N/world, (r+1)*N/world) of a weight and its scales, computes the matching column slab of
 * the output and stores every finished vector straight into ALL devices' copies of the full
 * output tensor through peer-mapped pointers, so the all-gather rides in the epilogue's stores
 * over NVLink instead of following as a separate collective.  Each output element is still one
 * full-K dot product of one CTA, so sharded results are bit-identical to the single-device ones.
 * When the last CTA of a launch has finished, slot `rank` of every destination's flag array is
 * set to `epoch` (+ *epoch_base); krea2_shard_wait makes a stream wait (bounded, 2 s, then the device status
 * word is raised) until all `world` slots of the local array have reached `epoch`. */
typedef struct krea2_shard {
    uint32_t world;     /* destination buffers, 1..8 */
    uint32_t rank;      /* this launch's flag slot; dest[rank] is this device's own buffer (and the
                           source of the residual for the resid kind) */
    void *dest[8];      /* every device's copy of the full output [m][pitch], 16-bit elements */
    size_t pitch;       /* elements per row of the full output (N, or N/2 for swiglu) */
    size_t offset;      /* first output column of this shard; multiple of 16 */
    uint32_t *flags[8]; /* per destination, `world` u32 slots; NULL entries are not signalled */
    uint32_t epoch;     /* value published when this launch's stores are complete */
    uint32_t *counter;  /* u32 on this device, zero before the first launch (the kernel re-zeroes it) */
    const uint32_t *epoch_base; /* optional device word added to `epoch` when publishing: a chain captured
                                   in a CUDA graph keeps its epochs relative and advances this word (with
                                   krea2_shard_advance) at the end of every replay */
} krea2_shard;

enum { KREA2_SHARD_PLAIN = 0, KREA2_SHARD_RESID = 1, KREA2_SHARD_SWIGLU = 2 };

/* n_size = rows of this shard of w (interleaved gate|up rows for swiglu, a multiple of 128). */
int krea2_gemm_i8_sharded(krea2_stream stream, int kind, size_t m, const void *a, const void *w, const float *scale,
                          const float *a_scale, const float *gate, size_t k_size, size_t k_stride, size_t n_size,
                          const krea2_shard *shard);
int krea2_shard_wait(krea2_stream stream, const uint32_t *flags, uint32_t world, uint32_t epoch,
                     const uint32_t *epoch_base);
int krea2_shard_advance(krea2_stream stream, uint32_t *epoch_base, uint32_t delta);

/* ---------------------------------------------------------------- token-sharded blocks
 * New with this library.  Every prologue, GEMM row and query row of a block belongs to one token, so with the
 * weights replicated device r can run rows [first_row, first_row + tokens) of the sequence through the whole
 * block alone; the one thing a token needs from the others is their keys and values.  The sharded QK-norm +
 * RoPE launch therefore stores its K and V rows into EVERY device's full-length K and V tensors through
 * peer-mapped pointers (the all-gather rides in the kernel's own stores over NVLink) and publishes `epoch` in
 * slot `rank` of every device's flag array when its last block has finished; krea2_shard_wait holds a stream
 * until all `world` slots have arrived, and the attention launch then takes this device's query rows against
 * all keys.  Per block that moves 2 * tokens * kv_heads * 128 f16 values per device instead of the column-sharded
 * chain's full activations.  Results are bit-identical to the single-device block. */
typedef struct krea2_row_shard {
    uint32_t world;     /* devices, 1..8 */
    uint32_t rank;      /* this device's flag slot */
    void *k_dest[8];    /* every device's K tensor, f16 [all tokens][kv_heads * 128] */
    void *v_dest[8];    /* every device's V tensor, same shape */
    size_t first_row;   /* row of the full sequence that this launch's first token is */
    uint32_t *flags[8]; /* per device, `world` u32 slots; NULL entries are not signalled */
    uint32_t epoch;     /* value published when this launch's stores are complete */
    uint32_t *counter;  /* u32 on this device, zero before the first launch (the kernel re-zeroes it) */
    const uint32_t *epoch_base; /* optional device word added to `epoch` (see krea2_shard) */
} krea2_row_shard;

/* krea2_rope_qknorm_f16 on this device's rows: q_out holds the local rows, K and V go to the shard's
 * destinations at row first_row + local row; cos/sin are the local rows' tables. */
int krea2_rope_qknorm_f16_sharded(krea2_stream stream, size_t tokens, const void *qkv, const float *q_scale,
                                  const float *k_scale, const float *cos_table, const float *sin_table, void *q_out,
                                  size_t row_stride, size_t q_heads, size_t kv_heads, size_t k_offset, float eps,
                                  const krea2_row_shard *shard);
/* Publishes the shard's epoch in every device's flag slot once the stream's earlier work has finished (no
 * rows are stored; k_dest / v_dest / first_row / counter are ignored): the fence that ends a sharded forward,
 * after which no device still reads what the next forward's launches overwrite. */
int krea2_shard_signal(krea2_stream stream, const krea2_row_shard *shard);
/* Grouped-query attention of `q_rows` query rows (q and out hold just those rows) against all `tokens` keys
 * and values: krea2_attention_gqa_lds_f16_wmma is this call with q_rows = tokens. */
int krea2_attention_gqa_f16_rows(krea2_stream stream, size_t q_rows, size_t tokens, size_t kv_heads, const void *q,
                                 const void *k, const void *v_transposed, void *out, size_t q_stride, size_t kv_stride,
                                 size_t out_stride, size_t token_capacity, float scale);

/* bf16 <-> f16 transport of src/training/quantized.rs:63-72,102-110 (`lora_transport`,
 * reverse = 1: bf16 -> f16, reverse = 2: f16 -> bf16). */
int krea2_lora_transport(krea2_stream stream, size_t elements, const void *src, void *dst, int reverse);

/* Quantized::forward (src/training/quantized.rs:51-112) as one call: x bf16 [rows][inputs] ->
 * out bf16 [rows][outputs] through the transport, prepare_plain_i8, gemm_i8_256 and the transport
 * back; weight int8 [outputs][gemm_pitch(inputs)], scales f32 [outputs].  The four intermediates
 * the reference takes from its buffer pool (:55-58) live in `workspace`, a device buffer of at
 * least krea2_quantized_workspace_bytes(rows, inputs, outputs) bytes. */
size_t krea2_quantized_workspace_bytes(size_t rows, size_t inputs, size_t outputs);
int krea2_quantized_forward(krea2_stream stream, size_t rows, const void *x, const void *weight,
                            const float *scales, void *out, size_t inputs, size_t outputs, void *workspace,
                            size_t workspace_bytes);

/* The same projection for callers that must not allocate.  No counterpart in the reference.
 * Some hosts cannot hand this library a workspace: a plugin inside an engine that froze its
 * device-memory arena at start-up, a serving loop whose allocator must not be entered on the
 * request path, code that runs where cudaMalloc would synchronise or fail.  For them the four
 * intermediates live in a 4 MiB array that is part of the library image (every GPU that loads
 * the library carries it until the process exits), so this call needs nothing but its inputs
 * and outputs and itself performs no cudaMalloc, cudaFree or other allocating call.
 *  - Limit: krea2_quantized_workspace_bytes(rows, inputs, outputs) must not exceed
 *    krea2_quantized_static_workspace_bytes() (4 MiB; e.g. 64 rows of 6144 -> 6144, 16 rows of
 *    16384 -> 6144).  Larger calls are refused with KREA2_INVALID_ARGUMENT.
 *  - The first call on each device resolves the array's device address (with that device
 *    current).  That lookup may make the CUDA runtime load the library's device image, which is
 *    where the 4 MiB are reserved, so "allocates nothing" holds from the second call on: make the
 *    first call per device at start-up, outside any stream capture.
 *  - The stream and the buffers must belong to the device that is current in the calling
 *    thread; a call that mixes devices is refused with KREA2_INVALID_ARGUMENT.
 *  - All calls on a device share the one array and it keeps the previous call's bytes.  Every
 *    byte that is read is written earlier in the same call, so nothing needs clearing; but two
 *    calls that overlap on the GPU (different streams, or graph branches) race on it. */
size_t krea2_quantized_static_workspace_bytes(void);
int krea2_quantized_forward_static(krea2_stream stream, size_t rows, const void *x, const void *weight,
                                   const float *scales, void *out, size_t inputs, size_t outputs);

/* ---------------------------------------------------------------- generic dispatch
 * Ops::launch (src/ops/mod.rs:673-693): kernel by stem, config keys by name, packed
 * scalars, buffers in binding order, and the launch geometry the reference would use
 * (checked against the kernel's rules, then ignored: the B200 kernels size their own grid). */
typedef struct krea2_config_entry {
    const char *key; /* e.g. "k_size"; "eps" takes its value from the float field */
    uint64_t value;
    float fvalue;
} krea2_config_entry;

typedef struct krea2_binding {
    void *ptr;    /* device pointer */
    size_t bytes; /* extent the kernel may touch from ptr */
} krea2_binding;

int krea2_launch(krea2_stream stream, const char *name, const krea2_config_entry *config, size_t config_count,
                 const uint64_t *indices, size_t index_count, const krea2_binding *bindings,
                 size_t binding_count, size_t grid_x, size_t grid_y, uint32_t threads);

/* ---------------------------------------------------------------- launch-shape rules
 * src/kernels/shape.rs:8-112. */
size_t krea2_shape_tokens_min(void);
size_t krea2_shape_tokens_max(void);
size_t krea2_shape_capacity(size_t tokens);
size_t krea2_shape_gemm_pitch(size_t k);
size_t krea2_shape_gemm_grid_rows(size_t tokens);
size_t krea2_shape_gemm_m_group(void);
int krea2_shape_gemm_schedule_rows(size_t tokens);
size_t krea2_shape_attention_rows(size_t tokens);
/* tile of a bundle stem ("gemm_qkvg", "gemm_gu", "gemm_wo", "gemm_down"): columns and threads. */
size_t krea2_shape_gemm_tile_columns(const char *stem);
uint32_t krea2_shape_gemm_tile_threads(const char *stem);
/* kernel source name of a family on that stem's tile (shape::gemm_source). */
const char *krea2_shape_gemm_source(const char *family, const char *stem);

/* ---------------------------------------------------------------- resident session
 * krea2::session::Session (src/session/mod.rs:147-588) over synthetic or caller-supplied
 * weights laid out by the checkpoint plan's rules (src/checkpoint/plan.rs:88-226,
 * src/session/weights.rs:47-125). */
typedef struct krea2_dims {
    size_t hidden;   /* residual width d            (reference: 6144)  */
    size_t kv_heads; /* key/value heads             (reference: 12)    */
    size_t head_dim; /* channels per head           (reference: 128)   */
    size_t inter;    /* SwiGLU inner width          (reference: 16384) */
} krea2_dims;

typedef struct krea2_weights krea2_weights;
typedef struct krea2_session krea2_session;

/* Session::validate_dimensions (src/session/mod.rs:278-287): no device is touched. */
int krea2_session_validate_dimensions(size_t tokens, size_t layers);

/* Bytes of the one device allocation that holds `layers` blocks at kernel pitches, each
 * span starting on a 256-byte boundary in name order (plan.rs:135-141). */
int krea2_weights_plan_bytes(const krea2_dims *dims, size_t layers, size_t *bytes);
/* Allocates that block on the current device.  krea2_weights_locate gives the device
 * address and byte length of a span by the plan's names ("blocks.3.qkvg.q", "blocks.3.gu.s",
 * "blocks.0.prenorm", ...; session/weights.rs:112-125). */
int krea2_weights_create(const krea2_dims *dims, size_t layers, krea2_weights **out);
int krea2_weights_locate(const krea2_weights *weights, const char *name, void **ptr, size_t *bytes);
/* Fills every span with seeded synthetic values on the device: int8 rows uniform in
 * [-127, 127], channel scales uniform in [1e-3, 1e-2], norm scales ~N(0, 0.1). */
int krea2_weights_fill_synthetic(krea2_weights *weights, uint64_t seed, krea2_stream stream);
/* Host-side upload of one span (rows are re-pitched by the caller's layout = plan layout). */
int krea2_weights_upload(krea2_weights *weights, const char *name, const void *host_bytes, size_t bytes,
                         krea2_stream stream);
/* Blocking read of one span back into host memory (the same layout upload takes). */
int krea2_weights_download(const krea2_weights *weights, const char *name, void *host_bytes, size_t bytes,
                           krea2_stream stream);
void krea2_weights_retain(krea2_weights *weights);
void krea2_weights_release(krea2_weights *weights);

/* ---------------------------------------------------------------- checkpoint ingestion
 * A ComfyUI int8 ConvRot checkpoint (.safetensors) mapped read-only and indexed under the transformer's
 * own tensor names (src/checkpoint/file.rs), the device layout derived from it (src/checkpoint/plan.rs)
 * and the upload (src/session/weights.rs).  Everything up to krea2_weights_load_checkpoint is host work:
 * a malformed file is refused without touching a device. */
typedef struct krea2_checkpoint krea2_checkpoint;

/* Plan::span (plan.rs:23-43).  segments = checkpoint row ranges that fill it in order (0 for the spans
 * assembled on the host: gathered channel scales, bf16 norm vectors); file_bytes = bytes before padding. */
typedef struct krea2_span_info {
    size_t device_offset, device_bytes, rows, row_bytes, device_row_bytes, segments, file_bytes;
} krea2_span_info;

/* Checkpoint::open (file.rs:72-90): the extension must be .safetensors; an unreadable or inconsistent
 * file is KREA2_INVALID_ARGUMENT with a message that starts "cannot read <path>".  A namespace every
 * tensor shares in front of "blocks.0.attn.wq.weight" is removed (file.rs:39-57). */
int krea2_checkpoint_open(const char *path, krea2_checkpoint **out);
void krea2_checkpoint_close(krea2_checkpoint *checkpoint);
int krea2_checkpoint_has(const krea2_checkpoint *checkpoint, const char *name);
/* Blocks counted by their attention weights (file.rs:119-125). */
size_t krea2_checkpoint_block_count(const krea2_checkpoint *checkpoint);
/* Tensor names in sorted order; returns the count, fills at most `capacity` pointers. */
size_t krea2_checkpoint_names(const krea2_checkpoint *checkpoint, const char **names, size_t capacity);
/* Checkpoint::get (file.rs:103-109): dtype string, shape, raw little-endian bytes inside the mapping. */
int krea2_checkpoint_tensor(const krea2_checkpoint *checkpoint, const char *name, const char **dtype,
                            const size_t **shape, size_t *rank, const void **bytes, size_t *byte_count);
/* Plan::for_checkpoint (plan.rs:85-144); the plan is derived on first use and kept. */
int krea2_checkpoint_plan(krea2_checkpoint *checkpoint, size_t *total_bytes, size_t *layers, size_t *span_count);
int krea2_checkpoint_span_name(krea2_checkpoint *checkpoint, size_t index, const char **name);
int krea2_checkpoint_span(krea2_checkpoint *checkpoint, const char *name, krea2_span_info *info);
int krea2_checkpoint_segment(krea2_checkpoint *checkpoint, const char *span, size_t index, const char **tensor,
                             size_t *row_begin, size_t *row_end);
/* The span as it lies on the device (rows at the device pitch, padding zero), written to host memory. */
int krea2_checkpoint_assemble(krea2_checkpoint *checkpoint, const char *span, void *host_bytes, size_t bytes);
/* The block shape the file's tensors declare. */
int krea2_checkpoint_dims(krea2_checkpoint *checkpoint, krea2_dims *dims, size_t *layers);
/* Session::validate (src/session/mod.rs:249-261): dimensions, then the checkpoint's header and layout;
 * no device is touched (tests/constructor.rs). */
int krea2_session_validate(const char *checkpoint_path, size_t tokens, size_t layers);
/* Weights::load (src/session/weights.rs:40-98): allocates the block on the current device and fills it. */
int krea2_weights_load_checkpoint(krea2_checkpoint *checkpoint, krea2_stream stream, krea2_weights **out);

/* Session::with_weights (src/session/mod.rs:265-276): buffers at shape::capacity(tokens)
 * rows, zero-filled headroom, bound to `stream` (calls on another stream are refused,
 * :375-380). */
int krea2_session_create(krea2_stream stream, krea2_weights *weights, size_t tokens, size_t layers,
                         krea2_session **out);
void krea2_session_destroy(krea2_session *session);
size_t krea2_session_tokens(const krea2_session *session);
size_t krea2_session_layers(const krea2_session *session);
/* Session::set_profile (:367-373): returns the previous setting. */
int krea2_session_set_profile(krea2_session *session, int enable);
/* After a profiled forward: per-stage device milliseconds, stage labels as the reference's
 * (:461-494).  Returns the number of stages written (<= capacity). */
size_t krea2_session_stage_profile(const krea2_session *session, const char **labels, double *millis,
                                   size_t capacity);

/* Session::run (:502-540): HOST x bf16 [tokens][hidden] in/out, HOST mods f32
 * [layers][6][hidden], HOST cos/sin f32 [tokens][head_dim]; uploads, runs blocks
 * first_block..first_block+block_count eagerly, reads x back (blocking).
 * block_count 0 means "to the last layer". */
int krea2_session_run(krea2_session *session, krea2_stream stream, uint16_t *host_x, const float *host_mods,
                      const float *host_cos, const float *host_sin, size_t first_block, size_t block_count);

/* Session::run_device (:553-588): DEVICE x and mods; copies them into the session's fixed
 * buffers, replays the recorded graph of all layers, copies x back; asynchronous on `stream`.
 * x_bytes / mods_bytes are the extents of the caller's views. */
int krea2_session_run_device(krea2_session *session, krea2_stream stream, void *x, size_t x_bytes,
                             const void *mods, size_t mods_bytes, const float *host_cos,
                             const float *host_sin);

/* Device address of a session buffer by name ("x", "a_q", "a_s", "fused", "attn_gu", "mods",
 * "q", "k", "v", "v_transposed"), for tests that compare intermediates. */
int krea2_session_buffer(const krea2_session *session, const char *name, void **ptr, size_t *bytes);

/* Chooses between the full block (1, the default where the head shape allows: 128 channels per
 * head) and the W8A8 chain alone (0): QK-norm + RoPE, V transpose and attention are left out and
 * the gated prologue reads the query columns of the q|k|v|gate output in place of an attention
 * output, which keeps every remaining stage reproducible bit for bit on a CPU.  Returns the previous setting; a recorded graph is dropped. */
int krea2_session_set_attention(krea2_session *session, int enable);

/* Chooses how the SwiGLU output reaches the down projection's prologue: 0 = the reference's two launches
 * (gemm_i8_swiglu_256, prepare_plain_i8), 1 = the fused pair (krea2_gemm_i8_swiglu_rotated_256,
 * krea2_prepare_rotated_i8).  The results are the same bits.  A new session takes the build's default unless the
 * environment sets KREA2_FUSED_ROTATION=0 or 1.  Returns the previous setting; a recorded graph is dropped. */
int krea2_session_set_fused_rotation(krea2_session *session, int enable);

/* Chooses whether the q|k|v|gate GEMM also does the QK-norm + RoPE launch's work (krea2_gemm_i8_rope_256: ten
 * launches per block instead of eleven; only with attention on).  The results are the same bits.  A new session
 * takes the build's default unless the environment sets KREA2_FUSED_ROPE=0 or 1.  Returns the previous setting;
 * a recorded graph is dropped. */
int krea2_session_set_fused_rope(krea2_session *session, int enable);

/* Number of kernels of this library that one forward of `layers` blocks launches. */
size_t krea2_session_launches_per_forward(const krea2_session *session);

#ifdef __cplusplus
}
#endif
#endif /* KREA2_B200_H */
