// The resident block session of krea2-hrx (src/session/mod.rs) on CUDA: one device
// allocation for the weights at kernel pitches (src/session/weights.rs, src/checkpoint/plan.rs),
// fixed scratch buffers sized by shape::capacity, the per-block launch chain, and a CUDA graph
// of the whole chain that every device-side forward replays.
//
// A block is the reference's eleven launches (src/session/mod.rs:671-840): prepare_norm, qkv|gate
// GEMM, QK-norm + RoPE, V transpose, fp16 attention, prepare_gated, wo GEMM + residual,
// prepare_norm, gate|up GEMM + SwiGLU, prepare_plain, down GEMM + residual.  With attention
// switched off (krea2_session_set_attention) the three launches that are not W8A8 products are
// left out and the gated prologue reads the query columns of the fused buffer in place of an
// attention output: the W8A8 chain alone, which the CPU oracle reproduces bit for bit.
#include <atomic>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "common.cuh"

using namespace krea2;

namespace {

size_t pitch_of(size_t k) { return krea2_shape_gemm_pitch(k); }

struct Span {
    size_t offset = 0, bytes = 0;
    size_t rows = 0, row_bytes = 0, pitch = 0;  // rows == 0: a plain f32 vector
    char kind = 'v';                            // 'q' int8 rows, 's' channel scales, 'n' norm scale vector
};

}  // namespace

struct krea2_weights {
    krea2_dims dims{};
    size_t layers = 0;
    size_t qkvg = 0;
    std::map<std::string, Span> spans;  // name order = device order (plan.rs:135-141)
    size_t total_bytes = 0;
    uint8_t *base = nullptr;
    int device = 0;
    std::atomic<int> references{1};
};

namespace {

int check_dims(const krea2_dims *d) {
    KREA2_REQUIRE(d, "dims is null");
    KREA2_REQUIRE(d->hidden >= 2048 && d->hidden <= 32768 && d->hidden % 2048 == 0,
                  "hidden %zu must be a multiple of 2048 in 2048..32768", d->hidden);
    KREA2_REQUIRE(d->inter >= 2048 && d->inter <= 32768 && d->inter % 2048 == 0,
                  "inter %zu must be a multiple of 2048 in 2048..32768", d->inter);
    KREA2_REQUIRE(d->head_dim >= 32 && d->head_dim % 32 == 0 && d->kv_heads >= 1, "bad head shape");
    KREA2_REQUIRE((2 * d->kv_heads * d->head_dim) % 256 == 0 && 2 * d->hidden + 2 * d->kv_heads * d->head_dim <= 32768,
                  "the fused q|k|v|gate width must be a multiple of 256 up to 32768");
    return KREA2_OK;
}

// The device layout of src/checkpoint/plan.rs:88-144 for `layers` blocks.
void plan(krea2_weights &w) {
    const krea2_dims &d = w.dims;
    w.qkvg = d.hidden + 2 * d.kv_heads * d.head_dim + d.hidden;  // src/session/mod.rs:43
    auto rows = [&](const std::string &name, size_t n, size_t k) {
        Span q;
        q.rows = n, q.row_bytes = k, q.pitch = pitch_of(k), q.bytes = n * q.pitch, q.kind = 'q';
        w.spans[name + ".q"] = q;
        Span s;
        s.bytes = n * 4, s.kind = 's';
        w.spans[name + ".s"] = s;
    };
    auto vec = [&](const std::string &name, size_t n) {
        Span v;
        v.bytes = n * 4, v.kind = 'n';
        w.spans[name] = v;
    };
    for (size_t i = 0; i < w.layers; i++) {
        const std::string p = "blocks." + std::to_string(i);
        rows(p + ".qkvg", w.qkvg, d.hidden);
        rows(p + ".wo", d.hidden, d.hidden);
        rows(p + ".down", d.hidden, d.inter);
        rows(p + ".gu", 2 * d.inter, d.hidden);
        vec(p + ".prenorm", d.hidden);
        vec(p + ".postnorm", d.hidden);
        vec(p + ".qnorm", d.head_dim);
        vec(p + ".knorm", d.head_dim);
    }
    size_t total = 0;
    for (auto &entry : w.spans) {
        entry.second.offset = total;
        total += (entry.second.bytes + 255) / 256 * 256;
    }
    w.total_bytes = total;
}

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x += 0x9e3779b97f4a7c15ull;
    x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
    x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
    return x ^ (x >> 31);
}

// Seeded synthetic weights, a pure function of (seed, span offset, element index).
__global__ void fill_rows_kernel(int8_t *dst, size_t rows, size_t row_bytes, size_t pitch, uint64_t seed) {
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    size_t words = rows * (pitch / 4);
    for (; i < words; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        size_t row = i / (pitch / 4), col = (i % (pitch / 4)) * 4;
        uint64_t r = mix64(seed + row * row_bytes + col);
        uint32_t word = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            int v = static_cast<int>((r >> (16 * b)) & 0xffff) % 255 - 127;
            if (col + b >= row_bytes) v = 0;
            word |= (static_cast<uint32_t>(v) & 0xffu) << (8 * b);
        }
        reinterpret_cast<uint32_t *>(dst)[i] = word;
    }
}
__global__ void fill_vector_kernel(float *dst, size_t n, uint64_t seed, int normal) {
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint64_t r = mix64(seed + i);
    float u1 = (static_cast<float>(r & 0xffffff) + 0.5f) * (1.0f / 16777216.0f);
    float u2 = (static_cast<float>((r >> 24) & 0xffffff) + 0.5f) * (1.0f / 16777216.0f);
    if (normal)
        dst[i] = 0.1f * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
    else
        dst[i] = 1e-3f + 9e-3f * u1;
}

struct Stage {
    const char *label;
    double millis = 0.0;
};

}  // namespace

struct krea2_session {
    cudaStream_t stream = nullptr;
    size_t tokens = 0, layers = 0, capacity = 0;
    krea2_weights *weights = nullptr;
    krea2_dims dims{};
    size_t qkvg = 0, gate_offset = 0;
    // src/session/mod.rs:76-93
    uint8_t *x = nullptr, *a_q = nullptr, *fused = nullptr, *attn_gu = nullptr;
    uint8_t *q = nullptr, *k = nullptr, *v = nullptr, *v_transposed = nullptr;
    float *a_s = nullptr, *mods = nullptr, *cos = nullptr, *sin = nullptr;
    size_t x_bytes = 0, a_q_bytes = 0, fused_bytes = 0, attn_gu_bytes = 0, mods_bytes = 0, rope_bytes = 0;
    size_t q_bytes = 0, kv_bytes = 0;
    cudaGraphExec_t graph = nullptr;
    bool profile = false, poisoned = false;
    bool attention = true;  // false: the W8A8 chain alone, the query columns in the attention output's place
    bool fused_rotation = false;  // the gate|up epilogue starts the down projection's rotation (same bits either way)
    bool fused_rope = false;      // the q|k|v|gate epilogue does the QK-norm + RoPE launch's work (same bits either way)
    bool dependent_launch = false;  // the chain's launches let the next kernel's blocks start under the last blocks of this one
    bool rope_valid = false;
    uint64_t rope_print[2] = {0, 0};
    std::vector<Stage> stages;
    std::vector<cudaEvent_t> events;
};

namespace {

// FNV-1a over the table bytes (src/session/mod.rs:48-56).
uint64_t fingerprint(const float *values, size_t count) {
    uint64_t hash = 0xcbf29ce484222325ull;
    const uint8_t *bytes = reinterpret_cast<const uint8_t *>(values);
    for (size_t i = 0; i < count * 4; i++) {
        hash ^= bytes[i];
        hash *= 0x100000001b3ull;
    }
    return hash;
}

struct BlockPointers {
    const int8_t *qkvg_q, *wo_q, *gu_q, *down_q;
    const float *qkvg_s, *wo_s, *gu_s, *down_s, *prenorm, *postnorm, *qnorm, *knorm;
};

int locate(const krea2_weights *w, const std::string &name, size_t expect_bytes, const void **out) {
    auto it = w->spans.find(name);
    if (it == w->spans.end()) return fail(KREA2_INVALID_ARGUMENT, "no span named %s", name.c_str());
    if (it->second.bytes != expect_bytes)
        return fail(KREA2_INVALID_ARGUMENT, "%s spans %zu bytes, expected %zu", name.c_str(), it->second.bytes,
                    expect_bytes);
    *out = w->base + it->second.offset;
    return KREA2_OK;
}

int block_pointers(const krea2_session *s, size_t index, BlockPointers *b) {
    const krea2_dims &d = s->dims;
    const std::string p = "blocks." + std::to_string(index);
    const size_t ph = pitch_of(d.hidden), pi = pitch_of(d.inter);
    const void *ptr = nullptr;
#define KREA2_AT(field, type, name, bytes)                        \
    if (int status = locate(s->weights, p + name, bytes, &ptr)) return status; \
    b->field = static_cast<type>(ptr);
    KREA2_AT(qkvg_q, const int8_t *, ".qkvg.q", s->qkvg * ph)
    KREA2_AT(qkvg_s, const float *, ".qkvg.s", s->qkvg * 4)
    KREA2_AT(wo_q, const int8_t *, ".wo.q", d.hidden * ph)
    KREA2_AT(wo_s, const float *, ".wo.s", d.hidden * 4)
    KREA2_AT(gu_q, const int8_t *, ".gu.q", 2 * d.inter * ph)
    KREA2_AT(gu_s, const float *, ".gu.s", 2 * d.inter * 4)
    KREA2_AT(down_q, const int8_t *, ".down.q", d.hidden * pi)
    KREA2_AT(down_s, const float *, ".down.s", d.hidden * 4)
    KREA2_AT(prenorm, const float *, ".prenorm", d.hidden * 4)
    KREA2_AT(postnorm, const float *, ".postnorm", d.hidden * 4)
    KREA2_AT(qnorm, const float *, ".qnorm", d.head_dim * 4)
    KREA2_AT(knorm, const float *, ".knorm", d.head_dim * 4)
#undef KREA2_AT
    return KREA2_OK;
}

// At most eleven launches per block (src/session/mod.rs:671-840); a profiled forward brackets
// each with an event and sums device time per label.
constexpr int kMaxStagesPerBlock = 11;
// Whether a new session hands the SwiGLU output to the down projection's prologue through the fused pair
// (krea2_gemm_i8_swiglu_rotated_256 + krea2_prepare_rotated_i8); KREA2_FUSED_ROTATION=0/1 overrides it.
constexpr bool kFusedRotationDefault = false;
// The same for the q|k|v|gate GEMM doing the QK-norm + RoPE launch's work (krea2_gemm_i8_rope_256);
// KREA2_FUSED_ROPE=0/1 overrides it.
constexpr bool kFusedRopeDefault = false;
// Whether the launches of a forward carry the programmatic-stream-serialization attribute (every launch but the
// first, and none in a profiled forward, whose events sit between the kernels); KREA2_DEPENDENT_LAUNCH=0/1
// overrides it.  The kernels wait for their predecessor before their first global access, so the results do
// not change.
constexpr bool kDependentLaunchDefault = false;

// One block's launches in the reference's order.  `events`, when given, receives one event before
// every stage and one after the last; `labels`, when given, the stage labels in launch order.
int run_block(krea2_session *s, cudaStream_t stream, size_t index, cudaEvent_t *events,
              std::vector<const char *> *labels = nullptr) {
    BlockPointers w{};
    if (int status = block_pointers(s, index, &w)) return status;
    const krea2_dims &d = s->dims;
    const size_t t = s->tokens, hidden = d.hidden, inter = d.inter;
    const size_t ph = pitch_of(hidden), pi = pitch_of(inter);
    const size_t group = krea2_shape_gemm_m_group();
    const size_t q_heads = hidden / d.head_dim, kv_width = d.kv_heads * d.head_dim;
    const float *mods = s->mods + index * 6 * hidden;  // prescale, preshift, pregate, postscale, postshift, postgate
    int stage = 0;
    auto mark = [&](const char *label) -> int {
        if (events) KREA2_CUDA(cudaEventRecord(events[stage], stream));
        if (labels && label) labels->push_back(label);
        stage++;
        return KREA2_OK;
    };
    int status = KREA2_OK;
    // The very first launch of a forward follows copies, not a kernel: it is an ordinary launch.
    const bool chain = s->dependent_launch && events == nullptr;
#define KREA2_STEP(label, call)                                 \
    if ((status = mark(label))) return status;                  \
    dependent_launches() = chain && !(index == 0 && stage == 1); \
    status = (call);                                            \
    dependent_launches() = false;                               \
    if (status) return status;
    KREA2_STEP("prepare", krea2_prepare_norm_i8(stream, t, s->x, w.prenorm, mods, mods + hidden, s->a_q, s->a_s, hidden, ph,
                                                1e-5f))
    const bool rope_in_gemm = s->attention && s->fused_rope;
    if (rope_in_gemm) {
        // The same two stages as one launch: q and k leave the GEMM's epilogue normalised and rotated.
        KREA2_STEP("gemm qkvg", krea2_gemm_i8_rope_256(stream, t, s->a_q, w.qkvg_q, w.qkvg_s, s->a_s, s->fused, w.qnorm, w.knorm,
                                                       s->cos, s->sin, s->q, s->k, s->v, hidden, ph, s->qkvg, group, q_heads,
                                                       d.kv_heads, 1e-5f))
    } else {
        KREA2_STEP("gemm qkvg",
                   krea2_gemm_i8_256(stream, t, s->a_q, w.qkvg_q, w.qkvg_s, s->a_s, s->fused, hidden, ph, s->qkvg, group))
    }
    if (s->attention) {
        // src/session/mod.rs:714-755: QK norm + RoPE out of the fused buffer, V transposed, fp16 attention
        if (!rope_in_gemm) {
            KREA2_STEP("qk norm + rope",
                       krea2_rope_qknorm_f16(stream, t, s->fused, w.qnorm, w.knorm, s->cos, s->sin, s->q, s->k, s->v, s->qkvg,
                                             q_heads, d.kv_heads, hidden, 1e-5f))
        }
        KREA2_STEP("V transpose", krea2_v_transpose(stream, t, s->v, s->v_transposed, kv_width, s->capacity))
        // shape::attention_source (src/kernels/shape.rs:24-31): the 32-query-row export from 8192 tokens on
        auto attention = krea2_shape_attention_rows(t) == 32 ? krea2_attention_gqa_lds_f16_wmma_q32
                                                             : krea2_attention_gqa_lds_f16_wmma;
        KREA2_STEP("f16 attention", attention(stream, t, d.kv_heads, s->q, s->k, s->v_transposed, s->attn_gu, hidden, kv_width,
                                              hidden, s->capacity, 0.08838834764831845f))
        KREA2_STEP("prepare gated", krea2_prepare_gated_i8(stream, t, s->attn_gu, s->fused + s->gate_offset * 2, s->a_q,
                                                           s->a_s, hidden, ph, s->qkvg))
    } else {
        // W8A8-only mode: the q columns of the fused buffer stand in for the attention output and
        // are read where they lie, through the row pitch of that buffer.
        KREA2_STEP("prepare gated", prepare_gated_pitched(stream, t, s->fused, s->qkvg, s->fused + s->gate_offset * 2, s->a_q,
                                                          s->a_s, hidden, ph, s->qkvg))
    }
    KREA2_STEP("gemm wo + residual", krea2_gemm_i8_resid_256(stream, t, s->a_q, w.wo_q, w.wo_s, s->a_s, s->x,
                                                             mods + 2 * hidden, hidden, ph, hidden, group))
    KREA2_STEP("prepare", krea2_prepare_norm_i8(stream, t, s->x, w.postnorm, mods + 3 * hidden, mods + 4 * hidden, s->a_q,
                                                s->a_s, hidden, ph, 1e-5f))
    if (s->fused_rotation) {
        // The same two stages with three of the prologue's four rotation stages moved into the GEMM's epilogue.
        KREA2_STEP("gemm gate|up + swiglu", krea2_gemm_i8_swiglu_rotated_256(stream, t, s->a_q, w.gu_q, w.gu_s, s->a_s,
                                                                             s->attn_gu, hidden, ph, 2 * inter, group))
        KREA2_STEP("prepare swiglu", krea2_prepare_rotated_i8(stream, t, s->attn_gu, s->a_q, s->a_s, inter, pi))
    } else {
        KREA2_STEP("gemm gate|up + swiglu", krea2_gemm_i8_swiglu_256(stream, t, s->a_q, w.gu_q, w.gu_s, s->a_s, s->attn_gu,
                                                                     hidden, ph, 2 * inter, group))
        KREA2_STEP("prepare swiglu", krea2_prepare_plain_i8(stream, t, s->attn_gu, s->a_q, s->a_s, inter, pi))
    }
    KREA2_STEP("gemm down + residual",
               krea2_gemm_i8_resid_256x256(stream, t, s->a_q, w.down_q, w.down_s, s->a_s, s->x, mods + 5 * hidden, inter, pi,
                                           hidden, group, static_cast<size_t>(krea2_shape_gemm_schedule_rows(t))))
#undef KREA2_STEP
    if ((status = mark(nullptr))) return status;
    return KREA2_OK;
}

int upload_rope(krea2_session *s, const float *host_cos, const float *host_sin) {
    const size_t count = s->tokens * s->dims.head_dim;
    const uint64_t print[2] = {fingerprint(host_cos, count), fingerprint(host_sin, count)};
    if (s->rope_valid && print[0] == s->rope_print[0] && print[1] == s->rope_print[1]) return KREA2_OK;
    s->rope_valid = false;  // a failed upload must not leave the tables claimed (src/session/mod.rs:430-431)
    KREA2_CUDA(cudaMemcpyAsync(s->cos, host_cos, count * 4, cudaMemcpyHostToDevice, s->stream));
    KREA2_CUDA(cudaMemcpyAsync(s->sin, host_sin, count * 4, cudaMemcpyHostToDevice, s->stream));
    s->rope_print[0] = print[0], s->rope_print[1] = print[1];
    s->rope_valid = true;
    return KREA2_OK;
}

int record_graph(krea2_session *s) {
    // Captured on a stream of its own: the session's stream may be the legacy default stream,
    // which cannot be captured.  Capturing executes nothing; the graph is launched on s->stream.
    cudaGraph_t graph = nullptr;
    cudaStream_t capture = nullptr;
    KREA2_CUDA(cudaStreamCreateWithFlags(&capture, cudaStreamNonBlocking));
    cudaError_t begin = cudaStreamBeginCapture(capture, cudaStreamCaptureModeThreadLocal);
    if (begin != cudaSuccess) {
        cudaStreamDestroy(capture);
        return fail(KREA2_RUNTIME, "cannot begin a stream capture: %s", cudaGetErrorString(begin));
    }
    int status = KREA2_OK;
    for (size_t i = 0; i < s->layers && status == KREA2_OK; i++) status = run_block(s, capture, i, nullptr);
    cudaError_t end = cudaStreamEndCapture(capture, &graph);
    cudaStreamDestroy(capture);
    if (status != KREA2_OK) {
        if (graph) cudaGraphDestroy(graph);
        return status;
    }
    if (end != cudaSuccess) return fail(KREA2_RUNTIME, "graph capture failed: %s", cudaGetErrorString(end));
    cudaError_t inst = cudaGraphInstantiate(&s->graph, graph, 0);
    cudaGraphDestroy(graph);
    if (inst != cudaSuccess) return fail(KREA2_RUNTIME, "graph instantiation failed: %s", cudaGetErrorString(inst));
    return KREA2_OK;
}

// Every block eagerly with an event between stages; the stage table adds up device time per
// label (src/session/mod.rs:627-647 reports the same sums from a profiled replay).
int run_profiled(krea2_session *s, size_t first, size_t count) {
    const size_t per = kMaxStagesPerBlock + 1;
    if (s->events.size() < count * per) {
        size_t old = s->events.size();
        s->events.resize(count * per);
        for (size_t i = old; i < s->events.size(); i++) KREA2_CUDA(cudaEventCreate(&s->events[i]));
    }
    std::vector<const char *> labels;
    for (size_t i = 0; i < count; i++) {
        labels.clear();
        if (int status = run_block(s, s->stream, first + i, s->events.data() + i * per, &labels)) return status;
    }
    KREA2_CUDA(cudaStreamSynchronize(s->stream));
    s->stages.clear();
    // KREA2_PROFILE_JSON=FILE (src/session/mod.rs:438-459): the raw device intervals of this forward, appended
    // as one JSON line.  Ticks are nanoseconds from the forward's first launch.
    const char *json_path = getenv("KREA2_PROFILE_JSON");
    std::string record;
    if (json_path && *json_path)
        record = "{\"tokens\":" + std::to_string(s->tokens) + ",\"layers\":" + std::to_string(count) +
                 ",\"profile\":{\"frequency_hz\":1000000000,\"gaps_ms\":0.0,\"intervals\":[";
    bool first_interval = true;
    for (size_t i = 0; i < count; i++)
        for (size_t k = 0; k < labels.size(); k++) {
            float ms = 0.0f;
            KREA2_CUDA(cudaEventElapsedTime(&ms, s->events[i * per + k], s->events[i * per + k + 1]));
            bool found = false;
            for (auto &stage : s->stages)
                if (std::string(stage.label) == labels[k]) stage.millis += ms, found = true;
            if (!found) s->stages.push_back(Stage{labels[k], ms});
            if (!record.empty()) {
                float begin_ms = 0.0f;
                KREA2_CUDA(cudaEventElapsedTime(&begin_ms, s->events[0], s->events[i * per + k]));
                const long long start_tick = static_cast<long long>(static_cast<double>(begin_ms) * 1e6 + 0.5);
                const long long end_tick = start_tick + static_cast<long long>(static_cast<double>(ms) * 1e6 + 0.5);
                record += std::string(first_interval ? "" : ",") + "{\"label\":\"" + labels[k] + "\",\"block\":" +
                          std::to_string(first + i) + ",\"start_tick\":" + std::to_string(start_tick) + ",\"end_tick\":" +
                          std::to_string(end_tick) + "}";
                first_interval = false;
            }
        }
    if (!record.empty()) {
        record += "]}}\n";
        FILE *file = fopen(json_path, "a");
        if (!file) return fail(KREA2_INVALID_ARGUMENT, "KREA2_PROFILE_JSON %s: %s", json_path, strerror(errno));
        const bool written = fwrite(record.data(), 1, record.size(), file) == record.size();
        if (fclose(file) != 0 || !written)
            return fail(KREA2_INVALID_ARGUMENT, "KREA2_PROFILE_JSON %s: write failed", json_path);
    }
    return KREA2_OK;
}

int check_session(krea2_session *s, krea2_stream stream) {
    KREA2_REQUIRE(s, "session is null");
    if (s->poisoned) return fail(KREA2_POISONED, "the session failed earlier and cannot be used again");
    KREA2_REQUIRE(static_cast<cudaStream_t>(stream) == s->stream, "a session must use the stream that created it");
    return KREA2_OK;
}

int poison(krea2_session *s, int status) {
    if (status == KREA2_RUNTIME || status == KREA2_INTERNAL) s->poisoned = true;
    return status;
}

}  // namespace

// ---------------------------------------------------------------- weights
extern "C" int krea2_session_validate_dimensions(size_t tokens, size_t layers) {
    clear_error();
    KREA2_REQUIRE(tokens >= krea2_shape_tokens_min() && tokens <= krea2_shape_tokens_max() && layers >= 1 && layers <= 28,
                  "tokens must be %zu..%zu and layers must be 1..28", krea2_shape_tokens_min(), krea2_shape_tokens_max());
    return KREA2_OK;
}

extern "C" int krea2_weights_plan_bytes(const krea2_dims *dims, size_t layers, size_t *bytes) {
    clear_error();
    if (int status = check_dims(dims)) return status;
    KREA2_REQUIRE(layers >= 1 && layers <= 28 && bytes, "layers must be 1..28");
    krea2_weights w;
    w.dims = *dims, w.layers = layers;
    plan(w);
    *bytes = w.total_bytes;
    return KREA2_OK;
}

extern "C" int krea2_weights_create(const krea2_dims *dims, size_t layers, krea2_weights **out) {
    clear_error();
    if (int status = check_dims(dims)) return status;
    KREA2_REQUIRE(layers >= 1 && layers <= 28 && out, "layers must be 1..28");
    std::unique_ptr<krea2_weights> w(new krea2_weights);
    w->dims = *dims, w->layers = layers;
    plan(*w);
    KREA2_CUDA(cudaGetDevice(&w->device));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&w->base), w->total_bytes));
    *out = w.release();
    return KREA2_OK;
}

extern "C" int krea2_weights_locate(const krea2_weights *weights, const char *name, void **ptr, size_t *bytes) {
    clear_error();
    KREA2_REQUIRE(weights && name && ptr && bytes, "weights_locate: null argument");
    auto it = weights->spans.find(name);
    if (it == weights->spans.end()) return fail(KREA2_INVALID_ARGUMENT, "no span named %s", name);
    *ptr = weights->base + it->second.offset;
    *bytes = it->second.bytes;
    return KREA2_OK;
}

extern "C" int krea2_weights_fill_synthetic(krea2_weights *weights, uint64_t seed, krea2_stream stream) {
    clear_error();
    KREA2_REQUIRE(weights, "weights is null");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (const auto &entry : weights->spans) {
        const Span &span = entry.second;
        uint8_t *dst = weights->base + span.offset;
        const uint64_t span_seed = seed * 0x100000001b3ull + span.offset;
        if (span.kind == 'q') {
            fill_rows_kernel<<<1184, 256, 0, st>>>(reinterpret_cast<int8_t *>(dst), span.rows, span.row_bytes, span.pitch,
                                                   span_seed);
        } else {
            const size_t n = span.bytes / 4;
            fill_vector_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, st>>>(reinterpret_cast<float *>(dst), n,
                                                                                      span_seed, span.kind == 'n');
        }
    }
    KREA2_CUDA(cudaGetLastError());
    return KREA2_OK;
}

extern "C" int krea2_weights_upload(krea2_weights *weights, const char *name, const void *host_bytes, size_t bytes,
                                    krea2_stream stream) {
    clear_error();
    KREA2_REQUIRE(weights && name && host_bytes, "weights_upload: null argument");
    auto it = weights->spans.find(name);
    if (it == weights->spans.end()) return fail(KREA2_INVALID_ARGUMENT, "no span named %s", name);
    KREA2_REQUIRE(bytes == it->second.bytes, "%s spans %zu bytes, got %zu", name, it->second.bytes, bytes);
    KREA2_CUDA(cudaMemcpyAsync(weights->base + it->second.offset, host_bytes, bytes, cudaMemcpyHostToDevice,
                               static_cast<cudaStream_t>(stream)));
    return KREA2_OK;
}

extern "C" int krea2_weights_download(const krea2_weights *weights, const char *name, void *host_bytes, size_t bytes,
                                      krea2_stream stream) {
    clear_error();
    KREA2_REQUIRE(weights && name && host_bytes, "weights_download: null argument");
    auto it = weights->spans.find(name);
    if (it == weights->spans.end()) return fail(KREA2_INVALID_ARGUMENT, "no span named %s", name);
    KREA2_REQUIRE(bytes == it->second.bytes, "%s spans %zu bytes, got %zu", name, it->second.bytes, bytes);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    KREA2_CUDA(cudaMemcpyAsync(host_bytes, weights->base + it->second.offset, bytes, cudaMemcpyDeviceToHost, st));
    KREA2_CUDA(cudaStreamSynchronize(st));
    return KREA2_OK;
}

extern "C" void krea2_weights_retain(krea2_weights *weights) {
    if (weights) weights->references.fetch_add(1);
}
extern "C" void krea2_weights_release(krea2_weights *weights) {
    if (weights && weights->references.fetch_sub(1) == 1) {
        if (weights->base) cudaFree(weights->base);
        delete weights;
    }
}

// ---------------------------------------------------------------- session
extern "C" int krea2_session_create(krea2_stream stream, krea2_weights *weights, size_t tokens, size_t layers,
                                    krea2_session **out) {
    clear_error();
    if (int status = krea2_session_validate_dimensions(tokens, layers)) return status;
    KREA2_REQUIRE(weights && out, "session_create: null argument");
    KREA2_REQUIRE(layers <= weights->layers, "the weights hold %zu blocks, %zu were asked for", weights->layers, layers);
    int current_device = 0;
    KREA2_CUDA(cudaGetDevice(&current_device));
    KREA2_REQUIRE(current_device == weights->device, "the weights live on device %d but device %d is current",
                  weights->device, current_device);
    if (int status = prepare_gemm_device()) return status;
    if (int status = prepare_attention_device()) return status;
    if (int status = prepare_prologue_device(static_cast<cudaStream_t>(stream))) return status;
    std::unique_ptr<krea2_session> s(new krea2_session);
    s->stream = static_cast<cudaStream_t>(stream);
    s->tokens = tokens, s->layers = layers, s->capacity = krea2_shape_capacity(tokens);
    s->dims = weights->dims, s->qkvg = weights->qkvg;
    s->gate_offset = s->dims.hidden + 2 * s->dims.kv_heads * s->dims.head_dim;  // src/session/mod.rs:45
    const size_t cap = s->capacity, hidden = s->dims.hidden, inter = s->dims.inter;
    s->x_bytes = cap * hidden * 2;
    s->a_q_bytes = cap * pitch_of(inter > hidden ? inter : hidden);  // the widest prepared operand (:323-325)
    s->fused_bytes = cap * s->qkvg * 2;
    s->attn_gu_bytes = cap * (inter > hidden ? inter : hidden) * 2;
    s->mods_bytes = layers * 6 * hidden * 4;
    s->rope_bytes = cap * s->dims.head_dim * 4;
    s->q_bytes = cap * hidden * 2;
    s->kv_bytes = cap * s->dims.kv_heads * s->dims.head_dim * 2;
    // The attention kernel is built for 128 channels per head; other shapes keep the W8A8 chain only.
    s->attention = s->dims.head_dim == 128 && hidden % 128 == 0 && (hidden / 128) % s->dims.kv_heads == 0;
    auto destroy = [](krea2_session *p) { krea2_session_destroy(p); };
    std::unique_ptr<krea2_session, decltype(destroy)> guard(s.release(), destroy);
    krea2_session *p = guard.get();
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->x), p->x_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->a_q), p->a_q_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->a_s), cap * 4));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->fused), p->fused_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->attn_gu), p->attn_gu_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->mods), p->mods_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->cos), p->rope_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->sin), p->rope_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->q), p->q_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->k), p->kv_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->v), p->kv_bytes));
    KREA2_CUDA(cudaMalloc(reinterpret_cast<void **>(&p->v_transposed), p->kv_bytes));
    KREA2_CUDA(cudaMemsetAsync(p->q, 0, p->q_bytes, p->stream));
    KREA2_CUDA(cudaMemsetAsync(p->k, 0, p->kv_bytes, p->stream));
    KREA2_CUDA(cudaMemsetAsync(p->v, 0, p->kv_bytes, p->stream));
    KREA2_CUDA(cudaMemsetAsync(p->v_transposed, 0, p->kv_bytes, p->stream));  // the headroom columns stay zero
    KREA2_CUDA(cudaMemsetAsync(p->cos, 0, p->rope_bytes, p->stream));
    KREA2_CUDA(cudaMemsetAsync(p->sin, 0, p->rope_bytes, p->stream));
    // Headroom rows are read and must be zero (src/session/mod.rs:336-340).
    KREA2_CUDA(cudaMemsetAsync(p->x, 0, p->x_bytes, p->stream));
    KREA2_CUDA(cudaMemsetAsync(p->fused, 0, p->fused_bytes, p->stream));
    KREA2_CUDA(cudaMemsetAsync(p->a_q, 0, p->a_q_bytes, p->stream));
    KREA2_CUDA(cudaMemsetAsync(p->attn_gu, 0, p->attn_gu_bytes, p->stream));
    krea2_weights_retain(weights);
    p->weights = weights;
    const char *env = getenv("KREA2_NATIVE_PROFILE");  // src/kernels/mod.rs:43-45
    p->profile = env && std::string(env) == "1";
    const char *fused = getenv("KREA2_FUSED_ROTATION");
    p->fused_rotation = fused ? std::string(fused) == "1" : kFusedRotationDefault;
    const char *rope = getenv("KREA2_FUSED_ROPE");
    p->fused_rope = (rope ? std::string(rope) == "1" : kFusedRopeDefault) && p->qkvg % 256 == 0;
    const char *dependent = getenv("KREA2_DEPENDENT_LAUNCH");
    p->dependent_launch = dependent ? std::string(dependent) == "1" : kDependentLaunchDefault;
    *out = guard.release();
    return KREA2_OK;
}

extern "C" void krea2_session_destroy(krea2_session *s) {
    if (!s) return;
    if (s->graph) cudaGraphExecDestroy(s->graph);
    for (cudaEvent_t e : s->events) cudaEventDestroy(e);
    void *buffers[] = {s->x, s->a_q, s->a_s, s->fused, s->attn_gu, s->mods, s->cos, s->sin, s->q, s->k, s->v, s->v_transposed};
    for (void *b : buffers)
        if (b) cudaFree(b);
    krea2_weights_release(s->weights);
    delete s;
}

extern "C" size_t krea2_session_tokens(const krea2_session *s) { return s ? s->tokens : 0; }
extern "C" size_t krea2_session_layers(const krea2_session *s) { return s ? s->layers : 0; }
extern "C" int krea2_session_set_profile(krea2_session *s, int enable) {
    if (!s) return 0;
    int previous = s->profile ? 1 : 0;
    s->profile = enable != 0;
    return previous;
}
extern "C" size_t krea2_session_stage_profile(const krea2_session *s, const char **labels, double *millis,
                                              size_t capacity) {
    if (!s) return 0;
    size_t n = s->stages.size() < capacity ? s->stages.size() : capacity;
    for (size_t i = 0; i < n; i++) {
        if (labels) labels[i] = s->stages[i].label;
        if (millis) millis[i] = s->stages[i].millis;
    }
    return n;
}
extern "C" size_t krea2_session_launches_per_forward(const krea2_session *s) {
    // eleven kernels per block with attention (ten when the q|k|v|gate GEMM also rotates); eight without
    return s ? s->layers * (s->attention ? (s->fused_rope ? 10 : 11) : 8) : 0;
}

extern "C" int krea2_session_set_fused_rotation(krea2_session *s, int enable) {
    if (!s) return 0;
    const int previous = s->fused_rotation ? 1 : 0;
    if ((enable != 0) != s->fused_rotation) {
        s->fused_rotation = enable != 0;
        if (s->graph) {  // the recording holds the other launch list
            cudaGraphExecDestroy(s->graph);
            s->graph = nullptr;
        }
    }
    return previous;
}

extern "C" int krea2_session_set_fused_rope(krea2_session *s, int enable) {
    if (!s) return 0;
    const int previous = s->fused_rope ? 1 : 0;
    const bool next = enable != 0 && s->qkvg % 256 == 0;
    if (next != s->fused_rope) {
        s->fused_rope = next;
        if (s->graph) {  // the recording holds the other launch list
            cudaGraphExecDestroy(s->graph);
            s->graph = nullptr;
        }
    }
    return previous;
}

extern "C" int krea2_session_set_attention(krea2_session *s, int enable) {
    if (!s) return 0;
    const int previous = s->attention ? 1 : 0;
    const bool possible = s->dims.head_dim == 128 && s->dims.hidden % 128 == 0 && (s->dims.hidden / 128) % s->dims.kv_heads == 0;
    const bool next = enable != 0 && possible;
    if (next != s->attention) {
        s->attention = next;
        if (s->graph) {  // the recording holds the other launch list
            cudaGraphExecDestroy(s->graph);
            s->graph = nullptr;
        }
    }
    return previous;
}

extern "C" int krea2_session_run(krea2_session *s, krea2_stream stream, uint16_t *host_x, const float *host_mods,
                                 const float *host_cos, const float *host_sin, size_t first_block,
                                 size_t block_count) {
    clear_error();
    if (int status = check_session(s, stream)) return status;
    KREA2_REQUIRE(host_x && host_mods && host_cos && host_sin, "session_run: null host buffer");
    const size_t count = block_count ? block_count : (s->layers > first_block ? s->layers - first_block : 0);
    KREA2_REQUIRE(first_block < s->layers && count >= 1 && count <= s->layers - first_block,
                  "block range must be within the loaded layers");
    const size_t rows = s->tokens * s->dims.hidden * 2;
    auto body = [&]() -> int {
        KREA2_CUDA(cudaMemcpyAsync(s->x, host_x, rows, cudaMemcpyHostToDevice, s->stream));
        KREA2_CUDA(cudaMemcpyAsync(s->mods, host_mods, s->mods_bytes, cudaMemcpyHostToDevice, s->stream));
        if (int status = upload_rope(s, host_cos, host_sin)) return status;
        if (s->profile) {
            if (int status = run_profiled(s, first_block, count)) return status;
        } else if (first_block == 0 && count == s->layers) {
            // The whole chain: the recorded graph, as run_device replays it (same launches, fewer gaps).
            if (!s->graph)
                if (int status = record_graph(s)) return status;
            KREA2_CUDA(cudaGraphLaunch(s->graph, s->stream));
        } else {
            for (size_t i = first_block; i < first_block + count; i++)
                if (int status = run_block(s, s->stream, i, nullptr)) return status;
        }
        KREA2_CUDA(cudaMemcpyAsync(host_x, s->x, rows, cudaMemcpyDeviceToHost, s->stream));
        KREA2_CUDA(cudaStreamSynchronize(s->stream));
        return KREA2_OK;
    };
    return poison(s, body());
}

extern "C" int krea2_session_run_device(krea2_session *s, krea2_stream stream, void *x, size_t x_bytes,
                                        const void *mods, size_t mods_bytes, const float *host_cos,
                                        const float *host_sin) {
    clear_error();
    if (int status = check_session(s, stream)) return status;
    KREA2_REQUIRE(x && mods && host_cos && host_sin, "session_run_device: null buffer");
    const size_t rows = s->tokens * s->dims.hidden * 2;
    KREA2_REQUIRE(x_bytes >= rows, "x spans %zu bytes, expected at least %zu", x_bytes, rows);
    KREA2_REQUIRE(mods_bytes >= s->mods_bytes, "mods spans %zu bytes, expected at least %zu", mods_bytes, s->mods_bytes);
    auto body = [&]() -> int {
        // Inputs go into the session's own buffers: a recorded graph fixes its addresses
        // (src/session/mod.rs:560-580).
        KREA2_CUDA(cudaMemcpyAsync(s->x, x, rows, cudaMemcpyDeviceToDevice, s->stream));
        KREA2_CUDA(cudaMemcpyAsync(s->mods, mods, s->mods_bytes, cudaMemcpyDeviceToDevice, s->stream));
        if (int status = upload_rope(s, host_cos, host_sin)) return status;
        if (s->profile) {
            if (int status = run_profiled(s, 0, s->layers)) return status;
        } else {
            if (!s->graph)
                if (int status = record_graph(s)) return status;
            KREA2_CUDA(cudaGraphLaunch(s->graph, s->stream));
        }
        KREA2_CUDA(cudaMemcpyAsync(x, s->x, rows, cudaMemcpyDeviceToDevice, s->stream));
        return KREA2_OK;
    };
    return poison(s, body());
}

extern "C" int krea2_session_buffer(const krea2_session *s, const char *name, void **ptr, size_t *bytes) {
    clear_error();
    KREA2_REQUIRE(s && name && ptr && bytes, "session_buffer: null argument");
    const std::string n(name);
    if (n == "x") *ptr = s->x, *bytes = s->x_bytes;
    else if (n == "a_q") *ptr = s->a_q, *bytes = s->a_q_bytes;
    else if (n == "a_s") *ptr = s->a_s, *bytes = s->capacity * 4;
    else if (n == "fused") *ptr = s->fused, *bytes = s->fused_bytes;
    else if (n == "attn_gu") *ptr = s->attn_gu, *bytes = s->attn_gu_bytes;
    else if (n == "mods") *ptr = s->mods, *bytes = s->mods_bytes;
    else if (n == "q") *ptr = s->q, *bytes = s->q_bytes;
    else if (n == "k") *ptr = s->k, *bytes = s->kv_bytes;
    else if (n == "v") *ptr = s->v, *bytes = s->kv_bytes;
    else if (n == "v_transposed") *ptr = s->v_transposed, *bytes = s->kv_bytes;
    else return fail(KREA2_INVALID_ARGUMENT, "no session buffer named %s", name);
    return KREA2_OK;
}
