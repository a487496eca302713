// The parts of the C ABI that launch nothing themselves: the error channel, the
// launch-shape rules of src/kernels/shape.rs, and the name-keyed dispatcher that mirrors
// Ops::launch (src/ops/mod.rs:673-693).
#include <cstring>
#include <string>

#include "common.cuh"

namespace krea2 {

namespace {
thread_local char g_last_error[512] = "";
}

int fail(krea2_status status, const char *format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(g_last_error, sizeof g_last_error, format, args);
    va_end(args);
    return status;
}

void clear_error() { g_last_error[0] = '\0'; }

bool &dependent_launches() {
    static thread_local bool flag = false;
    return flag;
}

}  // namespace krea2

using namespace krea2;

extern "C" const char *krea2_last_error(void) { return g_last_error; }
extern "C" const char *krea2_version(void) { return "krea2_b200 0.1 (sm_100a)"; }

// ---------------------------------------------------------------- src/kernels/shape.rs
extern "C" size_t krea2_shape_tokens_min(void) { return 16; }      // shape.rs:8
extern "C" size_t krea2_shape_tokens_max(void) { return 16896; }   // shape.rs:8

extern "C" size_t krea2_shape_capacity(size_t tokens) {  // shape.rs:12-16
    size_t tiles = (tokens + 16 + 31) / 32 * 32;
    size_t blocks = (tokens + 63) / 64 * 64;
    return tiles > blocks ? tiles : blocks;
}
extern "C" size_t krea2_shape_attention_rows(size_t tokens) { return tokens >= 8192 ? 32 : 16; }  // :20-22
extern "C" size_t krea2_shape_gemm_pitch(size_t k) { return k % 8192 == 0 ? k + 64 : k; }         // :105-107
extern "C" size_t krea2_shape_gemm_grid_rows(size_t tokens) { return (tokens + 255) / 256; }      // :110-112
extern "C" size_t krea2_shape_gemm_m_group(void) { return 4; }                                    // :93
extern "C" int krea2_shape_gemm_schedule_rows(size_t tokens) { return tokens >= 4096 ? 1 : 0; }   // :97-99

namespace {
bool wide_stem(const char *stem) { return stem && std::strcmp(stem, "gemm_down") == 0; }  // shape.rs:67-72
}
extern "C" size_t krea2_shape_gemm_tile_columns(const char *stem) { return wide_stem(stem) ? 256 : 128; }
extern "C" uint32_t krea2_shape_gemm_tile_threads(const char *stem) { return wide_stem(stem) ? 512 : 256; }
extern "C" const char *krea2_shape_gemm_source(const char *family, const char *stem) {  // shape.rs:84-89
    if (family && std::strcmp(family, "gemm_i8_resid_256") == 0 && wide_stem(stem)) return "gemm_i8_resid_256x256";
    return family;
}

// ---------------------------------------------------------------- Ops::launch
namespace {

struct Config {
    const krea2_config_entry *entries;
    size_t count;
    // Looks `key` up; both the bare spelling ("k_size") and the kernel-qualified one
    // ("krea2.gemm_i8_256.k_size") are accepted.
    const krea2_config_entry *find(const char *key) const {
        for (size_t i = 0; i < count; i++) {
            const char *name = entries[i].key;
            if (!name) continue;
            const char *dot = std::strrchr(name, '.');
            if (std::strcmp(dot ? dot + 1 : name, key) == 0) return entries + i;
        }
        return nullptr;
    }
};

int need(const Config &config, const char *kernel, const char *key, uint64_t *value) {
    const krea2_config_entry *e = config.find(key);
    if (!e) return fail(KREA2_INVALID_ARGUMENT, "%s: config key '%s' is missing", kernel, key);
    *value = e->value;
    return KREA2_OK;
}

int check_bindings(const char *kernel, const krea2_binding *bindings, size_t count, size_t expected,
                   const size_t *min_bytes) {
    if (count != expected)
        return fail(KREA2_INVALID_ARGUMENT, "%s takes %zu buffers, got %zu", kernel, expected, count);
    for (size_t i = 0; i < count; i++) {
        if (!bindings[i].ptr) return fail(KREA2_INVALID_ARGUMENT, "%s: buffer %zu is null", kernel, i);
        if (bindings[i].bytes < min_bytes[i])
            return fail(KREA2_INVALID_ARGUMENT, "%s: buffer %zu spans %zu bytes, the launch touches %zu", kernel, i,
                        bindings[i].bytes, min_bytes[i]);
    }
    return KREA2_OK;
}

// The reference's grid and workgroup rules (src/kernels/mod.rs:77-98): counts must fit a
// u32, and the block size must be the one the kernel is built for.
int check_geometry(const char *kernel, size_t grid_x, size_t grid_y, uint32_t threads, size_t want_x, size_t want_y,
                   uint32_t want_threads) {
    if (grid_x > 0xffffffffull || grid_y > 0xffffffffull)
        return fail(KREA2_INTERNAL, "%s: %zu workgroups exceed the grid", kernel, grid_x > grid_y ? grid_x : grid_y);
    if (threads != want_threads)
        return fail(KREA2_INTERNAL, "%s: compiled for workgroup [%u, 1, 1] but the host asked for %u", kernel,
                    want_threads, threads);
    if (grid_x != want_x || grid_y != want_y)
        return fail(KREA2_INVALID_ARGUMENT, "%s: grid %zu x %zu does not cover the launch (%zu x %zu expected)",
                    kernel, grid_x, grid_y, want_x, want_y);
    return KREA2_OK;
}

}  // namespace

extern "C" int krea2_launch(krea2_stream stream, const char *name, const krea2_config_entry *config_entries,
                            size_t config_count, const uint64_t *indices, size_t index_count,
                            const krea2_binding *bindings, size_t binding_count, size_t grid_x, size_t grid_y,
                            uint32_t threads) {
    clear_error();
    KREA2_REQUIRE(name, "launch: kernel name is null");
    KREA2_REQUIRE(config_entries || config_count == 0, "launch: config is null");
    KREA2_REQUIRE(bindings || binding_count == 0, "launch: bindings are null");
    KREA2_REQUIRE(index_count <= 4, "a kernel takes at most four indices");  // src/kernels/mod.rs:119
    KREA2_REQUIRE(indices && index_count == 1, "%s takes one index scalar (its row count)", name);
    const Config config{config_entries, config_count};
    const size_t rows = static_cast<size_t>(indices[0]);
    KREA2_REQUIRE(rows >= 1, "%s: the row count must be at least 1", name);
    const krea2_binding *b = bindings;

    const bool norm = std::strcmp(name, "prepare_norm_i8") == 0;
    const bool gated = std::strcmp(name, "prepare_gated_i8") == 0;
    const bool plain = std::strcmp(name, "prepare_plain_i8") == 0;
    if (norm || gated || plain) {
        uint64_t width = 0, out_stride = 0, gate_stride = 0;
        if (int s = need(config, name, "width", &width)) return s;
        if (int s = need(config, name, "out_stride", &out_stride)) return s;
        if (int s = check_geometry(name, grid_x, grid_y, threads, rows, 1, 256)) return s;
        if (norm) {
            const krea2_config_entry *eps = config.find("eps");
            if (!eps) return fail(KREA2_INVALID_ARGUMENT, "%s: config key 'eps' is missing", name);
            const size_t min_bytes[6] = {rows * width * 2, width * 4, width * 4, width * 4,
                                         (rows - 1) * out_stride + width, rows * 4};
            if (int s = check_bindings(name, b, binding_count, 6, min_bytes)) return s;
            return krea2_prepare_norm_i8(stream, rows, b[0].ptr, static_cast<const float *>(b[1].ptr),
                                         static_cast<const float *>(b[2].ptr), static_cast<const float *>(b[3].ptr),
                                         b[4].ptr, static_cast<float *>(b[5].ptr), width, out_stride, eps->fvalue);
        }
        if (gated) {
            if (int s = need(config, name, "gate_stride", &gate_stride)) return s;
            const size_t min_bytes[4] = {rows * width * 2, ((rows - 1) * gate_stride + width) * 2,
                                         (rows - 1) * out_stride + width, rows * 4};
            if (int s = check_bindings(name, b, binding_count, 4, min_bytes)) return s;
            return krea2_prepare_gated_i8(stream, rows, b[0].ptr, b[1].ptr, b[2].ptr, static_cast<float *>(b[3].ptr),
                                          width, out_stride, gate_stride);
        }
        const size_t min_bytes[3] = {rows * width * 2, (rows - 1) * out_stride + width, rows * 4};
        if (int s = check_bindings(name, b, binding_count, 3, min_bytes)) return s;
        return krea2_prepare_plain_i8(stream, rows, b[0].ptr, b[1].ptr, static_cast<float *>(b[2].ptr), width,
                                      out_stride);
    }

    const bool g_plain = std::strcmp(name, "gemm_i8_256") == 0;
    const bool g_resid = std::strcmp(name, "gemm_i8_resid_256") == 0;
    const bool g_wide = std::strcmp(name, "gemm_i8_resid_256x256") == 0;
    const bool g_swiglu = std::strcmp(name, "gemm_i8_swiglu_256") == 0;
    if (g_plain || g_resid || g_wide || g_swiglu) {
        uint64_t k = 0, stride = 0, n = 0, group = 0, schedule = 0;
        if (int s = need(config, name, "k_size", &k)) return s;
        if (int s = need(config, name, "k_stride", &stride)) return s;
        if (int s = need(config, name, "n_size", &n)) return s;
        if (int s = need(config, name, "m_group", &group)) return s;
        if (g_wide)
            if (int s = need(config, name, "schedule_rows", &schedule)) return s;
        const size_t columns = g_wide ? 256 : 128;
        if (int s = check_geometry(name, grid_x, grid_y, threads, n / columns, (rows + 255) / 256, g_wide ? 512 : 256))
            return s;
        const size_t out_bytes = g_swiglu ? rows * (n / 2) * 2 : rows * n * 2;
        const size_t min_bytes[6] = {(rows - 1) * stride + k, (n - 1) * stride + k, n * 4, rows * 4, out_bytes, n * 4};
        const size_t expected = (g_resid || g_wide) ? 6 : 5;
        if (int s = check_bindings(name, b, binding_count, expected, min_bytes)) return s;
        const float *scale = static_cast<const float *>(b[2].ptr);
        const float *a_scale = static_cast<const float *>(b[3].ptr);
        if (g_plain) return krea2_gemm_i8_256(stream, rows, b[0].ptr, b[1].ptr, scale, a_scale, b[4].ptr, k, stride, n, group);
        if (g_swiglu)
            return krea2_gemm_i8_swiglu_256(stream, rows, b[0].ptr, b[1].ptr, scale, a_scale, b[4].ptr, k, stride, n, group);
        const float *gate = static_cast<const float *>(b[5].ptr);
        if (g_resid)
            return krea2_gemm_i8_resid_256(stream, rows, b[0].ptr, b[1].ptr, scale, a_scale, b[4].ptr, gate, k, stride, n,
                                           group);
        return krea2_gemm_i8_resid_256x256(stream, rows, b[0].ptr, b[1].ptr, scale, a_scale, b[4].ptr, gate, k, stride, n,
                                           group, schedule);
    }

    if (std::strcmp(name, "lora_transport") == 0) {
        uint64_t reverse = 0;
        if (int s = need(config, name, "reverse", &reverse)) return s;
        if (int s = check_geometry(name, grid_x, grid_y, threads, (rows + 255) / 256, 1, 256)) return s;
        const size_t min_bytes[2] = {rows * 2, rows * 2};
        if (int s = check_bindings(name, b, binding_count, 2, min_bytes)) return s;
        return krea2_lora_transport(stream, rows, b[0].ptr, b[1].ptr, static_cast<int>(reverse));
    }
    // The pointwise kernels of the sampler loop, launched by Ops::launch_1d over `rows` elements.  Their
    // float scalar (Scalars::float, src/kernels/mod.rs:125-134) travels as the `fvalue` of a config entry.
    const bool euler = std::strcmp(name, "euler") == 0, guide = std::strcmp(name, "guidance") == 0;
    if (euler || guide) {
        const char *key = euler ? "delta" : "scale";
        const krea2_config_entry *scalar = config.find(key);
        if (!scalar) return fail(KREA2_INVALID_ARGUMENT, "%s: float scalar '%s' is missing", name, key);
        if (int s = check_geometry(name, grid_x, grid_y, threads, (rows + 255) / 256, 1, 256)) return s;
        const size_t min_bytes[2] = {rows * 2, rows * 2};
        if (int s = check_bindings(name, b, binding_count, 2, min_bytes)) return s;
        return euler ? krea2_euler(stream, rows, scalar->fvalue, b[0].ptr, b[1].ptr)
                     : krea2_guidance(stream, rows, scalar->fvalue, b[0].ptr, b[1].ptr);
    }
    if (std::strcmp(name, "modulation") == 0) {
        uint64_t xsize = 0;
        if (int s = need(config, name, "xsize", &xsize)) return s;
        if (int s = check_geometry(name, grid_x, grid_y, threads, (rows + 255) / 256, 1, 256)) return s;
        const size_t min_bytes[3] = {static_cast<size_t>(xsize) * 2, rows * 2, rows * 4};
        if (int s = check_bindings(name, b, binding_count, 3, min_bytes)) return s;
        return krea2_modulation(stream, rows, b[0].ptr, b[1].ptr, static_cast<float *>(b[2].ptr), xsize);
    }
    return fail(KREA2_INVALID_ARGUMENT, "no kernel named %s", name);
}
