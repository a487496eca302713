// The pointwise kernels around the block chain and the sigma schedule of the sampler loop:
//   krea2_modulation  (kernels/native/modulation.loom; launched at src/models/graph.rs:405-425)
//   krea2_euler       (kernels/native/euler.loom;      src/ops/mod.rs:373-390)
//   krea2_guidance    (kernels/native/guidance.loom;   src/ops/mod.rs:392-410)
//   krea2_schedule_*  (src/pipeline/schedule.rs)
// The kernels are HBM streams: eight elements per thread through 128-bit accesses where the
// pointers and the count allow, one element per thread otherwise.  Every bf16 rounding point of
// the reference is kept, each f32 step is one round-to-nearest operation.
#include <cmath>

#include "common.cuh"

namespace krea2 {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float bf16_value(uint16_t bits) { return __uint_as_float(static_cast<uint32_t>(bits) << 16); }
__device__ __forceinline__ uint16_t bf16_bits(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }

// y = bf16(x + t), widened (kernels/native/modulation.loom:33-42).
__device__ __forceinline__ float modulation_value(uint16_t x, uint16_t t) {
    return bf_round(__fadd_rn(bf16_value(x), bf16_value(t)));
}
// sample = bf16(sample + bf16(dt * velocity)), dt = bf16(delta) (kernels/native/euler.loom:29-40).
__device__ __forceinline__ uint16_t euler_value(uint16_t sample, uint16_t velocity, float dt) {
    return bf16_bits(__fadd_rn(bf16_value(sample), bf_round(__fmul_rn(dt, bf16_value(velocity)))));
}
// cond = bf16(cond + bf16(scale * bf16(cond - uncond))) (kernels/native/guidance.loom:29-42).
__device__ __forceinline__ uint16_t guidance_value(uint16_t cond, uint16_t uncond, float scale) {
    const float c = bf16_value(cond);
    const float difference = bf_round(__fsub_rn(c, bf16_value(uncond)));
    return bf16_bits(__fadd_rn(c, bf_round(__fmul_rn(scale, difference))));
}

__device__ __forceinline__ uint32_t pair(uint16_t lo, uint16_t hi) { return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16); }

template <bool kVector>
__global__ void __launch_bounds__(kThreads)
modulation_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ tables, float *__restrict__ y,
                  size_t count, size_t xsize) {
    const size_t i = (static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x) * (kVector ? 8 : 1);
    if (i >= count) return;
    if constexpr (kVector) {
        // count and xsize are multiples of 8 here, so the eight elements share one period of x.
        const uint4 t = *reinterpret_cast<const uint4 *>(tables + i);
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(x + i % xsize));
        const uint32_t tw[4] = {t.x, t.y, t.z, t.w}, vw[4] = {v.x, v.y, v.z, v.w};
        float out[8];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            out[2 * k] = modulation_value(static_cast<uint16_t>(vw[k]), static_cast<uint16_t>(tw[k]));
            out[2 * k + 1] = modulation_value(static_cast<uint16_t>(vw[k] >> 16), static_cast<uint16_t>(tw[k] >> 16));
        }
        *reinterpret_cast<float4 *>(y + i) = make_float4(out[0], out[1], out[2], out[3]);
        *reinterpret_cast<float4 *>(y + i + 4) = make_float4(out[4], out[5], out[6], out[7]);
    } else {
        y[i] = modulation_value(x[i % xsize], tables[i]);
    }
}

// In-place update of `target` from `other`; Euler when kEuler, guidance otherwise.
template <bool kEuler, bool kVector>
__global__ void __launch_bounds__(kThreads)
update_kernel(uint16_t *__restrict__ target, const uint16_t *__restrict__ other, size_t count, float scalar) {
    const float s = kEuler ? bf_round(scalar) : scalar;
    const size_t i = (static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x) * (kVector ? 8 : 1);
    if (i >= count) return;
    if constexpr (kVector) {
        if (i + 8 <= count) {
            const uint4 a = *reinterpret_cast<const uint4 *>(target + i);
            const uint4 b = *reinterpret_cast<const uint4 *>(other + i);
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
            uint32_t out[4];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const uint16_t a0 = static_cast<uint16_t>(aw[k]), a1 = static_cast<uint16_t>(aw[k] >> 16);
                const uint16_t b0 = static_cast<uint16_t>(bw[k]), b1 = static_cast<uint16_t>(bw[k] >> 16);
                out[k] = kEuler ? pair(euler_value(a0, b0, s), euler_value(a1, b1, s))
                                : pair(guidance_value(a0, b0, s), guidance_value(a1, b1, s));
            }
            *reinterpret_cast<uint4 *>(target + i) = make_uint4(out[0], out[1], out[2], out[3]);
        } else {
            for (size_t j = i; j < count; j++)
                target[j] = kEuler ? euler_value(target[j], other[j], s) : guidance_value(target[j], other[j], s);
        }
    } else {
        target[i] = kEuler ? euler_value(target[i], other[i], s) : guidance_value(target[i], other[i], s);
    }
}

int finish(const char *what) {
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return fail(KREA2_RUNTIME, "%s launch failed: %s", what, cudaGetErrorString(status));
    return KREA2_OK;
}

unsigned blocks_for(size_t count, int per_thread) {
    const size_t threads = (count + per_thread - 1) / per_thread;
    return static_cast<unsigned>((threads + kThreads - 1) / kThreads);
}

// The `count` range of the three kernels (kernels/native/euler.loom:17, modulation.loom:21).
int check_count(const char *name, size_t count) {
    KREA2_REQUIRE(count >= 1 && count <= 1073741824, "%s: element count %zu outside 1..2^30", name, count);
    return KREA2_OK;
}

template <bool kEuler>
int run_update(const char *name, cudaStream_t stream, size_t count, float scalar, void *target, const void *other) {
    if (int status = check_count(name, count)) return status;
    KREA2_REQUIRE(target && other, "%s: null buffer", name);
    KREA2_REQUIRE(reinterpret_cast<uintptr_t>(target) % 2 == 0 && reinterpret_cast<uintptr_t>(other) % 2 == 0,
                  "%s: bf16 buffers must be 2-byte aligned", name);
    uint16_t *t = static_cast<uint16_t *>(target);
    const uint16_t *o = static_cast<const uint16_t *>(other);
    if (aligned16(target) && aligned16(other) && count >= 8)
        update_kernel<kEuler, true><<<blocks_for(count, 8), kThreads, 0, stream>>>(t, o, count, scalar);
    else
        update_kernel<kEuler, false><<<blocks_for(count, 1), kThreads, 0, stream>>>(t, o, count, scalar);
    return finish(name);
}

}  // namespace
}  // namespace krea2

using namespace krea2;

extern "C" int krea2_modulation(krea2_stream stream, size_t count, const void *x, const void *tables, float *y,
                                size_t xsize) {
    clear_error();
    if (int status = check_count("modulation", count)) return status;
    KREA2_REQUIRE(xsize >= 1 && xsize <= 1073741824, "modulation: xsize %zu outside 1..2^30", xsize);
    KREA2_REQUIRE(x && tables && y, "modulation: null buffer");
    KREA2_REQUIRE(reinterpret_cast<uintptr_t>(x) % 2 == 0 && reinterpret_cast<uintptr_t>(tables) % 2 == 0 &&
                      reinterpret_cast<uintptr_t>(y) % 4 == 0,
                  "modulation: buffers must be aligned to their element size");
    const uint16_t *xs = static_cast<const uint16_t *>(x), *ts = static_cast<const uint16_t *>(tables);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (aligned16(x) && aligned16(tables) && aligned16(y) && count % 8 == 0 && xsize % 8 == 0)
        modulation_kernel<true><<<blocks_for(count, 8), kThreads, 0, s>>>(xs, ts, y, count, xsize);
    else
        modulation_kernel<false><<<blocks_for(count, 1), kThreads, 0, s>>>(xs, ts, y, count, xsize);
    return finish("modulation");
}

extern "C" int krea2_euler(krea2_stream stream, size_t count, float delta, void *sample, const void *velocity) {
    clear_error();
    return run_update<true>("euler", static_cast<cudaStream_t>(stream), count, delta, sample, velocity);
}

extern "C" int krea2_guidance(krea2_stream stream, size_t count, float scale, void *cond, const void *uncond) {
    clear_error();
    return run_update<false>("guidance", static_cast<cudaStream_t>(stream), count, scale, cond, uncond);
}

// src/pipeline/schedule.rs:11-14
extern "C" double krea2_schedule_dynamic_mu(size_t image_tokens) {
    const double slope = (1.15 - 0.5) / (6400.0 - 256.0);
    return static_cast<double>(image_tokens) * slope + (0.5 - slope * 256.0);
}

// src/pipeline/schedule.rs:17-27: the linspace value rounds to f32 first; mu stays in double
// through exp and only the shift is rounded.
extern "C" float krea2_schedule_sigma(size_t step, size_t steps, double mu) {
    if (step == steps) return 0.0f;
    const float raw = static_cast<float>(1.0 - static_cast<double>(step) / static_cast<double>(steps));
    const float shift = static_cast<float>(std::exp(mu));
    const float offset = 1.0f / raw - 1.0f;
    return shift / (shift + offset);
}

// src/pipeline/schedule.rs:33-35
extern "C" float krea2_schedule_next_sigma(size_t step, size_t last, size_t steps, double mu) {
    return step + 1 >= last ? 0.0f : krea2_schedule_sigma(step + 1, steps, mu);
}
