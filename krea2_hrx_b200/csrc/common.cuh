// Shared host/device helpers of the krea2_b200 library: the error channel of the C ABI
// and the f32 arithmetic whose every step is one IEEE operation (no contraction, no
// fast-math), so that results do not depend on compiler flags.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/krea2_b200.h"

namespace krea2 {

// ---------------------------------------------------------------- error channel
// Records the message of a failing call for krea2_last_error() and returns `status`.
int fail(krea2_status status, const char *format, ...);
void clear_error();

#define KREA2_CUDA(call)                                                                        \
    do {                                                                                        \
        cudaError_t status_ = (call);                                                           \
        if (status_ != cudaSuccess)                                                             \
            return ::krea2::fail(KREA2_RUNTIME, "%s failed: %s", #call, cudaGetErrorString(status_)); \
    } while (0)

#define KREA2_REQUIRE(condition, ...)                                                           \
    do {                                                                                        \
        if (!(condition)) return ::krea2::fail(KREA2_INVALID_ARGUMENT, __VA_ARGS__);            \
    } while (0)

// Defined with the GEMM: first-use initialisation done ahead of a stream capture.
int prepare_gemm_device();
// Defined with the attention kernel: the same for it, and its share of the device status word.
int prepare_attention_device();
int take_attention_status(int *value);
// Defined with the prologues: their first-use work, for callers about to capture a stream; and
// prepare_gated_i8 whose attention rows have a pitch of their own (in elements).
int prepare_prologue_device(cudaStream_t stream);
int prepare_gated_pitched(cudaStream_t stream, size_t tokens, const void *attn, size_t attn_stride, const void *gate,
                          void *q, float *q_scale, size_t width, size_t out_stride, size_t gate_stride);

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------- dependent launches
// While a session queues the launches of a block chain it raises this thread-local flag: the chain's kernels are
// then launched with programmatic stream serialization, so a kernel's blocks may start -- and run up to their
// chain_wait() -- while the last blocks of the kernel before it are still running.  Every kernel of the chain
// calls chain_wait() before its first access to global memory; without the launch attribute that call returns at
// once, so the same kernels serve ordinary launches.
bool &dependent_launches();

template <typename... Params, typename... Args>
cudaError_t launch_chain_kernel(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream,
                                Args &&...args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attribute = {};
    if (dependent_launches()) {
        attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute.val.programmaticStreamSerializationAllowed = 1;
        config.attrs = &attribute;
        config.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&config, kernel, static_cast<Args &&>(args)...);
}

// ---------------------------------------------------------------- device arithmetic
#ifdef __CUDACC__

// Waits until the kernels this launch depends on have completed and their writes are visible, then lets the next
// launch of the chain start its blocks early in turn (they stop at their own chain_wait()).
__device__ __forceinline__ void chain_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// f32 -> bf16 -> f32, round to nearest even (the `fptrunc ... to bf16` + `extf` pairs of the
// reference kernels; src/numerics.rs:18-26 states the rule).
__device__ __forceinline__ float bf_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// f32 -> f16 -> f32, IEEE round to nearest even.
__device__ __forceinline__ float hf_round(float x) { return __half2float(__float2half_rn(x)); }

// exp with a fixed evaluation order: Cody-Waite reduction by ln 2 in two pieces, the degree-6
// Cephes polynomial, scaling by two exact powers of two.  It stands in for the reference's
// approximate `expf<afn>` (kernels/prepare_gated_i8.loom:99, gemm_i8_swiglu_256.loom:650).
__device__ __forceinline__ float canonical_exp(float x) {
    // Clamped, not branched: above 89 the scaled result overflows to +inf by itself, below -104 it
    // underflows to zero or the smallest subnormal; a NaN passes through.
    float xc = fminf(fmaxf(x, -104.0f), 89.0f);
    float t = __fmul_rn(xc, 1.44269502162933349609375f);
    float n = rintf(t);
    float r = __fmaf_rn(n, -0.693359375f, xc);
    r = __fmaf_rn(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = __fmaf_rn(p, r, 1.3981999507e-3f);
    p = __fmaf_rn(p, r, 8.3334519073e-3f);
    p = __fmaf_rn(p, r, 4.1665795894e-2f);
    p = __fmaf_rn(p, r, 1.6666665459e-1f);
    p = __fmaf_rn(p, r, 5.0000001201e-1f);
    float r2 = __fmul_rn(r, r);
    float y = __fmaf_rn(p, r2, r);
    y = __fadd_rn(y, 1.0f);
    int ni = __float2int_rn(n);
    int h1 = ni >> 1, h2 = ni - h1;  // floor(n/2) and the rest: both exponents stay in range
    float a = __int_as_float((h1 + 127) << 23);
    float b = __int_as_float((h2 + 127) << 23);
    float result = __fmul_rn(__fmul_rn(y, a), b);
    return x != x ? x : result;
}

// 1 / (1 + exp(0 - g)), unrounded f32 (kernels/prepare_gated_i8.loom:98-101).
__device__ __forceinline__ float sigmoid_f32(float g) {
    float e = canonical_exp(__fsub_rn(0.0f, g));
    return __frcp_rn(__fadd_rn(1.0f, e));  // the correctly rounded reciprocal equals the IEEE quotient 1 / den
}

#endif  // __CUDACC__

}  // namespace krea2
