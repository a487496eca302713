// Activation-quantisation prologues of the W8A8 path for sm_100a:
//   krea2_prepare_norm_i8   (kernels/prepare_norm_i8.loom)
//   krea2_prepare_gated_i8  (kernels/prepare_gated_i8.loom)
//   krea2_prepare_plain_i8  (kernels/prepare_plain_i8.loom)
//
// One 256-thread block per token, as the reference lays the row out: thread l owns the
// 8-element chunks j*256 + l (one 128-bit load each), so warp w holds the aligned
// 256-element Hadamard group j*8 + w of every step j.  The row lives in registers from
// the single global read to the packed int8 store; the four radix-4 Hadamard stages run
// inside the warp (stride 1 in-thread, stride 4 across lane bit 0, strides 16 and 64 by
// pairs of xor shuffles), and the only block-wide exchanges are the sum of squares and
// the absmax.  Every f32 step uses the round-to-nearest intrinsics, so the compiler can
// neither fuse nor reorder them and the bits match the CPU statement of the same order.
#include "common.cuh"

namespace krea2 {
namespace {

constexpr int kThreads = 256;
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ uint4 load_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void unpack_bf16(const uint4 &raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[2 * i] = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ void unpack_f16(const uint4 &raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
        v[2 * i] = __low2float(h);
        v[2 * i + 1] = __high2float(h);
    }
}

// bf16 rounding of two values with one packed conversion (cvt.rn.bf16x2.f32).
__device__ __forceinline__ void bf_round2(float &a, float &b) {
    __nv_bfloat162 packed = __floats2bfloat162_rn(a, b);
    const uint32_t u = *reinterpret_cast<uint32_t *>(&packed);
    a = __uint_as_float(u << 16);
    b = __uint_as_float(u & 0xffff0000u);
}

// What each Hadamard stage does to its pair of outputs: nothing for the f32 rotation; a quarter
// and an f16 rounding for the plain prologue (kernels/prepare_plain_i8.loom:120-127).
template <bool kHalf>
__device__ __forceinline__ void stage_round2(float &a, float &b) {
    if constexpr (kHalf) {
        const float2 f = __half22float2(__floats2half2_rn(__fmul_rn(a, 0.25f), __fmul_rn(b, 0.25f)));
        a = f.x;
        b = f.y;
    }
}

// One radix-4 butterfly (kernels/prepare_norm_i8.loom:194-201).
template <bool kHalf>
__device__ __forceinline__ void butterfly(float &e0, float &e1, float &e2, float &e3) {
    float s01 = __fadd_rn(e0, e1), s23 = __fadd_rn(e2, e3);
    float d01 = __fsub_rn(e0, e1), d23 = __fsub_rn(e2, e3);
    e0 = __fadd_rn(s01, d23);
    e1 = __fsub_rn(s01, d23);
    e2 = __fadd_rn(d01, s23);
    e3 = __fsub_rn(s23, d01);
    stage_round2<kHalf>(e0, e1);
    stage_round2<kHalf>(e2, e3);
}

// A radix-4 stage whose four inputs e0..e3 sit in four lanes: lane bit `m1` separates e0|e1
// (and e2|e3), lane bit `m2` separates the pairs.  Every lane forms s = own + partner and
// d = own - partner with its m1 partner, then adds the d of its m2 partner.  For the lanes
// holding e1 and e3, d is the negated pair difference, which is exactly the sign the outputs
// o1 = s01 - d23 and o3 = s23 - d01 want, so one formula serves all four lanes.
template <bool kHalf>
__device__ __forceinline__ void cross_stage(float (&v)[8], int m1, int m2) {
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        float p0 = __shfl_xor_sync(kFull, v[e], m1), p1 = __shfl_xor_sync(kFull, v[e + 1], m1);
        float s0 = __fadd_rn(v[e], p0), s1 = __fadd_rn(v[e + 1], p1);
        float d0 = __fsub_rn(v[e], p0), d1 = __fsub_rn(v[e + 1], p1);
        float q0 = __shfl_xor_sync(kFull, d0, m2), q1 = __shfl_xor_sync(kFull, d1, m2);
        v[e] = __fadd_rn(s0, q0);
        v[e + 1] = __fadd_rn(s1, q1);
        stage_round2<kHalf>(v[e], v[e + 1]);
    }
}

// The group-256 Hadamard of the 8 x 32 values a warp holds (position 8*lane + e), strides
// 1, 4, 16, 64 (kernels/prepare_norm_i8.loom:174-309; prepare_plain_i8.loom:82-279 with the
// f16 rounding after every stage).
template <bool kHalf>
__device__ __forceinline__ void hadamard256(float (&v)[8]) {
    butterfly<kHalf>(v[0], v[1], v[2], v[3]);
    butterfly<kHalf>(v[4], v[5], v[6], v[7]);
    // stride 4: e0, e1 = v[c], v[c+4] of the even lane; e2, e3 = the same of the odd lane.
#pragma unroll
    for (int c = 0; c < 4; c++) {
        float s = __fadd_rn(v[c], v[c + 4]);
        float d = __fsub_rn(v[c], v[c + 4]);
        float dp = __shfl_xor_sync(kFull, d, 1);
        v[c] = __fadd_rn(s, dp);
        v[c + 4] = __fsub_rn(s, dp);
        stage_round2<kHalf>(v[c], v[c + 4]);
    }
    cross_stage<kHalf>(v, 2, 4);
    cross_stage<kHalf>(v, 8, 16);
}

// Four i32 to four saturated int8, first value in the low byte.
__device__ __forceinline__ uint32_t pack_s8x4(int x0, int x1, int x2, int x3) {
    uint32_t out;
    asm("{ .reg .u32 hi;\n"
        "cvt.pack.sat.s8.s32.b32 hi, %4, %3, 0;\n"
        "cvt.pack.sat.s8.s32.b32 %0, %2, %1, hi;\n"
        "}"
        : "=r"(out)
        : "r"(x0), "r"(x1), "r"(x2), "r"(x3));
    return out;
}

__device__ __forceinline__ float block_max(float value, float *scratch, int lane, int warp) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) value = fmaxf(value, __shfl_xor_sync(kFull, value, off));
    if (lane == 0) scratch[warp] = value;
    __syncthreads();
    float m = scratch[0];
#pragma unroll
    for (int i = 1; i < 8; i++) m = fmaxf(m, scratch[i]);
    return m;
}

// absmax -> scale -> packed codes (kernels/prepare_norm_i8.loom:312-372).  `rotation` is what
// is left of the orthonormal 1/16 after the stages: 1/16 for the f32 rotation, 16 for the
// f16 one whose stages already divided by 4 each.
template <int CPL>
__device__ __forceinline__ void quantise_and_store(float (&v)[CPL][8], float rotation, int8_t *q_row,
                                                   float *q_scale, size_t row, float *scratch, int t) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < CPL; j++)
#pragma unroll
        for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[j][e]));
    amax = block_max(amax, scratch, t & 31, t >> 5);
    float row_max = __fmul_rn(amax, rotation);
    float safe = fmaxf(row_max, 1.0000000000000001e-30f);
    float s = __fdiv_rn(safe, 127.0f);
    float inv = __fdiv_rn(rotation, s);
#pragma unroll
    for (int j = 0; j < CPL; j++) {
        // max(x, -127) before rounding equals the clamp after it (-127 is an integer) and sends a
        // NaN to -127 as the reference's maxnum does; the saturating pack clamps at +127.
        int code[8];
#pragma unroll
        for (int e = 0; e < 8; e++) code[e] = __float2int_rn(fmaxf(__fmul_rn(v[j][e], inv), -127.0f));
        *reinterpret_cast<uint2 *>(q_row + 8 * (j * kThreads + t)) =
            make_uint2(pack_s8x4(code[0], code[1], code[2], code[3]), pack_s8x4(code[4], code[5], code[6], code[7]));
    }
    if (t == 0) q_scale[row] = s;
}

template <int CPL>
__global__ void __launch_bounds__(kThreads)
prepare_norm_kernel(const uint16_t *__restrict__ h, const float *__restrict__ norm_scale,
                    const float *__restrict__ mod_scale, const float *__restrict__ mod_shift,
                    int8_t *__restrict__ q, float *__restrict__ q_scale, size_t out_stride, float eps) {
    constexpr int width = CPL * 2048;
    __shared__ float wave_sum[8];
    __shared__ float wave_max[8];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const size_t row = blockIdx.x;
    const uint4 *src = reinterpret_cast<const uint4 *>(h + row * width);
    uint4 raw[CPL];
#pragma unroll
    for (int j = 0; j < CPL; j++) raw[j] = load_stream(src + j * kThreads + t);
    float v[CPL][8];
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < CPL; j++) {
        unpack_bf16(raw[j], v[j]);
#pragma unroll
        for (int e = 0; e < 8; e++) acc[e] = __fmaf_rn(v[j][e], v[j][e], acc[e]);  // the square of a bf16 is exact in f32
    }
    // 8-wide fold, then the wave by xor butterfly, then the eight waves in the reference's
    // written order (kernels/prepare_norm_i8.loom:101-138).
    float ss = __fadd_rn(__fadd_rn(__fadd_rn(acc[0], acc[1]), __fadd_rn(acc[2], acc[3])),
                         __fadd_rn(__fadd_rn(acc[4], acc[5]), __fadd_rn(acc[6], acc[7])));
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(kFull, ss, off));
    if (lane == 0) wave_sum[warp] = ss;
    __syncthreads();
    float total = __fadd_rn(__fadd_rn(__fadd_rn(wave_sum[0], wave_sum[4]), __fadd_rn(wave_sum[2], wave_sum[6])),
                            __fadd_rn(__fadd_rn(wave_sum[1], wave_sum[5]), __fadd_rn(wave_sum[3], wave_sum[7])));
    float mean_eps = __fadd_rn(__fdiv_rn(total, static_cast<float>(width)), eps);
    float rinv = __fdiv_rn(1.0f, __fsqrt_rn(mean_eps));
#pragma unroll
    for (int j = 0; j < CPL; j++) {
        const int base = 8 * (j * kThreads + t);
        float ns[8], ms[8], sh[8];
        *reinterpret_cast<float4 *>(ns) = __ldg(reinterpret_cast<const float4 *>(norm_scale + base));
        *reinterpret_cast<float4 *>(ns + 4) = __ldg(reinterpret_cast<const float4 *>(norm_scale + base + 4));
        *reinterpret_cast<float4 *>(ms) = __ldg(reinterpret_cast<const float4 *>(mod_scale + base));
        *reinterpret_cast<float4 *>(ms + 4) = __ldg(reinterpret_cast<const float4 *>(mod_scale + base + 4));
        *reinterpret_cast<float4 *>(sh) = __ldg(reinterpret_cast<const float4 *>(mod_shift + base));
        *reinterpret_cast<float4 *>(sh + 4) = __ldg(reinterpret_cast<const float4 *>(mod_shift + base + 4));
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            // :152-168: bf16 after the norm scale, bf16 of (1 + mod_scale), bf16 of the product,
            // bf16 after the shift.
            float n0 = __fmul_rn(__fmul_rn(v[j][e], rinv), __fadd_rn(ns[e], 1.0f));
            float n1 = __fmul_rn(__fmul_rn(v[j][e + 1], rinv), __fadd_rn(ns[e + 1], 1.0f));
            bf_round2(n0, n1);
            float m0 = __fadd_rn(ms[e], 1.0f), m1 = __fadd_rn(ms[e + 1], 1.0f);
            bf_round2(m0, m1);
            float s0 = __fmul_rn(n0, m0), s1 = __fmul_rn(n1, m1);
            bf_round2(s0, s1);
            float o0 = __fadd_rn(s0, sh[e]), o1 = __fadd_rn(s1, sh[e + 1]);
            bf_round2(o0, o1);
            v[j][e] = o0;
            v[j][e + 1] = o1;
        }
        hadamard256<false>(v[j]);
    }
    quantise_and_store<CPL>(v, 0.0625f, q + row * out_stride, q_scale, row, wave_max, t);
}

template <int CPL>
__global__ void __launch_bounds__(kThreads)
prepare_gated_kernel(const uint16_t *__restrict__ attn, const uint16_t *__restrict__ gate,
                     int8_t *__restrict__ q, float *__restrict__ q_scale, size_t out_stride,
                     size_t gate_stride) {
    constexpr int width = CPL * 2048;
    __shared__ float wave_max[8];
    const int t = threadIdx.x, lane = t & 31;
    const size_t row = blockIdx.x;
    const uint4 *a_src = reinterpret_cast<const uint4 *>(attn + row * width);
    const uint4 *g_src = reinterpret_cast<const uint4 *>(gate + row * gate_stride);
    uint4 a_raw[CPL], g_raw[CPL];
#pragma unroll
    for (int j = 0; j < CPL; j++) {
        a_raw[j] = load_stream(a_src + j * kThreads + t);
        g_raw[j] = load_stream(g_src + j * kThreads + t);
    }
    float v[CPL][8];
#pragma unroll
    for (int j = 0; j < CPL; j++) {
        float g[8];
        unpack_f16(a_raw[j], v[j]);
        unpack_f16(g_raw[j], g);
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
            // kernels/prepare_gated_i8.loom:94-106
            float a0 = v[j][e], a1 = v[j][e + 1];
            bf_round2(a0, a1);
            float g0 = sigmoid_f32(g[e]), g1 = sigmoid_f32(g[e + 1]);
            bf_round2(g0, g1);
            float o0 = __fmul_rn(a0, g0), o1 = __fmul_rn(a1, g1);
            bf_round2(o0, o1);
            v[j][e] = o0;
            v[j][e + 1] = o1;
        }
        hadamard256<false>(v[j]);
    }
    quantise_and_store<CPL>(v, 0.0625f, q + row * out_stride, q_scale, row, wave_max, t);
}

template <int CPL>
__global__ void __launch_bounds__(kThreads)
prepare_plain_kernel(const uint16_t *__restrict__ h, int8_t *__restrict__ q, float *__restrict__ q_scale,
                     size_t out_stride) {
    constexpr int width = CPL * 2048;
    __shared__ float wave_max[8];
    const int t = threadIdx.x, lane = t & 31;
    const size_t row = blockIdx.x;
    const uint4 *src = reinterpret_cast<const uint4 *>(h + row * width);
    uint4 raw[CPL];
#pragma unroll
    for (int j = 0; j < CPL; j++) raw[j] = load_stream(src + j * kThreads + t);
    float v[CPL][8];
#pragma unroll
    for (int j = 0; j < CPL; j++) {
        unpack_f16(raw[j], v[j]);
        hadamard256<true>(v[j]);
    }
    quantise_and_store<CPL>(v, 16.0f, q + row * out_stride, q_scale, row, wave_max, t);
}

template <template <int> class Launch, typename... Args>
int dispatch_width(size_t width, Args... args) {
    switch (width / 2048) {
#define KREA2_CASE(n) case n: return Launch<n>::run(args...);
        KREA2_CASE(1) KREA2_CASE(2) KREA2_CASE(3) KREA2_CASE(4) KREA2_CASE(5) KREA2_CASE(6) KREA2_CASE(7)
        KREA2_CASE(8) KREA2_CASE(9) KREA2_CASE(10) KREA2_CASE(11) KREA2_CASE(12) KREA2_CASE(13)
        KREA2_CASE(14) KREA2_CASE(15) KREA2_CASE(16)
#undef KREA2_CASE
    }
    return fail(KREA2_INTERNAL, "no prologue instance for width %zu", width);
}

int finish_launch(const char *what) {
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return fail(KREA2_RUNTIME, "%s launch failed: %s", what, cudaGetErrorString(status));
    return KREA2_OK;
}

template <int CPL>
struct LaunchNorm {
    static int run(cudaStream_t stream, size_t tokens, const void *h, const float *ns, const float *ms,
                   const float *sh, void *q, float *q_scale, size_t out_stride, float eps) {
        prepare_norm_kernel<CPL><<<static_cast<unsigned>(tokens), kThreads, 0, stream>>>(
            static_cast<const uint16_t *>(h), ns, ms, sh, static_cast<int8_t *>(q), q_scale, out_stride, eps);
        return finish_launch("prepare_norm_i8");
    }
};
template <int CPL>
struct LaunchGated {
    static int run(cudaStream_t stream, size_t tokens, const void *attn, const void *gate, void *q,
                   float *q_scale, size_t out_stride, size_t gate_stride) {
        prepare_gated_kernel<CPL><<<static_cast<unsigned>(tokens), kThreads, 0, stream>>>(
            static_cast<const uint16_t *>(attn), static_cast<const uint16_t *>(gate), static_cast<int8_t *>(q),
            q_scale, out_stride, gate_stride);
        return finish_launch("prepare_gated_i8");
    }
};
template <int CPL>
struct LaunchPlain {
    static int run(cudaStream_t stream, size_t tokens, const void *h, void *q, float *q_scale,
                   size_t out_stride) {
        prepare_plain_kernel<CPL><<<static_cast<unsigned>(tokens), kThreads, 0, stream>>>(
            static_cast<const uint16_t *>(h), static_cast<int8_t *>(q), q_scale, out_stride);
        return finish_launch("prepare_plain_i8");
    }
};

// The `config.decl` ranges of the three kernels (kernels/prepare_norm_i8.loom:11-16,
// prepare_gated_i8.loom:11-16, prepare_plain_i8.loom:10-13) and the reference's launch
// assumption that tokens is in 1..2^20 (:56).
int check_prologue(const char *name, size_t tokens, size_t width, size_t out_stride) {
    KREA2_REQUIRE(tokens >= 1 && tokens <= 1048576, "%s: tokens %zu outside 1..1048576", name, tokens);
    KREA2_REQUIRE(width >= 2048 && width <= 32768 && width % 2048 == 0,
                  "%s: width %zu must be a multiple of 2048 in 2048..32768", name, width);
    KREA2_REQUIRE(out_stride >= 2048 && out_stride <= 65536 && out_stride % 64 == 0 && out_stride >= width,
                  "%s: out_stride %zu must be a multiple of 64 in 2048..65536 and at least the width", name,
                  out_stride);
    return KREA2_OK;
}

}  // namespace

__global__ void transport_kernel(const uint16_t *__restrict__ src, uint16_t *__restrict__ dst, size_t n,
                                 int reverse) {
    size_t i = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (i >= n) return;
    if (i + 8 <= n) {
        uint4 raw = *reinterpret_cast<const uint4 *>(src + i);
        float v[8];
        uint32_t out[4];
        if (reverse == 1) {
            unpack_bf16(raw, v);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                __half2 h = __halves2half2(__float2half_rn(v[2 * k]), __float2half_rn(v[2 * k + 1]));
                out[k] = *reinterpret_cast<uint32_t *>(&h);
            }
        } else {
            unpack_f16(raw, v);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                __nv_bfloat162 b = __halves2bfloat162(__float2bfloat16_rn(v[2 * k]), __float2bfloat16_rn(v[2 * k + 1]));
                out[k] = *reinterpret_cast<uint32_t *>(&b);
            }
        }
        *reinterpret_cast<uint4 *>(dst + i) = make_uint4(out[0], out[1], out[2], out[3]);
    } else {
        for (; i < n; i++) {
            if (reverse == 1) {
                __half h = __float2half_rn(__uint_as_float(static_cast<uint32_t>(src[i]) << 16));
                dst[i] = *reinterpret_cast<uint16_t *>(&h);
            } else {
                __half h = *reinterpret_cast<const __half *>(&src[i]);
                __nv_bfloat16 b = __float2bfloat16_rn(__half2float(h));
                dst[i] = *reinterpret_cast<uint16_t *>(&b);
            }
        }
    }
}

}  // namespace krea2

using namespace krea2;

extern "C" int krea2_prepare_norm_i8(krea2_stream stream, size_t tokens, const void *h, const float *norm_scale,
                                     const float *mod_scale, const float *mod_shift, void *q, float *q_scale,
                                     size_t width, size_t out_stride, float eps) {
    clear_error();
    if (int status = check_prologue("prepare_norm_i8", tokens, width, out_stride)) return status;
    KREA2_REQUIRE(h && norm_scale && mod_scale && mod_shift && q && q_scale, "prepare_norm_i8: null buffer");
    KREA2_REQUIRE(aligned16(h) && aligned16(norm_scale) && aligned16(mod_scale) && aligned16(mod_shift) &&
                      aligned16(q),
                  "prepare_norm_i8: buffers must be 16-byte aligned");
    KREA2_REQUIRE(eps == eps && eps >= 0.0f, "prepare_norm_i8: eps must be a non-negative number");
    return dispatch_width<LaunchNorm>(width, static_cast<cudaStream_t>(stream), tokens, h, norm_scale, mod_scale,
                                      mod_shift, q, q_scale, out_stride, eps);
}

extern "C" int krea2_prepare_gated_i8(krea2_stream stream, size_t tokens, const void *attn, const void *gate,
                                      void *q, float *q_scale, size_t width, size_t out_stride,
                                      size_t gate_stride) {
    clear_error();
    if (int status = check_prologue("prepare_gated_i8", tokens, width, out_stride)) return status;
    KREA2_REQUIRE(gate_stride >= 256 && gate_stride <= 65536 && gate_stride % 256 == 0 && gate_stride >= width,
                  "prepare_gated_i8: gate_stride %zu must be a multiple of 256 in 256..65536 and at least the width",
                  gate_stride);
    KREA2_REQUIRE(attn && gate && q && q_scale, "prepare_gated_i8: null buffer");
    KREA2_REQUIRE(aligned16(attn) && aligned16(gate) && aligned16(q),
                  "prepare_gated_i8: buffers must be 16-byte aligned");
    return dispatch_width<LaunchGated>(width, static_cast<cudaStream_t>(stream), tokens, attn, gate, q, q_scale,
                                       out_stride, gate_stride);
}

extern "C" int krea2_prepare_plain_i8(krea2_stream stream, size_t tokens, const void *h, void *q, float *q_scale,
                                      size_t width, size_t out_stride) {
    clear_error();
    if (int status = check_prologue("prepare_plain_i8", tokens, width, out_stride)) return status;
    KREA2_REQUIRE(h && q && q_scale, "prepare_plain_i8: null buffer");
    KREA2_REQUIRE(aligned16(h) && aligned16(q), "prepare_plain_i8: buffers must be 16-byte aligned");
    return dispatch_width<LaunchPlain>(width, static_cast<cudaStream_t>(stream), tokens, h, q, q_scale, out_stride);
}

extern "C" int krea2_lora_transport(krea2_stream stream, size_t elements, const void *src, void *dst, int reverse) {
    clear_error();
    KREA2_REQUIRE(reverse == 1 || reverse == 2, "lora_transport: reverse must be 1 (bf16->f16) or 2 (f16->bf16)");
    KREA2_REQUIRE(src && dst && aligned16(src) && aligned16(dst), "lora_transport: buffers must be 16-byte aligned");
    if (elements == 0) return KREA2_OK;
    size_t groups = (elements + 7) / 8;
    unsigned blocks = static_cast<unsigned>((groups + 255) / 256);
    transport_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t *>(src), static_cast<uint16_t *>(dst), elements, reverse);
    return finish_launch("lora_transport");
}
