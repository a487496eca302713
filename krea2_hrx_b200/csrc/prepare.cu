// Activation-quantisation prologues of the W8A8 path for sm_100a:
//   krea2_prepare_norm_i8   (kernels/prepare_norm_i8.loom)
//   krea2_prepare_gated_i8  (kernels/prepare_gated_i8.loom)
//   krea2_prepare_plain_i8  (kernels/prepare_plain_i8.loom)
//
// The kernels are bound by instruction issue, not by HBM, so the layout is chosen to issue few
// instructions per element:
//   * one persistent block per SM; inside it several independent row workers (64 threads per
//     2048 columns each, synchronised by named barriers) so that one worker's loads overlap the
//     others' arithmetic, and what every row needs is staged in shared memory once per block
//     (the norm and modulation vectors; the 64 Ki-entry table of bf16(sigmoid(f16)));
//   * a thread owns 32 positions of one 256-element Hadamard group - the index bits 0-2, 4 and
//     6 - so each radix-4 stage after the first keeps one of its two digits in the thread and
//     needs one shuffle per two outputs (1.5 shuffles per element, not 4.5);
//   * the two values of index bit 6 travel as the halves of packed f32x2 registers through the
//     first three stages, the adaLN arithmetic and the scaling (add/sub/mul.rn.f32x2 are the
//     IEEE operations of their lanes), which halves those issue slots.
// Every f32 step is a single round-to-nearest operation in the order the reference writes, so
// the bits match the CPU statement; the sum of squares is still taken over the reference's
// own thread layout (thread l of 256 owns the 8-element chunks j*256 + l).
#include <atomic>

#include "common.cuh"

namespace krea2 {
namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kSmemLimit = 232448;       // opt-in dynamic shared memory of one sm_100 block
constexpr int kWideThreads = 1024;       // block size limit of the f32 prologues
constexpr int kPlainThreads = 1024;      // of the f16 prologue
constexpr int kSlotFloats = 40;          // per worker and parity: 32 per-warp maxima, the reciprocal, padding

template <int CPL, int MAX_THREADS>
struct Geometry {
    static constexpr int kWidth = 2048 * CPL;
    static constexpr int kChunks = kWidth / 8;          // 16-byte chunks of 8 elements
    static constexpr int kWorkerThreads = 64 * CPL;     // eight lanes per group
    static constexpr int kFit = MAX_THREADS / kWorkerThreads;
    static constexpr int kWorkers = kFit < 1 ? 1 : (kFit > 15 ? 15 : kFit);
    static constexpr int kBlockThreads = kWorkers * kWorkerThreads;
};

// ---------------------------------------------------------------- small pieces
__device__ __forceinline__ uint4 load_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void worker_barrier(int worker, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(worker + 1), "r"(threads) : "memory");
}

__device__ __forceinline__ void copy_async16(void *shared_dst, const void *global_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(shared_dst))),
                 "l"(global_src)
                 : "memory");
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Two f32 values in one 64-bit register pair: `a` is the position with index bit 6 clear, `b`
// the one with it set (or, in the adaLN arithmetic, the next column).
struct F2 {
    float a, b;
};

#define KREA2_PACKED_OP(name, op)                                                                         \
    __device__ __forceinline__ F2 name(F2 x, F2 y) {                                                      \
        F2 d;                                                                                             \
        asm("{ .reg .b64 p, q, r;\n mov.b64 p, {%2, %3};\n mov.b64 q, {%4, %5};\n " op                   \
            ".rn.f32x2 r, p, q;\n mov.b64 {%0, %1}, r;\n }"                                               \
            : "=f"(d.a), "=f"(d.b)                                                                        \
            : "f"(x.a), "f"(x.b), "f"(y.a), "f"(y.b));                                                    \
        return d;                                                                                         \
    }
KREA2_PACKED_OP(add2, "add")
KREA2_PACKED_OP(sub2, "sub")
KREA2_PACKED_OP(mul2, "mul")
#undef KREA2_PACKED_OP

__device__ __forceinline__ F2 both(float v) { return F2{v, v}; }

__device__ __forceinline__ F2 shfl2(F2 v, int mask) {
    return F2{__shfl_xor_sync(kFull, v.a, mask), __shfl_xor_sync(kFull, v.b, mask)};
}

// Columns 2k and 2k+1 of a bf16x2 word.
__device__ __forceinline__ F2 unpack_bf16x2(uint32_t w) {
    return F2{__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u)};
}

__device__ __forceinline__ F2 unpack_f16x2(uint32_t w) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
    return F2{f.x, f.y};
}

// The mixed-precision forms below read a 16-bit operand as the IEEE value it encodes and do one
// f32 operation with one rounding, so each equals the convert-then-operate sequence it replaces
// (every bf16 or f16 value is an f32 value).
// f32(h) * 0.25 for both halves of an f16x2 word: the f16 stage scale folded into the unpack.  A
// power-of-two scale commutes with every later rounding of the stage, nothing being near the f32
// or f16 underflow range after it (|x| >= 2^-26 or zero).
__device__ __forceinline__ F2 unpack_quarter_f16x2(uint32_t w) {
    F2 d;
    asm("{ .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %2;\n fma.rn.f32.f16 %0, lo, %3, %4;\n fma.rn.f32.f16 %1, hi, %3, %4;\n }"
        : "=f"(d.a), "=f"(d.b)
        : "r"(w), "h"(static_cast<unsigned short>(0x3400)), "f"(-0.0f));
    return d;
}
// acc + x*x for both bf16 halves of w.
__device__ __forceinline__ void square_accumulate_bf16x2(uint32_t w, float &lo_acc, float &hi_acc) {
    asm("{ .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %2;\n fma.rn.f32.bf16 %0, lo, lo, %0;\n fma.rn.f32.bf16 %1, hi, hi, %1;\n }"
        : "+f"(lo_acc), "+f"(hi_acc)
        : "r"(w));
}
// The f32 products of the halves of two bf16x2 words (x*y + -0 is the rounded product, signed zeros kept).
__device__ __forceinline__ F2 product_bf16x2(uint32_t x, uint32_t y) {
    F2 d;
    asm("{ .reg .b16 xl, xh, yl, yh;\n mov.b32 {xl, xh}, %2;\n mov.b32 {yl, yh}, %3;\n"
        " fma.rn.f32.bf16 %0, xl, yl, %4;\n fma.rn.f32.bf16 %1, xh, yh, %4;\n }"
        : "=f"(d.a), "=f"(d.b)
        : "r"(x), "r"(y), "f"(-0.0f));
    return d;
}
// The halves of a bf16x2 word plus two f32 addends.
__device__ __forceinline__ F2 add_bf16x2(uint32_t x, F2 addend) {
    F2 d;
    asm("{ .reg .b16 lo, hi;\n mov.b32 {lo, hi}, %2;\n add.rn.f32.bf16 %0, lo, %3;\n add.rn.f32.bf16 %1, hi, %4;\n }"
        : "=f"(d.a), "=f"(d.b)
        : "r"(x), "f"(addend.a), "f"(addend.b));
    return d;
}
__device__ __forceinline__ uint32_t pack_bf16x2(F2 v) {
    __nv_bfloat162 packed = __floats2bfloat162_rn(v.a, v.b);
    return *reinterpret_cast<uint32_t *>(&packed);
}

// bf16 rounding of both halves with one packed conversion (cvt.rn.bf16x2.f32).
__device__ __forceinline__ F2 bf_round2(F2 v) {
    __nv_bfloat162 packed = __floats2bfloat162_rn(v.a, v.b);
    return unpack_bf16x2(*reinterpret_cast<uint32_t *>(&packed));
}

__device__ __forceinline__ uint32_t pack_f16x2(F2 v) {
    __half2 h = __floats2half2_rn(v.a, v.b);
    return *reinterpret_cast<uint32_t *>(&h);
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

// ---------------------------------------------------------------- thread layout
// Chunk c of a group (its index bits 3-7) is split as c = c0 + 2 c1 + 4 c2 + 8 c3 + 16 c4:
// c0, c2, c4 are lane bits 0-2, c1 and c3 live in the thread, lane bits 3-4 and the warp pick
// the group.  `first_chunk` is the thread's chunk at c1 = c3 = 0.
struct Layout {
    int first_chunk;
    __device__ __forceinline__ int chunk(int c3, int c1) const { return first_chunk + 8 * c3 + 2 * c1; }
};

__device__ __forceinline__ Layout make_layout(int warp_in_worker, int lane) {
    const int group = warp_in_worker * 4 + (lane >> 3);
    return Layout{group * 32 + (lane & 1) + 4 * ((lane >> 1) & 1) + 16 * ((lane >> 2) & 1)};
}

// Row staging in shared memory: chunk i sits in slot i ^ 2*(bit 4 of i), so that the eight
// lanes of a quarter warp (which differ in c0, c2 and c4) hit eight different 16-byte columns.
__device__ __forceinline__ int staged_slot(int chunk) { return chunk ^ (((chunk >> 4) & 1) << 1); }
// The same for the staged f32 vectors, whose 16-byte unit u = column / 4 carries c0, c2, c4 in
// its bits 1, 3, 5: unit u sits in slot u ^ bit 3 ^ 4*bit 5.
__device__ __forceinline__ int vector_slot(int unit) { return unit ^ ((unit >> 3) & 1) ^ (((unit >> 5) & 1) << 2); }

// ---------------------------------------------------------------- Hadamard, f32 (norm, gated)
// One radix-4 butterfly on both halves (kernels/prepare_norm_i8.loom:194-201).
__device__ __forceinline__ void butterfly2(F2 &e0, F2 &e1, F2 &e2, F2 &e3) {
    F2 s01 = add2(e0, e1), s23 = add2(e2, e3);
    F2 d01 = sub2(e0, e1), d23 = sub2(e2, e3);
    e0 = add2(s01, d23);
    e1 = sub2(s01, d23);
    e2 = add2(d01, s23);
    e3 = sub2(s23, d01);
}

// A radix-4 stage whose low digit is in the thread (`lo`, `hi`) and whose high digit is the
// lane bit `mask`: the lane computes the sum and difference of its own pair and receives the
// partner's difference.  For the lane holding e2, e3 the received value is d01 and its own sum is
// s23, and o2 = d01 + s23, o3 = s23 - d01 are the same two expressions.
__device__ __forceinline__ void split_stage(F2 &lo, F2 &hi, int mask) {
    F2 s = add2(lo, hi), d = sub2(lo, hi);
    F2 dp = shfl2(d, mask);
    lo = add2(s, dp);
    hi = sub2(s, dp);
}

// The last stage (strides 64 | 128): its low digit is the packing dimension itself.
__device__ __forceinline__ void unpacked_stage(F2 &v, int mask) {
    float s = __fadd_rn(v.a, v.b), d = __fsub_rn(v.a, v.b);
    float dp = __shfl_xor_sync(kFull, d, mask);
    v.a = __fadd_rn(s, dp);
    v.b = __fsub_rn(s, dp);
}

// The group-256 Hadamard of the thread's group, strides 1, 4, 16, 64
// (kernels/prepare_norm_i8.loom:174-309).  x[c1][e]: positions e + 16 c1 (+ lanes), halves c3.
__device__ __forceinline__ void hadamard256(F2 (&x)[2][8]) {
#pragma unroll
    for (int c1 = 0; c1 < 2; c1++) {
        butterfly2(x[c1][0], x[c1][1], x[c1][2], x[c1][3]);
        butterfly2(x[c1][4], x[c1][5], x[c1][6], x[c1][7]);
#pragma unroll
        for (int c = 0; c < 4; c++) split_stage(x[c1][c], x[c1][c + 4], 1);  // strides 4 | 8
    }
#pragma unroll
    for (int e = 0; e < 8; e++) split_stage(x[0][e], x[1][e], 2);  // strides 16 | 32
#pragma unroll
    for (int c1 = 0; c1 < 2; c1++)
#pragma unroll
        for (int e = 0; e < 8; e++) unpacked_stage(x[c1][e], 4);  // strides 64 | 128
}

// ---------------------------------------------------------------- absmax and codes
__device__ __forceinline__ float warp_max(float value) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) value = fmaxf(value, __shfl_xor_sync(kFull, value, off));
    return value;
}

// scale and its reciprocal from the row absmax (kernels/prepare_norm_i8.loom:312-330).  `rotation`
// is what is left of the orthonormal 1/16 after the stages: 1/16 for the f32 rotation, 16 for
// the f16 one whose stages already divided by 4 each.
__device__ __forceinline__ void row_scale(float amax, float rotation, float &s, float &inv) {
    float row_max = __fmul_rn(amax, rotation);
    float safe = fmaxf(row_max, 1.0000000000000001e-30f);
    s = __fdiv_rn(safe, 127.0f);
    inv = __fdiv_rn(rotation, s);
}

// Eight values of each half to eight codes each (:331-372).  max(x, -127) before rounding
// equals the clamp after it (-127 is an integer) and sends a NaN to -127 as the reference's
// maxnum does; the saturating pack clamps at +127.
__device__ __forceinline__ void store_codes(const F2 (&v)[8], float inv, int8_t *first, int8_t *second) {
    int ca[8], cb[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {
        F2 t = mul2(v[e], both(inv));
        ca[e] = __float2int_rn(fmaxf(t.a, -127.0f));
        cb[e] = __float2int_rn(fmaxf(t.b, -127.0f));
    }
    *reinterpret_cast<uint2 *>(first) = make_uint2(pack_s8x4(ca[0], ca[1], ca[2], ca[3]), pack_s8x4(ca[4], ca[5], ca[6], ca[7]));
    *reinterpret_cast<uint2 *>(second) = make_uint2(pack_s8x4(cb[0], cb[1], cb[2], cb[3]), pack_s8x4(cb[4], cb[5], cb[6], cb[7]));
}

// From the threads' absmax to the row's scale and its reciprocal.  The warps' maxima meet in `slots`
// (32 floats, then two for the results); the worker's first warp alone reduces them and does the two
// divisions, the others wait at a second barrier and read the reciprocal, so the scalar work is issued once
// per row instead of once per warp.  `slots` is double-buffered by the caller.
template <int WARPS>
__device__ __forceinline__ float row_reciprocal(float amax, float rotation, float *slots, int worker, int warp_in_worker,
                                                int lane, float *scale_out) {
    amax = warp_max(amax);
    if (lane == 0) slots[warp_in_worker] = amax;
    worker_barrier(worker, 32 * WARPS);
    if (warp_in_worker == 0) {
        const float m = warp_max(lane < WARPS ? slots[lane] : 0.0f);
        float s, inv;
        row_scale(m, rotation, s, inv);
        if (lane == 0) {
            slots[32] = inv;
            *scale_out = s;
        }
    }
    worker_barrier(worker, 32 * WARPS);
    return slots[32];
}

// Row absmax over the worker (per-warp maxima in `slots`, double-buffered by the caller),
// then the codes of the thread's 32 positions and the row scale.
template <int WARPS>
__device__ __forceinline__ void quantise_f32(F2 (&x)[2][8], float *slots, int worker, int warp_in_worker,
                                             int lane, const Layout &layout, int8_t *q_row, float *scale_out) {
    float amax = 0.0f;
#pragma unroll
    for (int c1 = 0; c1 < 2; c1++)
#pragma unroll
        for (int e = 0; e < 8; e++) amax = fmaxf(amax, fmaxf(fabsf(x[c1][e].a), fabsf(x[c1][e].b)));
    const float inv = row_reciprocal<WARPS>(amax, 0.0625f, slots, worker, warp_in_worker, lane, scale_out);
#pragma unroll
    for (int c1 = 0; c1 < 2; c1++)
        store_codes(x[c1], inv, q_row + 8 * layout.chunk(0, c1), q_row + 8 * layout.chunk(1, c1));
}

// The rows of one block and of one worker in it: blocks split the rows evenly, workers
// interleave inside a block.
struct Rows {
    size_t next, end;
};
__device__ __forceinline__ Rows worker_rows(size_t tokens, int worker) {
    const size_t first = tokens * blockIdx.x / gridDim.x, last = tokens * (blockIdx.x + 1) / gridDim.x;
    return Rows{first + worker, last};
}

// ---------------------------------------------------------------- prepare_norm_i8
template <int CPL>
struct NormPlan {
    using G = Geometry<CPL, kWideThreads>;
    static constexpr int kRowBytes = 2 * G::kWorkers * G::kWidth * 2;  // two buffers per worker
    static constexpr int kSmallBytes = G::kWorkers * (12 + 2 * kSlotFloats) * 4;
    static constexpr int kVectorBytes = G::kWidth * (4 + 4 + 2);
    static constexpr bool kStaged = kVectorBytes + kRowBytes + kSmallBytes <= kSmemLimit;
    static constexpr int kBytes = (kStaged ? kVectorBytes : 0) + kRowBytes + kSmallBytes;
};

// adaLN on the eight columns of one chunk (kernels/prepare_norm_i8.loom:152-168): bf16 after the
// norm scale, bf16 of (1 + mod_scale), bf16 of the product, bf16 after the shift.  `one_plus_norm`
// is 1 + norm_scale per column, `modulation` the bf16x2 words of bf16(1 + mod_scale).
__device__ __forceinline__ void adaln_chunk(const uint4 &raw, float rinv, const float *one_plus_norm,
                                            const uint32_t *modulation, const float *shift, float (&out)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const uint32_t n = pack_bf16x2(
            mul2(mul2(unpack_bf16x2(w[k]), both(rinv)), F2{one_plus_norm[2 * k], one_plus_norm[2 * k + 1]}));
        const uint32_t s = pack_bf16x2(product_bf16x2(n, modulation[k]));
        const F2 o = bf_round2(add_bf16x2(s, F2{shift[2 * k], shift[2 * k + 1]}));
        out[2 * k] = o.a;
        out[2 * k + 1] = o.b;
    }
}

template <int CPL>
__global__ void __launch_bounds__(Geometry<CPL, kWideThreads>::kBlockThreads, 1)
prepare_norm_kernel(const uint16_t *__restrict__ h, const float *__restrict__ norm_scale,
                    const float *__restrict__ mod_scale, const float *__restrict__ mod_shift,
                    int8_t *__restrict__ q, float *__restrict__ q_scale, size_t out_stride, float eps,
                    size_t tokens) {
    chain_wait();
    using G = Geometry<CPL, kWideThreads>;
    using Plan = NormPlan<CPL>;
    constexpr int width = G::kWidth;
    constexpr int kWarps = 2 * CPL;                      // of one worker
    constexpr int kVirtual = (8 + kWarps - 1) / kWarps;  // reference waves (of 8) a warp sums
    extern __shared__ __align__(16) uint8_t smem[];
    float *vec_norm = reinterpret_cast<float *>(smem);
    float *vec_shift = vec_norm + width;
    uint4 *vec_mod = reinterpret_cast<uint4 *>(vec_shift + width);  // one 16-byte unit per chunk
    uint4 *row_store = reinterpret_cast<uint4 *>(smem + (Plan::kStaged ? Plan::kVectorBytes : 0));
    float *sum_store = reinterpret_cast<float *>(row_store + 2 * G::kWorkers * G::kChunks);
    float *max_store = sum_store + G::kWorkers * 12;

    if constexpr (Plan::kStaged) {
        for (int chunk = threadIdx.x; chunk < G::kChunks; chunk += G::kBlockThreads) {
            const int c = chunk * 8;
            uint32_t m[4];
#pragma unroll
            for (int half = 0; half < 2; half++) {
                float4 ns = __ldg(reinterpret_cast<const float4 *>(norm_scale + c + 4 * half));
                float4 ms = __ldg(reinterpret_cast<const float4 *>(mod_scale + c + 4 * half));
                float4 sh = __ldg(reinterpret_cast<const float4 *>(mod_shift + c + 4 * half));
                const int slot = 4 * vector_slot(2 * chunk + half);
                *reinterpret_cast<float4 *>(vec_norm + slot) = make_float4(
                    __fadd_rn(ns.x, 1.0f), __fadd_rn(ns.y, 1.0f), __fadd_rn(ns.z, 1.0f), __fadd_rn(ns.w, 1.0f));
                *reinterpret_cast<float4 *>(vec_shift + slot) = sh;
                m[2 * half] = pack_bf16x2(F2{__fadd_rn(ms.x, 1.0f), __fadd_rn(ms.y, 1.0f)});
                m[2 * half + 1] = pack_bf16x2(F2{__fadd_rn(ms.z, 1.0f), __fadd_rn(ms.w, 1.0f)});
            }
            vec_mod[staged_slot(chunk)] = make_uint4(m[0], m[1], m[2], m[3]);
        }
        __syncthreads();
    }

    const int worker = threadIdx.x / G::kWorkerThreads, t = threadIdx.x % G::kWorkerThreads;
    const int lane = t & 31, warp = t >> 5;
    const Layout layout = make_layout(warp, lane);
    uint4 *row_bufs = row_store + 2 * worker * G::kChunks;
    float *sums = sum_store + worker * 12;  // eight wave sums, then the row's 1 / rms
    float *maxes = max_store + worker * 2 * kSlotFloats;
    int parity = 0;

    // The next row streams into the worker's other buffer (16-byte asynchronous copies, slot-swizzled)
    // while this one is worked on; the wait for it sits in front of a barrier the row needs anyway.
    auto fetch = [&](size_t row, int buffer) {
        const uint4 *src = reinterpret_cast<const uint4 *>(h + row * width);
        uint4 *dst = row_bufs + buffer * G::kChunks;
#pragma unroll
        for (int i = 0; i < 4; i++) copy_async16(dst + staged_slot(t + i * G::kWorkerThreads), src + t + i * G::kWorkerThreads);
        copy_async_commit();
    };
    Rows rows = worker_rows(tokens, worker);
    if (rows.next < rows.end) {
        fetch(rows.next, 0);
        copy_async_wait();
    }
    worker_barrier(worker, G::kWorkerThreads);

    for (; rows.next < rows.end; rows.next += G::kWorkers, parity ^= kSlotFloats) {
        const size_t row = rows.next;
        const uint4 *row_buf = row_bufs + (parity ? G::kChunks : 0);
        if (row + G::kWorkers < rows.end) fetch(row + G::kWorkers, parity ? 0 : 1);
        // Sum of squares in the reference's layout: its wave v, lane l, step j owns chunk
        // j*256 + v*32 + l.  A warp of this worker takes the waves warp, warp + 2 CPL, ...
#pragma unroll
        for (int i = 0; i < kVirtual; i++) {
            const int wave = warp + i * kWarps;
            if (wave < 8) {
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < CPL; j++) {
                    const uint4 raw = row_buf[staged_slot(j * 256 + wave * 32 + lane)];
                    square_accumulate_bf16x2(raw.x, acc[0], acc[1]);  // the square of a bf16 is exact in f32
                    square_accumulate_bf16x2(raw.y, acc[2], acc[3]);
                    square_accumulate_bf16x2(raw.z, acc[4], acc[5]);
                    square_accumulate_bf16x2(raw.w, acc[6], acc[7]);
                }
                // 8-wide fold, then the wave by xor butterfly (kernels/prepare_norm_i8.loom:101-125).
                float ss = __fadd_rn(__fadd_rn(__fadd_rn(acc[0], acc[1]), __fadd_rn(acc[2], acc[3])),
                                     __fadd_rn(__fadd_rn(acc[4], acc[5]), __fadd_rn(acc[6], acc[7])));
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(kFull, ss, off));
                if (lane == 0) sums[wave] = ss;
            }
        }
        worker_barrier(worker, G::kWorkerThreads);
        if (warp == 0) {
            // The eight waves in the reference's written order (:126-138); one warp does the divisions and
            // the square root for the row.
            float total = __fadd_rn(__fadd_rn(__fadd_rn(sums[0], sums[4]), __fadd_rn(sums[2], sums[6])),
                                    __fadd_rn(__fadd_rn(sums[1], sums[5]), __fadd_rn(sums[3], sums[7])));
            float mean_eps = __fadd_rn(__fdiv_rn(total, static_cast<float>(width)), eps);
            if (lane == 0) sums[8] = __fdiv_rn(1.0f, __fsqrt_rn(mean_eps));
        }
        worker_barrier(worker, G::kWorkerThreads);
        const float rinv = sums[8];

        F2 x[2][8];
#pragma unroll
        for (int c1 = 0; c1 < 2; c1++)
#pragma unroll
            for (int c3 = 0; c3 < 2; c3++) {
                {
                    const int chunk = layout.chunk(c3, c1), col = chunk * 8;
                    const uint4 packed = row_buf[staged_slot(chunk)];
                    float o[8], ns[8], sh[8];
                    uint32_t m[4];
                    if constexpr (Plan::kStaged) {
                        const int lo = 4 * vector_slot(2 * chunk), hi = 4 * vector_slot(2 * chunk + 1);
                        *reinterpret_cast<float4 *>(ns) = *reinterpret_cast<const float4 *>(vec_norm + lo);
                        *reinterpret_cast<float4 *>(ns + 4) = *reinterpret_cast<const float4 *>(vec_norm + hi);
                        *reinterpret_cast<float4 *>(sh) = *reinterpret_cast<const float4 *>(vec_shift + lo);
                        *reinterpret_cast<float4 *>(sh + 4) = *reinterpret_cast<const float4 *>(vec_shift + hi);
                        *reinterpret_cast<uint4 *>(m) = vec_mod[staged_slot(chunk)];
                    } else {
                        float ms[8];
                        *reinterpret_cast<float4 *>(ns) = __ldg(reinterpret_cast<const float4 *>(norm_scale + col));
                        *reinterpret_cast<float4 *>(ns + 4) = __ldg(reinterpret_cast<const float4 *>(norm_scale + col + 4));
                        *reinterpret_cast<float4 *>(ms) = __ldg(reinterpret_cast<const float4 *>(mod_scale + col));
                        *reinterpret_cast<float4 *>(ms + 4) = __ldg(reinterpret_cast<const float4 *>(mod_scale + col + 4));
                        *reinterpret_cast<float4 *>(sh) = __ldg(reinterpret_cast<const float4 *>(mod_shift + col));
                        *reinterpret_cast<float4 *>(sh + 4) = __ldg(reinterpret_cast<const float4 *>(mod_shift + col + 4));
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            m[k] = pack_bf16x2(F2{__fadd_rn(ms[2 * k], 1.0f), __fadd_rn(ms[2 * k + 1], 1.0f)});
                            ns[2 * k] = __fadd_rn(ns[2 * k], 1.0f);
                            ns[2 * k + 1] = __fadd_rn(ns[2 * k + 1], 1.0f);
                        }
                    }
                    adaln_chunk(packed, rinv, ns, m, sh, o);
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        if (c3 == 0) x[c1][e].a = o[e];
                        else x[c1][e].b = o[e];
                    }
                }
            }
        hadamard256(x);
        copy_async_wait();  // the next row: published by the barrier inside quantise_f32
        quantise_f32<kWarps>(x, maxes + parity, worker, warp, lane, layout, q + row * out_stride, q_scale + row);
    }
}

// ---------------------------------------------------------------- prepare_gated_i8
// bf16(sigmoid(g)) of every f16 bit pattern g, filled once per device by the kernel below; the
// blocks of the prologue copy it into shared memory (or compute it themselves while
// `g_sigmoid_ready` is still 0, e.g. when another stream's first call is filling it).
__device__ __align__(16) uint16_t g_sigmoid_table[65536];
__device__ unsigned g_sigmoid_blocks;
__device__ int g_sigmoid_ready;

// kernels/prepare_gated_i8.loom:98-102: the f32 sigmoid of the f16 gate, rounded to bf16.
__device__ __forceinline__ uint16_t sigmoid_entry(unsigned bits) {
    const __half g = __ushort_as_half(static_cast<unsigned short>(bits));
    const __nv_bfloat16 r = __float2bfloat16_rn(sigmoid_f32(__half2float(g)));
    return __bfloat16_as_ushort(r);
}

__global__ void __launch_bounds__(256) sigmoid_table_kernel() {
    const unsigned i = blockIdx.x * 256 + threadIdx.x;
    g_sigmoid_table[i] = sigmoid_entry(i);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(&g_sigmoid_blocks, 1u) + 1u;
        if (done % gridDim.x == 0) {
            __threadfence();
            atomicExch(&g_sigmoid_ready, 1);
        }
    }
}

constexpr int kTableBytes = 65536 * 2;

template <int CPL>
struct GatedPlan {
    using G = Geometry<CPL, kWideThreads>;
    static constexpr int kBytes = kTableBytes + G::kWorkers * 2 * kSlotFloats * 4 + 16;
};

template <int CPL>
__global__ void __launch_bounds__(Geometry<CPL, kWideThreads>::kBlockThreads, 1)
prepare_gated_kernel(const uint16_t *__restrict__ attn, const uint16_t *__restrict__ gate,
                     int8_t *__restrict__ q, float *__restrict__ q_scale, size_t out_stride,
                     size_t gate_stride, size_t attn_stride, size_t tokens) {
    chain_wait();
    using G = Geometry<CPL, kWideThreads>;
    constexpr int kWarps = 2 * CPL;
    extern __shared__ __align__(16) uint8_t smem[];
    uint16_t *table = reinterpret_cast<uint16_t *>(smem);
    float *max_store = reinterpret_cast<float *>(smem + kTableBytes);
    int *ready = reinterpret_cast<int *>(max_store + G::kWorkers * 2 * kSlotFloats);

    if (threadIdx.x == 0) {
        int flag;
        asm volatile("ld.acquire.gpu.s32 %0, [%1];" : "=r"(flag) : "l"(&g_sigmoid_ready) : "memory");
        *ready = flag;
    }
    __syncthreads();
    if (*ready) {
        const uint4 *src = reinterpret_cast<const uint4 *>(g_sigmoid_table);
        for (int i = threadIdx.x; i < kTableBytes / 16; i += G::kBlockThreads)
            reinterpret_cast<uint4 *>(table)[i] = __ldcg(src + i);
    } else {
        for (unsigned i = threadIdx.x; i < 65536u; i += G::kBlockThreads) table[i] = sigmoid_entry(i);
    }
    __syncthreads();

    const int worker = threadIdx.x / G::kWorkerThreads, t = threadIdx.x % G::kWorkerThreads;
    const int lane = t & 31, warp = t >> 5;
    const Layout layout = make_layout(warp, lane);
    float *maxes = max_store + worker * 2 * kSlotFloats;
    int parity = 0;

    for (Rows rows = worker_rows(tokens, worker); rows.next < rows.end; rows.next += G::kWorkers, parity ^= kSlotFloats) {
        const size_t row = rows.next;
        const uint4 *a_src = reinterpret_cast<const uint4 *>(attn + row * attn_stride);
        const uint4 *g_src = reinterpret_cast<const uint4 *>(gate + row * gate_stride);
        uint4 a_raw[2][2], g_raw[2][2];
#pragma unroll
        for (int c1 = 0; c1 < 2; c1++)
#pragma unroll
            for (int c3 = 0; c3 < 2; c3++) {
                a_raw[c1][c3] = load_stream(a_src + layout.chunk(c3, c1));
                g_raw[c1][c3] = load_stream(g_src + layout.chunk(c3, c1));
            }
        F2 x[2][8];
#pragma unroll
        for (int c1 = 0; c1 < 2; c1++)
#pragma unroll
            for (int c3 = 0; c3 < 2; c3++) {
                const uint4 &ar = a_raw[c1][c3], &gr = g_raw[c1][c3];
                const uint32_t aw[4] = {ar.x, ar.y, ar.z, ar.w}, gw[4] = {gr.x, gr.y, gr.z, gr.w};
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    // kernels/prepare_gated_i8.loom:94-106
                    const uint32_t a = pack_bf16x2(unpack_f16x2(aw[k]));
                    const uint32_t g = static_cast<uint32_t>(table[gw[k] & 0xffffu]) |
                                       (static_cast<uint32_t>(table[gw[k] >> 16]) << 16);
                    F2 o = bf_round2(product_bf16x2(a, g));
                    if (c3 == 0) {
                        x[c1][2 * k].a = o.a;
                        x[c1][2 * k + 1].a = o.b;
                    } else {
                        x[c1][2 * k].b = o.a;
                        x[c1][2 * k + 1].b = o.b;
                    }
                }
            }
        hadamard256(x);
        quantise_f32<kWarps>(x, maxes + parity, worker, warp, lane, layout, q + row * out_stride, q_scale + row);
    }
}

// ---------------------------------------------------------------- prepare_plain_i8
// The f16 Hadamard (kernels/prepare_plain_i8.loom:82-279): every stage ends in a quarter and an
// f16 rounding, so between stages the row is held as f16x2 words, low half = first group.
// A stage scales its inputs by a quarter while unpacking them (see unpack_quarter_f16x2) and
// rounds its outputs to f16.
__device__ __forceinline__ void split_stage_f16(uint32_t &lo, uint32_t &hi, int mask) {
    F2 a = unpack_quarter_f16x2(lo), b = unpack_quarter_f16x2(hi);
    F2 s = add2(a, b), d = sub2(a, b);
    F2 dp = shfl2(d, mask);
    lo = pack_f16x2(add2(s, dp));
    hi = pack_f16x2(sub2(s, dp));
}

__device__ __forceinline__ void unpacked_stage_f16(uint32_t &w, int mask) {
    F2 v = unpack_quarter_f16x2(w);
    float s = __fadd_rn(v.a, v.b), d = __fsub_rn(v.a, v.b);
    float dp = __shfl_xor_sync(kFull, d, mask);
    w = pack_f16x2(F2{__fadd_rn(s, dp), __fsub_rn(s, dp)});
}

template <int CPL>
struct PlainPlan {
    using G = Geometry<CPL, kPlainThreads>;
    static constexpr int kStageBytes = 2 * 4 * 16 * G::kBlockThreads;  // two rows of four chunks per thread
    static constexpr int kBytes = kStageBytes + G::kWorkers * 2 * kSlotFloats * 4;
};

// kRotated: the row arrives with the first three stages (strides 1, 4, 16) already applied by the SwiGLU
// epilogue that wrote it (krea2_gemm_i8_swiglu_rotated_256); only the last stage, the row maximum and the codes
// are left.
template <int CPL, bool kRotated>
__global__ void __launch_bounds__(Geometry<CPL, kPlainThreads>::kBlockThreads, 1)
prepare_plain_kernel(const uint16_t *__restrict__ h, int8_t *__restrict__ q, float *__restrict__ q_scale,
                     size_t out_stride, size_t tokens) {
    chain_wait();
    using G = Geometry<CPL, kPlainThreads>;
    constexpr int width = G::kWidth;
    constexpr int kWarps = 2 * CPL;
    extern __shared__ __align__(16) uint8_t smem[];
    uint4 *stage = reinterpret_cast<uint4 *>(smem);
    float *max_store = reinterpret_cast<float *>(smem + PlainPlan<CPL>::kStageBytes);
    const int worker = threadIdx.x / G::kWorkerThreads, t = threadIdx.x % G::kWorkerThreads;
    const int lane = t & 31, warp = t >> 5;
    const Layout layout = make_layout(warp, lane);
    float *maxes = max_store + worker * 2 * kSlotFloats;
    int parity = 0;

    // Each thread streams its own four chunks of the next row into shared memory while it works
    // on this one: slot (buffer, piece) of thread x is stage[(buffer*4 + piece) * threads + x].
    auto fetch = [&](size_t row, int buffer) {
        const uint4 *src = reinterpret_cast<const uint4 *>(h + row * width);
#pragma unroll
        for (int piece = 0; piece < 4; piece++)
            copy_async16(stage + (buffer * 4 + piece) * G::kBlockThreads + threadIdx.x,
                         src + layout.chunk(piece & 1, piece >> 1));
        copy_async_commit();
    };
    Rows rows = worker_rows(tokens, worker);
    if (rows.next < rows.end) fetch(rows.next, 0);

    for (; rows.next < rows.end; rows.next += G::kWorkers, parity ^= kSlotFloats) {
        const size_t row = rows.next;
        const int buffer = parity ? 1 : 0;
        copy_async_wait();
        uint32_t x[2][8];  // f16x2 words: low half c3 = 0, high half c3 = 1
#pragma unroll
        for (int c1 = 0; c1 < 2; c1++) {
            const uint4 ra = stage[(buffer * 4 + 2 * c1) * G::kBlockThreads + threadIdx.x];
            const uint4 rb = stage[(buffer * 4 + 2 * c1 + 1) * G::kBlockThreads + threadIdx.x];
            const uint32_t aw[4] = {ra.x, ra.y, ra.z, ra.w}, bw[4] = {rb.x, rb.y, rb.z, rb.w};
            if constexpr (kRotated) {
                // element k of chunk a (index bit 6 clear) in the low half, of chunk b in the high half
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    x[c1][2 * k] = __byte_perm(aw[k], bw[k], 0x5410);
                    x[c1][2 * k + 1] = __byte_perm(aw[k], bw[k], 0x7632);
                }
            } else {
                F2 e[8];
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const F2 fa = unpack_quarter_f16x2(aw[k]), fb = unpack_quarter_f16x2(bw[k]);
                    e[2 * k] = F2{fa.a, fb.a};
                    e[2 * k + 1] = F2{fa.b, fb.b};
                }
                butterfly2(e[0], e[1], e[2], e[3]);
                butterfly2(e[4], e[5], e[6], e[7]);
#pragma unroll
                for (int k = 0; k < 8; k++) x[c1][k] = pack_f16x2(e[k]);
#pragma unroll
                for (int c = 0; c < 4; c++) split_stage_f16(x[c1][c], x[c1][c + 4], 1);
            }
        }
        if (row + G::kWorkers < rows.end) fetch(row + G::kWorkers, buffer ^ 1);
        if constexpr (!kRotated) {
#pragma unroll
            for (int e = 0; e < 8; e++) split_stage_f16(x[0][e], x[1][e], 2);
        }
#pragma unroll
        for (int c1 = 0; c1 < 2; c1++)
#pragma unroll
            for (int e = 0; e < 8; e++) unpacked_stage_f16(x[c1][e], 4);

        // absmax on the packed halves (exact: a maximum of f16 values), then as in the f32 prologues.
        __half2 packed_max = __float2half2_rn(0.0f);
#pragma unroll
        for (int c1 = 0; c1 < 2; c1++)
#pragma unroll
            for (int e = 0; e < 8; e++)
                packed_max = __hmax2(packed_max, __habs2(*reinterpret_cast<const __half2 *>(&x[c1][e])));
        const float inv = row_reciprocal<kWarps>(fmaxf(__low2float(packed_max), __high2float(packed_max)), 16.0f, maxes + parity,
                                                 worker, warp, lane, q_scale + row);
        int8_t *q_row = q + row * out_stride;
#pragma unroll
        for (int c1 = 0; c1 < 2; c1++) {
            F2 v[8];
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = unpack_f16x2(x[c1][e]);
            store_codes(v, inv, q_row + 8 * layout.chunk(0, c1), q_row + 8 * layout.chunk(1, c1));
        }
    }
}

__device__ __forceinline__ void unpack_bf16(const uint4 &raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const F2 f = unpack_bf16x2(w[i]);
        v[2 * i] = f.a;
        v[2 * i + 1] = f.b;
    }
}

__device__ __forceinline__ void unpack_f16(const uint4 &raw, float (&v)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const F2 f = unpack_f16x2(w[i]);
        v[2 * i] = f.a;
        v[2 * i + 1] = f.b;
    }
}

// ---------------------------------------------------------------- launches
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

int finish_launch(const char *what, cudaError_t launched = cudaSuccess) {
    cudaError_t status = launched != cudaSuccess ? launched : cudaGetLastError();
    if (status != cudaSuccess) return fail(KREA2_RUNTIME, "%s launch failed: %s", what, cudaGetErrorString(status));
    return KREA2_OK;
}

constexpr int kMaxDevices = 64;

int current_device(int *device) {
    KREA2_CUDA(cudaGetDevice(device));
    if (*device < 0 || *device >= kMaxDevices) return fail(KREA2_INTERNAL, "device index %d out of range", *device);
    return KREA2_OK;
}

int device_sms(int device) {
    static std::atomic<int> cached[kMaxDevices];
    int n = cached[device].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        cached[device].store(n, std::memory_order_relaxed);
    }
    return n;
}

// Raises a kernel's dynamic shared-memory limit on first use per device (not a stream operation).
template <typename Kernel>
int allow_shared(Kernel kernel, int bytes, std::atomic<bool> (&done)[kMaxDevices], int device) {
    if (!done[device].load(std::memory_order_acquire)) {
        KREA2_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
        done[device].store(true, std::memory_order_release);
    }
    return KREA2_OK;
}

unsigned persistent_grid(int device, size_t tokens, int workers) {
    const size_t wanted = (tokens + workers - 1) / workers, sms = static_cast<size_t>(device_sms(device));
    return static_cast<unsigned>(wanted < sms ? wanted : sms);
}

template <int CPL>
struct LaunchNorm {
    static int run(cudaStream_t stream, size_t tokens, const void *h, const float *ns, const float *ms,
                   const float *sh, void *q, float *q_scale, size_t out_stride, float eps) {
        using G = Geometry<CPL, kWideThreads>;
        static std::atomic<bool> done[kMaxDevices];
        int device = 0;
        if (int s = current_device(&device)) return s;
        if (int s = allow_shared(prepare_norm_kernel<CPL>, NormPlan<CPL>::kBytes, done, device)) return s;
        const cudaError_t launched = launch_chain_kernel(
            prepare_norm_kernel<CPL>, dim3(persistent_grid(device, tokens, G::kWorkers)), dim3(G::kBlockThreads),
            NormPlan<CPL>::kBytes, stream, static_cast<const uint16_t *>(h), ns, ms, sh, static_cast<int8_t *>(q), q_scale,
            out_stride, eps, tokens);
        return finish_launch("prepare_norm_i8", launched);
    }
};

// The sigmoid table is filled by the first gated call on a device, on that call's stream; calls
// on other streams that overtake the fill compute the table in the kernel instead.
int ensure_sigmoid_table(cudaStream_t stream, int device) {
    static std::atomic<bool> launched[kMaxDevices];
    if (!launched[device].exchange(true, std::memory_order_acq_rel)) {
        sigmoid_table_kernel<<<256, 256, 0, stream>>>();
        if (int s = finish_launch("sigmoid table")) {
            launched[device].store(false, std::memory_order_release);
            return s;
        }
    }
    return KREA2_OK;
}

template <int CPL>
struct LaunchGated {
    static int run(cudaStream_t stream, size_t tokens, const void *attn, const void *gate, void *q,
                   float *q_scale, size_t out_stride, size_t gate_stride, size_t attn_stride) {
        using G = Geometry<CPL, kWideThreads>;
        static std::atomic<bool> done[kMaxDevices];
        int device = 0;
        if (int s = current_device(&device)) return s;
        if (int s = allow_shared(prepare_gated_kernel<CPL>, GatedPlan<CPL>::kBytes, done, device)) return s;
        if (int s = ensure_sigmoid_table(stream, device)) return s;
        const cudaError_t launched = launch_chain_kernel(
            prepare_gated_kernel<CPL>, dim3(persistent_grid(device, tokens, G::kWorkers)), dim3(G::kBlockThreads),
            GatedPlan<CPL>::kBytes, stream, static_cast<const uint16_t *>(attn), static_cast<const uint16_t *>(gate),
            static_cast<int8_t *>(q), q_scale, out_stride, gate_stride, attn_stride, tokens);
        return finish_launch("prepare_gated_i8", launched);
    }
};

template <int CPL, bool kRotated>
struct LaunchPlainAs {
    static int run(cudaStream_t stream, size_t tokens, const void *h, void *q, float *q_scale,
                   size_t out_stride) {
        using G = Geometry<CPL, kPlainThreads>;
        static std::atomic<bool> done[kMaxDevices];
        int device = 0;
        if (int s = current_device(&device)) return s;
        if (int s = allow_shared(prepare_plain_kernel<CPL, kRotated>, PlainPlan<CPL>::kBytes, done, device)) return s;
        const cudaError_t launched = launch_chain_kernel(
            prepare_plain_kernel<CPL, kRotated>, dim3(persistent_grid(device, tokens, G::kWorkers)), dim3(G::kBlockThreads),
            PlainPlan<CPL>::kBytes, stream, static_cast<const uint16_t *>(h), static_cast<int8_t *>(q), q_scale, out_stride,
            tokens);
        return finish_launch(kRotated ? "prepare_rotated_i8" : "prepare_plain_i8", launched);
    }
};
template <int CPL>
using LaunchPlain = LaunchPlainAs<CPL, false>;
template <int CPL>
using LaunchRotated = LaunchPlainAs<CPL, true>;

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

// First-use work of the gated prologue done ahead of a stream capture: the sigmoid table is filled on
// `stream` (a fill issued inside a capture would be replayed with the graph every time).
int krea2::prepare_prologue_device(cudaStream_t stream) {
    int device = 0;
    if (int s = current_device(&device)) return s;
    return ensure_sigmoid_table(stream, device);
}

// prepare_gated_i8 with a row pitch on the attention input as well (the C entry point below has
// the reference's signature, whose attention rows are dense).
int krea2::prepare_gated_pitched(cudaStream_t stream, size_t tokens, const void *attn, size_t attn_stride,
                                 const void *gate, void *q, float *q_scale, size_t width, size_t out_stride,
                                 size_t gate_stride) {
    if (int status = check_prologue("prepare_gated_i8", tokens, width, out_stride)) return status;
    KREA2_REQUIRE(gate_stride >= 256 && gate_stride <= 65536 && gate_stride % 256 == 0 && gate_stride >= width,
                  "prepare_gated_i8: gate_stride %zu must be a multiple of 256 in 256..65536 and at least the width",
                  gate_stride);
    KREA2_REQUIRE(attn_stride >= width && attn_stride % 8 == 0,
                  "prepare_gated_i8: attention pitch %zu must be a multiple of 8 and at least the width", attn_stride);
    KREA2_REQUIRE(attn && gate && q && q_scale, "prepare_gated_i8: null buffer");
    KREA2_REQUIRE(aligned16(attn) && aligned16(gate) && aligned16(q),
                  "prepare_gated_i8: buffers must be 16-byte aligned");
    return dispatch_width<LaunchGated>(width, stream, tokens, attn, gate, q, q_scale, out_stride, gate_stride,
                                       attn_stride);
}

extern "C" int krea2_prepare_gated_i8(krea2_stream stream, size_t tokens, const void *attn, const void *gate,
                                      void *q, float *q_scale, size_t width, size_t out_stride,
                                      size_t gate_stride) {
    clear_error();
    return prepare_gated_pitched(static_cast<cudaStream_t>(stream), tokens, attn, width, gate, q, q_scale, width,
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

extern "C" int krea2_prepare_rotated_i8(krea2_stream stream, size_t tokens, const void *h, void *q, float *q_scale,
                                        size_t width, size_t out_stride) {
    clear_error();
    if (int status = check_prologue("prepare_rotated_i8", tokens, width, out_stride)) return status;
    KREA2_REQUIRE(h && q && q_scale, "prepare_rotated_i8: null buffer");
    KREA2_REQUIRE(aligned16(h) && aligned16(q), "prepare_rotated_i8: buffers must be 16-byte aligned");
    return dispatch_width<LaunchRotated>(width, static_cast<cudaStream_t>(stream), tokens, h, q, q_scale, out_stride);
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
