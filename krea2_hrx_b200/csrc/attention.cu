// The three launches that sit between the q|k|v|gate GEMM and the gated prologue of a block
// (src/session/mod.rs:714-755): per-head QK-norm with rotary embedding, the V transpose, and
// grouped-query fp16 attention.  They are not W8A8 products; they complete the block so that
// a forward of the session is a real transformer block chain.
//
//   krea2_rope_qknorm_f16            kernels/rope_qknorm_f16.loom
//   krea2_v_transpose                kernels/native/v_transpose.loom
//   krea2_attention_gqa_lds_f16_wmma kernels/attention_gqa_lds_f16_wmma.loom (and the _q32 sibling,
//                                    which computes the same function on 32-row groups)
//
// Attention is a flash-attention forward on the fifth-generation tensor cores: one CTA per
// (256 query rows, query head), two softmax groups of four warps owning 128 rows each; S = Q K^T
// and O += P V are tcgen05.mma kind::f16 with f32 accumulators in tensor memory, K and V^T tiles of
// 128 keys arrive by TMA (128-byte swizzle, two stages each) and serve both groups, softmax warps
// read S from tensor memory (one query row per thread), keep the running maximum and sum in
// registers and write P back into tensor memory, where the second product reads it as its A
// operand.  O stays in tensor memory across key tiles; it is rescaled there only when a row's
// maximum moves by more than 2^8 (the reference maximum used for the exponentials is otherwise
// left stale, which changes neither O nor the sum's ratio).  The details are at the kernel.
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace krea2 {
namespace {

constexpr unsigned kFull = 0xffffffffu;

// ---------------------------------------------------------------- rope + qk norm
// One 256-thread block per token, a warp per head, four channels per lane
// (kernels/rope_qknorm_f16.loom:78-157).  The two sums the reference leaves unordered are fixed
// as ((s0+s1)+(s2+s3)) per lane and the xor butterfly 16..1 across the warp; rsqrt is 1/sqrt.
// Token-sharded launches (template flag S): this device computes rows first_row.. of the sequence and stores
// its K and V rows into EVERY device's full-length K and V tensors through peer-mapped pointers, so the
// all-gather of keys and values rides in this kernel's own stores over NVLink.  When the last block has
// finished, slot `rank` of every device's flag array receives `epoch` (+ *epoch_base).
struct RowPush {
    uint32_t world, rank, first_row, epoch;
    uint16_t *k_dest[8], *v_dest[8];
    uint32_t *flags[8];
    uint32_t *counter;
    const uint32_t *epoch_base;
};

template <bool S>
__device__ __forceinline__ void store_kv(const RowPush &push, uint16_t *const *dest, uint16_t *local, size_t at, uint2 value) {
    if constexpr (S) {
#pragma unroll
        for (int d = 0; d < 8; d++)
            if (d < static_cast<int>(push.world)) *reinterpret_cast<uint2 *>(dest[d] + at) = value;
    } else {
        *reinterpret_cast<uint2 *>(local + at) = value;
    }
}

template <bool S>
__global__ void __launch_bounds__(256)
rope_qknorm_kernel(const uint16_t *__restrict__ qkv, const float *__restrict__ q_scale,
                   const float *__restrict__ k_scale, const float *__restrict__ cos_table,
                   const float *__restrict__ sin_table, uint16_t *__restrict__ q_out, uint16_t *__restrict__ k_out,
                   uint16_t *__restrict__ v_out, uint32_t row_stride, uint32_t q_heads, uint32_t kv_heads,
                   uint32_t k_offset, float eps, const RowPush push) {
    chain_wait();
    const size_t row = blockIdx.x;
    const size_t kv_row = S ? row + push.first_row : row;  // the row of the full-length K and V tensors
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, col = lane * 4;
    const uint32_t heads_total = q_heads + 2 * kv_heads;
    const float4 cs = __ldg(reinterpret_cast<const float4 *>(cos_table + row * 128 + col));
    const float4 sn = __ldg(reinterpret_cast<const float4 *>(sin_table + row * 128 + col));
    // A warp's heads are taken three at a time with their loads issued together: one 8-byte load per lane
    // and head in flight at a time would leave the kernel waiting on memory latency.
    constexpr int kBatch = 3;
    for (uint32_t first = warp; first < heads_total; first += 8 * kBatch) {
        uint2 raws[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; b++) {
            const uint32_t head = first + 8 * b;
            if (head < heads_total) {
                const uint32_t base = head < q_heads ? head * 128 : k_offset + (head - q_heads) * 128;  // v follows k in the row
                raws[b] = *reinterpret_cast<const uint2 *>(qkv + row * row_stride + base + col);
            }
        }
#pragma unroll
        for (int b = 0; b < kBatch; b++) {
            const uint32_t head = first + 8 * b;
            if (head >= heads_total) break;
            const uint2 raw = raws[b];
            const bool is_q = head < q_heads, is_v = head >= q_heads + kv_heads;
            if (is_v) {
                store_kv<S>(push, push.v_dest, v_out, kv_row * (kv_heads * 128) + (head - q_heads - kv_heads) * 128 + col, raw);
                continue;
            }
            const __half2 lo = *reinterpret_cast<const __half2 *>(&raw.x), hi = *reinterpret_cast<const __half2 *>(&raw.y);
            const float v0 = __low2float(lo), v1 = __high2float(lo), v2 = __low2float(hi), v3 = __high2float(hi);
            float ss = __fadd_rn(__fadd_rn(__fmul_rn(v0, v0), __fmul_rn(v1, v1)), __fadd_rn(__fmul_rn(v2, v2), __fmul_rn(v3, v3)));
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(kFull, ss, off));
            const float rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss, 0.0078125f), eps)));
            const float4 sc = __ldg(reinterpret_cast<const float4 *>((is_q ? q_scale : k_scale) + col));
            // x = bf16((h * rinv) * (1 + scale)); out = bf16(x * cos + rot * sin), rot = (-x1, x0, -x3, x2)
            const float x0 = bf_round(__fmul_rn(__fmul_rn(v0, rinv), __fadd_rn(sc.x, 1.0f)));
            const float x1 = bf_round(__fmul_rn(__fmul_rn(v1, rinv), __fadd_rn(sc.y, 1.0f)));
            const float x2 = bf_round(__fmul_rn(__fmul_rn(v2, rinv), __fadd_rn(sc.z, 1.0f)));
            const float x3 = bf_round(__fmul_rn(__fmul_rn(v3, rinv), __fadd_rn(sc.w, 1.0f)));
            const float o0 = bf_round(__fadd_rn(__fmul_rn(x0, cs.x), __fmul_rn(__fsub_rn(0.0f, x1), sn.x)));
            const float o1 = bf_round(__fadd_rn(__fmul_rn(x1, cs.y), __fmul_rn(x0, sn.y)));
            const float o2 = bf_round(__fadd_rn(__fmul_rn(x2, cs.z), __fmul_rn(__fsub_rn(0.0f, x3), sn.z)));
            const float o3 = bf_round(__fadd_rn(__fmul_rn(x3, cs.w), __fmul_rn(x2, sn.w)));
            const __half2 out_lo = __floats2half2_rn(o0, o1), out_hi = __floats2half2_rn(o2, o3);
            uint2 packed;
            packed.x = *reinterpret_cast<const uint32_t *>(&out_lo);
            packed.y = *reinterpret_cast<const uint32_t *>(&out_hi);
            if (is_q)
                *reinterpret_cast<uint2 *>(q_out + row * (q_heads * 128) + head * 128 + col) = packed;
            else
                store_kv<S>(push, push.k_dest, k_out, kv_row * (kv_heads * 128) + (head - q_heads) * 128 + col, packed);
        }
    }
    if constexpr (S) {
        // Every storing thread fences at system scope; the last block to finish publishes the epoch, so
        // whoever observes the flag observes the rows.
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0 && push.counter != nullptr) {
            const uint32_t finished = atomicAdd(push.counter, 1u);
            if (finished == gridDim.x - 1) {
                *push.counter = 0;  // ready for the next launch on this stream
                const uint32_t value = push.epoch + (push.epoch_base ? *push.epoch_base : 0u);
                __threadfence_system();
#pragma unroll
                for (int d = 0; d < 8; d++)
                    if (d < static_cast<int>(push.world) && push.flags[d] != nullptr)
                        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(push.flags[d] + push.rank), "r"(value) : "memory");
            }
        }
    }
}

// Publishes an epoch in slot `rank` of every device's flag array once everything queued before it on the
// stream has finished: the fence a token-sharded forward ends with.
__global__ void shard_signal_kernel(const RowPush push) {
    if (threadIdx.x != 0) return;
    const uint32_t value = push.epoch + (push.epoch_base ? *push.epoch_base : 0u);
    __threadfence_system();
#pragma unroll
    for (int d = 0; d < 8; d++)
        if (d < static_cast<int>(push.world) && push.flags[d] != nullptr)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(push.flags[d] + push.rank), "r"(value) : "memory");
}

// ---------------------------------------------------------------- v transpose
// x [rows][width] -> out [width][capacity], 32 x 32 tiles through shared memory; columns past
// `rows` inside a tile are written as zero (kernels/native/v_transpose.loom).
__global__ void __launch_bounds__(256)
v_transpose_kernel(const uint16_t *__restrict__ x, uint16_t *__restrict__ out, uint32_t rows, uint32_t width,
                   uint32_t capacity) {
    chain_wait();
    __shared__ uint16_t tile[32][34];
    const uint32_t row0 = blockIdx.x * 32, col0 = blockIdx.y * 32;
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t r = row0 + ty + 8 * i;
        tile[ty + 8 * i][tx] = r < rows ? x[static_cast<size_t>(r) * width + col0 + tx] : uint16_t(0);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t c = col0 + ty + 8 * i, r = row0 + tx;
        if (r < capacity) out[static_cast<size_t>(c) * capacity + r] = tile[tx][ty + 8 * i];
    }
}

// ---------------------------------------------------------------- attention
// One CTA owns two query tiles of 128 rows (softmax groups A and B, four warps each) and walks the
// keys in tiles of 128.  Per group and key tile: S = Q K^T (tcgen05, f32 in tensor memory), the
// group's warps read their rows, keep a running maximum and sum, write P = 2^(S - max) as f16 back
// into the first 64 columns of the same S region, and O += P V takes P straight from tensor
// memory, so P never crosses shared memory (whose bandwidth a 128 x 128 f16 product with both
// operands in shared memory already saturates) and a K or V tile is loaded once for both groups.
// The tensor pipe runs one thread's products in issue order and a commit covers everything
// issued before it; that is what orders P V of tile j before the S of tile j + 1 that overwrites
// P, and P V of tile j - 1 before the softmax of tile j rescales O.  While one group is in its
// softmax the pipe works for the other.
constexpr int kTile = 128;            // query rows per group, keys per step, channels per head
constexpr int kSubtileBytes = 16384;  // [128 rows][64 f16]: one 128-byte swizzled column block
constexpr int kOperandBytes = 2 * kSubtileBytes;
constexpr int kAttnThreads = 352;     // warps 0-3 and 4-7: the two softmax groups; 8 Q+K loads; 9 MMA; 10 V loads
constexpr int kGroupWarps = 4;
constexpr int kTmaWarpAttn = 8, kMmaWarpAttn = 9, kTmaWarpV = 10;
constexpr int kKvStages = 2;
// Build-time choices of the softmax phase (the defaults are what measured best inside the block loop):
// KREA2_ATTN_TWO_PASS   1: the scores pass through registers in halves, once for the maximum and once for the
//                          exponentials; 0: the whole row stays in registers
// KREA2_ATTN_FMA_PAIRS  of every KREA2_ATTN_UNIT_PAIRS + KREA2_ATTN_FMA_PAIRS pairs of keys, how many take
//                          their exponentials on the FMA pipes (exp2_on_fma) instead of the exponential unit
#ifndef KREA2_ATTN_TWO_PASS
#define KREA2_ATTN_TWO_PASS 1
#endif
#ifndef KREA2_ATTN_FMA_PAIRS
#define KREA2_ATTN_FMA_PAIRS 1
#endif
#ifndef KREA2_ATTN_UNIT_PAIRS
#define KREA2_ATTN_UNIT_PAIRS 3
#endif
constexpr int kUnitPairs = KREA2_ATTN_UNIT_PAIRS, kFmaPairs = KREA2_ATTN_FMA_PAIRS;  // of every kUnitPairs + kFmaPairs pairs of keys, how many go where
constexpr uint64_t kAttnWaitLimitNs = 2000000000ull;
constexpr int kAttnSmemBytes = (2 + 2 * kKvStages) * kOperandBytes + 1024 + 1024;  // Q x2, K, V stages, barriers

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ uint64_t timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}
__device__ int g_attention_status = 0;  // folded into krea2_device_status by take_attention_status
constexpr int kAttentionTimedOut = 32;
// Bounded: after two seconds the CTA's abort flag and the device status word are raised and every
// role falls through to the end of the kernel.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = timer_ns();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (*abort_flag) return false;
            if (timer_ns() - start > kAttnWaitLimitNs) {
                *abort_flag = 1;
                atomicOr(&g_attention_status, kAttentionTimedOut);
                return false;
            }
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem] B[smem]
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] B[smem]: A is M rows (lanes) of f16 pairs, one K = 16 step per eight columns.
__device__ __forceinline__ void umma_f16_tmem_a(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_load() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_store() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Issues the load of 32 columns without waiting for it (tmem_wait_load completes all loads issued so far).
__device__ __forceinline__ void tmem_load_32_async(uint32_t address, float *r) {
    uint32_t *u = reinterpret_cast<uint32_t *>(r);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]),
          "=r"(u[9]), "=r"(u[10]), "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15]), "=r"(u[16]),
          "=r"(u[17]), "=r"(u[18]), "=r"(u[19]), "=r"(u[20]), "=r"(u[21]), "=r"(u[22]), "=r"(u[23]), "=r"(u[24]),
          "=r"(u[25]), "=r"(u[26]), "=r"(u[27]), "=r"(u[28]), "=r"(u[29]), "=r"(u[30]), "=r"(u[31])
        : "r"(address));
}
__device__ __forceinline__ void tmem_load_32(uint32_t address, float (&r)[32]) {
    tmem_load_32_async(address, r);
    tmem_wait_load();
}
// Issues the store of 32 columns (tmem_wait_store completes all stores issued so far).
__device__ __forceinline__ void tmem_store_32_async(uint32_t address, const uint32_t *u) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(address),
        "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]), "r"(u[9]),
        "r"(u[10]), "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(u[16]), "r"(u[17]), "r"(u[18]),
        "r"(u[19]), "r"(u[20]), "r"(u[21]), "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]),
        "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
        : "memory");
}
__device__ __forceinline__ void tmem_store_32(uint32_t address, const float (&r)[32]) {
    tmem_store_32_async(address, reinterpret_cast<const uint32_t *>(r));
    tmem_wait_store();
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two f32 values in one 64-bit register pair and the packed arithmetic on them (one issue slot for two lanes).
struct F2 {
    float a, b;
};
#define KREA2_ATTN_PACKED(name, op)                                                                            \
    __device__ __forceinline__ F2 name(F2 x, F2 y) {                                                           \
        F2 d;                                                                                                  \
        asm("{ .reg .b64 p, q, r;\n mov.b64 p, {%2, %3};\n mov.b64 q, {%4, %5};\n " op                        \
            ".rn.f32x2 r, p, q;\n mov.b64 {%0, %1}, r;\n }"                                                    \
            : "=f"(d.a), "=f"(d.b)                                                                             \
            : "f"(x.a), "f"(x.b), "f"(y.a), "f"(y.b));                                                         \
        return d;                                                                                              \
    }
KREA2_ATTN_PACKED(add2, "add")
KREA2_ATTN_PACKED(sub2, "sub")
#undef KREA2_ATTN_PACKED
__device__ __forceinline__ F2 fma2(F2 x, F2 y, F2 z) {
    F2 d;
    asm("{ .reg .b64 p, q, r, s;\n mov.b64 p, {%2, %3};\n mov.b64 q, {%4, %5};\n mov.b64 r, {%6, %7};\n"
        " fma.rn.f32x2 s, p, q, r;\n mov.b64 {%0, %1}, s;\n }"
        : "=f"(d.a), "=f"(d.b)
        : "f"(x.a), "f"(x.b), "f"(y.a), "f"(y.b), "f"(z.a), "f"(z.b));
    return d;
}
// 2^x for both lanes on the FMA pipes, for the share of the exponentials the exponential unit is spared:
// x = n + r with n the nearest integer (the magic-constant addition leaves it in the low mantissa bits) and
// |r| <= 1/2, 2^r by a cubic (relative error 7.5e-5, a fifth of an f16 ulp: the result is rounded to f16 next),
// and n added into the exponent field.  x is clamped at -120 so that the exponent never wraps; such
// probabilities round to zero in f16 either way.
__device__ __forceinline__ F2 exp2_on_fma(F2 x) {
    const F2 magic = {12582912.0f, 12582912.0f};  // 1.5 * 2^23
    x.a = fmaxf(x.a, -120.0f), x.b = fmaxf(x.b, -120.0f);
    const F2 t = add2(x, magic);
    const F2 r = sub2(x, sub2(t, magic));
    F2 p = fma2(F2{0.0551716685f, 0.0551716685f}, r, F2{0.2426111251f, 0.2426111251f});
    p = fma2(p, r, F2{0.6932609677f, 0.6932609677f});
    p = fma2(p, r, F2{0.9999280572f, 0.9999280572f});
    return F2{__uint_as_float(__float_as_uint(p.a) + (__float_as_uint(t.a) << 23)),
              __uint_as_float(__float_as_uint(p.b) + (__float_as_uint(t.b) << 23))};
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// K-major operand tile of 128-byte swizzled rows, eight rows per 1024-byte atom (as in the GEMM).
__device__ __forceinline__ uint64_t smem_descriptor(uint32_t address) {
    return static_cast<uint64_t>((address & 0x3ffffu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// kind::f16 with f16 operands, f32 accumulate (1 at bit 4), both K-major, N/8 at bit 17, M/16 at bit 24.
constexpr uint32_t kIdescF16 = (1u << 4) | (static_cast<uint32_t>(kTile >> 3) << 17) | (static_cast<uint32_t>(kTile >> 4) << 24);

struct AttnArgs {
    uint32_t tokens;  // keys and values
    uint32_t q_rows;  // query rows of this launch (= tokens unless the rows are sharded over devices)
    uint32_t q_heads_per_kv, out_stride;
    float scale_log2;  // softmax scale times log2(e)
    uint16_t *out;
};

// S = Q K^T: one 128 x 128 x 128 product from two 64-wide K-major subtiles per operand, 8 instructions of K = 16.
__device__ __forceinline__ void issue_scores(uint32_t tmem_d, uint32_t q_addr, uint32_t k_addr) {
#pragma unroll
    for (int sub = 0; sub < 2; sub++) {
        const uint64_t a_desc = smem_descriptor(q_addr + sub * kSubtileBytes);
        const uint64_t b_desc = smem_descriptor(k_addr + sub * kSubtileBytes);
#pragma unroll
        for (int k = 0; k < 4; k++) umma_f16(tmem_d, a_desc + 2 * k, b_desc + 2 * k, kIdescF16, (sub != 0 || k != 0) ? 1u : 0u);
    }
}
// O (+)= P V with P in tensor memory (eight columns per 16 keys) and V^T in shared memory.
__device__ __forceinline__ void issue_values(uint32_t tmem_d, uint32_t tmem_p, uint32_t v_addr, bool accumulate) {
#pragma unroll
    for (int sub = 0; sub < 2; sub++) {
        const uint64_t b_desc = smem_descriptor(v_addr + sub * kSubtileBytes);
#pragma unroll
        for (int k = 0; k < 4; k++)
            umma_f16_tmem_a(tmem_d, tmem_p + (sub * 4 + k) * 8, b_desc + 2 * k, kIdescF16, (accumulate || sub != 0 || k != 0) ? 1u : 0u);
    }
}

__global__ void __launch_bounds__(kAttnThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const AttnArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *q_smem = smem, *k_smem = smem + 2 * kOperandBytes, *v_smem = k_smem + kKvStages * kOperandBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(v_smem + kKvStages * kOperandBytes);
    uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = k_full + kKvStages, *v_full = k_empty + kKvStages;
    uint64_t *v_empty = v_full + kKvStages, *s_full = v_empty + kKvStages, *p_full = s_full + 2, *o_done = p_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_done + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q0 = blockIdx.x * 2 * kTile, head = blockIdx.y, kv_head = head / g.q_heads_per_kv;
    const uint32_t tiles = (g.tokens + kTile - 1) / kTile;
    uint32_t loads_issued = 0;  // loader threads: K (or V) tiles requested so far

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < kKvStages; s++) {
            mbar_init(k_full + s, 1);
            mbar_init(k_empty + s, 1);
            mbar_init(v_full + s, 1);
            mbar_init(v_empty + s, 1);
        }
        for (int grp = 0; grp < 2; grp++) {
            mbar_init(s_full + grp, 1);
            mbar_init(p_full + grp, kGroupWarps);
        }
        mbar_init(o_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kMmaWarpAttn) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;  // S (then P) of groups A and B at columns 0 and 128, their O at 256 and 384
    chain_wait();  // everything above touched only this CTA's shared and tensor memory

    if (warp == kTmaWarpAttn) {
        if (lane == 0) {
            mbar_expect_tx(q_full, 2 * kOperandBytes);
#pragma unroll
            for (int grp = 0; grp < 2; grp++) {
                uint8_t *dst = q_smem + grp * kOperandBytes;
                const int row = static_cast<int>(q0 + grp * kTile);
                tma_load_2d(dst, &map_q, q_full, static_cast<int>(head * kTile), row);
                tma_load_2d(dst + kSubtileBytes, &map_q, q_full, static_cast<int>(head * kTile + 64), row);
            }
            for (uint32_t j = 0; j < tiles; j++) {
                const uint32_t s = j % kKvStages, phase = (j / kKvStages) & 1u;
                const int key0 = static_cast<int>(j * kTile);
                if (!mbar_wait(k_empty + s, phase ^ 1u, abort_flag)) break;
                mbar_expect_tx(k_full + s, kOperandBytes);
                uint8_t *k_dst = k_smem + s * kOperandBytes;
                tma_load_2d(k_dst, &map_k, k_full + s, static_cast<int>(kv_head * kTile), key0);
                tma_load_2d(k_dst + kSubtileBytes, &map_k, k_full + s, static_cast<int>(kv_head * kTile + 64), key0);
                loads_issued = j + 1;
            }
        }
    } else if (warp == kTmaWarpV) {
        // V tiles have a producer of their own: a V stage frees up only after its P V products, later
        // than the K stage of the same tile, and must not hold back the next K load.
        if (lane == 0) {
            for (uint32_t j = 0; j < tiles; j++) {
                const uint32_t s = j % kKvStages, phase = (j / kKvStages) & 1u;
                const int key0 = static_cast<int>(j * kTile);
                if (!mbar_wait(v_empty + s, phase ^ 1u, abort_flag)) break;
                mbar_expect_tx(v_full + s, kOperandBytes);
                uint8_t *v_dst = v_smem + s * kOperandBytes;
                tma_load_2d(v_dst, &map_v, v_full + s, key0, static_cast<int>(kv_head * kTile));
                tma_load_2d(v_dst + kSubtileBytes, &map_v, v_full + s, key0 + 64, static_cast<int>(kv_head * kTile));
                loads_issued = j + 1;
            }
        }
    } else if (warp == kMmaWarpAttn) {
        // One thread issues both groups' products.  (One issuing thread per group was measured and is slower,
        // 0.62 ms against 0.48 ms at 4608 tokens: the pipe then interleaves the two threads' products, and each
        // group's P V and next scores complete later than when they are issued back to back.)
        if (lane == 0) {
            bool alive = mbar_wait(q_full, 0, abort_flag) && mbar_wait(k_full, 0, abort_flag);
            if (alive) {
                tc_fence_after();
#pragma unroll
                for (uint32_t grp = 0; grp < 2; grp++) {
                    issue_scores(tmem_base + grp * kTile, smem_u32(q_smem + grp * kOperandBytes), smem_u32(k_smem));
                    umma_commit(s_full + grp);
                }
                umma_commit(k_empty);
            }
            for (uint32_t j = 0; alive && j < tiles; j++) {
                const uint32_t s = j % kKvStages, phase = (j / kKvStages) & 1u;
                const uint32_t next = (j + 1) % kKvStages, next_phase = ((j + 1) / kKvStages) & 1u;
                const bool more = j + 1 < tiles;
                // The operands of this iteration (V of tile j, K of tile j + 1) were requested long ago: they are
                // waited for first, so that nothing stands between a group's P arriving and its products.
                alive = mbar_wait(v_full + s, phase, abort_flag) && (!more || mbar_wait(k_full + next, next_phase, abort_flag));
                if (!alive) break;
#pragma unroll
                for (uint32_t grp = 0; grp < 2; grp++) {
                    // P V of this tile, then the group's next scores: the pipe keeps them in this order,
                    // so the scores overwrite P only after it has been read.
                    alive = mbar_wait(p_full + grp, j & 1u, abort_flag);
                    if (!alive) break;
                    tc_fence_after();
                    issue_values(tmem_base + (2 + grp) * kTile, tmem_base + grp * kTile, smem_u32(v_smem + s * kOperandBytes), j > 0);
                    if (more) {
                        issue_scores(tmem_base + grp * kTile, smem_u32(q_smem + grp * kOperandBytes),
                                     smem_u32(k_smem + next * kOperandBytes));
                        umma_commit(s_full + grp);
                    }
                }
                if (!alive) break;
                umma_commit(v_empty + s);
                if (more) umma_commit(k_empty + next);
            }
            if (alive) umma_commit(o_done);
        }
    } else if (warp < 2 * kGroupWarps) {
        // Softmax group `grp` owns query rows q0 + 128 grp .. + 127: warp w reads TMEM lanes 32 (w % 4) .. + 31,
        // one row per thread.
        const int grp = warp >> 2, quarter = warp & 3;
        const uint32_t lane_bits = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t row_in_tile = quarter * 32 + lane;
        const uint32_t s_addr = tmem_base + grp * kTile + lane_bits, o_addr = tmem_base + (2 + grp) * kTile + lane_bits;
        float reference = -INFINITY, sum = 0.0f;  // in units of log2: scores are scaled by scale * log2(e)
        bool alive = true;
        for (uint32_t j = 0; j < tiles; j++) {
            const bool ready = mbar_wait(s_full + grp, j & 1u, abort_flag);
            if (!__all_sync(kFull, ready)) {
                alive = false;
                break;
            }
            tc_fence_after();
            const uint32_t valid = g.tokens - j * kTile;  // keys of this tile before the end of the sequence
            float part[8];  // eight running maxima, two new scores each per 3-input max
            auto mask_tail = [&](int first, int count, float *v) {
                if (valid < static_cast<uint32_t>(kTile)) {  // the last tile: keys past the sequence score -inf
#pragma unroll
                    for (int i = 0; i < count; i++)
                        if (static_cast<uint32_t>(first + i) >= valid) v[i] = -INFINITY;
                }
            };
#if KREA2_ATTN_TWO_PASS
            // Pass 1, the row maximum: the 128 scores pass through registers in two halves (they are read again
            // for the exponentials, which keeps half as many registers live as holding the row would).
            auto load_half = [&](int half, float (&v)[64]) {
                tmem_load_32_async(s_addr + half * 64, v);
                tmem_load_32_async(s_addr + half * 64 + 32, v + 32);
                tmem_wait_load();
                mask_tail(half * 64, 64, v);
            };
            {
                float v[64];
                load_half(0, v);
#pragma unroll
                for (int k = 0; k < 8; k++) part[k] = max3(v[k], v[k + 8], v[k + 16]);
#pragma unroll
                for (int i = 24; i < 56; i += 16)
#pragma unroll
                    for (int k = 0; k < 8; k++) part[k] = max3(part[k], v[i + k], v[i + 8 + k]);
#pragma unroll
                for (int k = 0; k < 8; k++) part[k] = fmaxf(part[k], v[56 + k]);
            }
            {
                float v[64];
                load_half(1, v);
#pragma unroll
                for (int i = 0; i < 64; i += 16)
#pragma unroll
                    for (int k = 0; k < 8; k++) part[k] = max3(part[k], v[i + k], v[i + 8 + k]);
            }
#else
            // The whole row of S (128 scores) comes into registers with four loads in flight at once.
            float row[kTile];
#pragma unroll
            for (int c = 0; c < 4; c++) tmem_load_32_async(s_addr + c * 32, row + c * 32);
            tmem_wait_load();
            mask_tail(0, kTile, row);
#pragma unroll
            for (int i = 0; i < 8; i++) part[i] = max3(row[i], row[i + 8], row[i + 16]);
#pragma unroll
            for (int i = 24; i < kTile - 8; i += 16)
#pragma unroll
                for (int k = 0; k < 8; k++) part[k] = max3(part[k], row[i + k], row[i + 8 + k]);
#pragma unroll
            for (int k = 0; k < 8; k++) part[k] = fmaxf(part[k], row[kTile - 8 + k]);
#endif
            float tile_max = fmaxf(max3(part[0], part[1], part[2]), max3(max3(part[3], part[4], part[5]), part[6], part[7]));
            tile_max *= g.scale_log2;
            // The exponent reference moves only when the maximum has grown by more than 2^8.
            float alpha = 1.0f;
            const bool move = tile_max > reference + 8.0f;
            if (move) {
                alpha = fast_exp2(reference - tile_max);  // 0 on the first tile
                reference = tile_max;
                sum *= alpha;
            }
            // O holds the products up to tile j - 1 (the commit behind s_full covered them): rescale it in place.
            if (j > 0 && __any_sync(kFull, move)) {
#pragma unroll 1
                for (int c = 0; c < 4; c++) {
                    float o[32];
                    tmem_load_32(o_addr + c * 32, o);
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] *= alpha;
                    tmem_store_32(o_addr + c * 32, o);
                }
            }
            // p = 2^(score - reference) as f16 pairs, back into the first 64 columns of the S region:
            // key 2c in the low half of column c, which is the A operand layout of the P V product.
            // The exponential unit does 16 lanes a clock per SM, which makes 128 x 128 exponentials the longest
            // part of this phase: of every kUnitPairs + kFmaPairs pairs of keys the first kUnitPairs go to the
            // unit and the others take the FMA pipes, in packed arithmetic (exp2_on_fma).
#if KREA2_ATTN_FMA_PAIRS == 0
            float partial[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int c = 0; c < 2; c++) {
#if KREA2_ATTN_TWO_PASS
                float v[64];
                load_half(c, v);
#else
                const float *v = row + c * 64;
#endif
                uint32_t packed[32];
#pragma unroll
                for (int i = 0; i < 64; i += 2) {
                    const float p0 = fast_exp2(fmaf(v[i], g.scale_log2, -reference));
                    const float p1 = fast_exp2(fmaf(v[i + 1], g.scale_log2, -reference));
                    partial[(i >> 1) & 3] += p0 + p1;
                    const __half2 h = __floats2half2_rn(p0, p1);
                    packed[i / 2] = *reinterpret_cast<const uint32_t *>(&h);
                }
                tmem_store_32_async(s_addr + c * 32, packed);
            }
            sum += (partial[0] + partial[1]) + (partial[2] + partial[3]);
#else
            const F2 scale2 = {g.scale_log2, g.scale_log2}, shift2 = {-reference, -reference};
            F2 partial[4] = {{0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}};
#pragma unroll
            for (int c = 0; c < 2; c++) {
                // keys 64 c .. 64 c + 63 become words 32 c .. of P; the columns a store overwrites have been read
#if KREA2_ATTN_TWO_PASS
                float v[64];
                load_half(c, v);
#else
                const float *v = row + c * 64;
#endif
                uint32_t packed[32];
#pragma unroll
                for (int i = 0; i < 64; i += 2) {
                    const F2 x = fma2(F2{v[i], v[i + 1]}, scale2, shift2);
                    F2 pr;
                    if ((i >> 1) % (kUnitPairs + kFmaPairs) < kUnitPairs) {
                        pr = F2{fast_exp2(x.a), fast_exp2(x.b)};
                    } else {
                        pr = exp2_on_fma(x);  // a masked key's -inf is clamped there and rounds to zero in f16
                    }
                    partial[(i >> 1) & 3] = add2(partial[(i >> 1) & 3], pr);
                    const __half2 h = __floats2half2_rn(pr.a, pr.b);
                    packed[i / 2] = *reinterpret_cast<const uint32_t *>(&h);
                }
                tmem_store_32_async(s_addr + c * 32, packed);
            }
            const F2 total = add2(add2(partial[0], partial[1]), add2(partial[2], partial[3]));
            sum += total.a + total.b;
#endif
            tmem_wait_store();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + grp);
        }
        const bool finished = alive && mbar_wait(o_done, 0, abort_flag);
        if (__all_sync(kFull, finished)) {
            tc_fence_after();
            const float inv = 1.0f / sum;
            const uint32_t row = q0 + grp * kTile + row_in_tile;
            uint16_t *dst = g.out + static_cast<size_t>(row) * g.out_stride + head * kTile;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                float o[32];
                tmem_load_32(o_addr + c * 32, o);
                if (row < g.q_rows) {
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int e = 8 * q + 2 * i;
                            const __half2 h = __floats2half2_rn(o[e] * inv, o[e + 1] * inv);
                            w[i] = *reinterpret_cast<const uint32_t *>(&h);
                        }
                        *reinterpret_cast<uint4 *>(dst + c * 32 + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();  // every role is done: the abort flag is final
    tc_fence_after();
    if (*abort_flag) {
        // No load may still be writing this CTA's shared memory when it exits: each loader waits (bounded) for
        // the last load it issued into every stage (Q rides on the first K wait: it was requested before it).
        const uint64_t start = timer_ns();
        if ((warp == kTmaWarpAttn || warp == kTmaWarpV) && lane == 0) {
            uint64_t *full = warp == kTmaWarpAttn ? k_full : v_full;
            if (warp == kTmaWarpAttn)
                while (!mbar_try_wait(q_full, 0))
                    if (timer_ns() - start > kAttnWaitLimitNs) break;
            for (uint32_t i = loads_issued > static_cast<uint32_t>(kKvStages) ? loads_issued - kKvStages : 0u; i < loads_issued; i++)
                while (!mbar_try_wait(full + i % kKvStages, (i / kKvStages) & 1u))
                    if (timer_ns() - start > kAttnWaitLimitNs) break;
        }
        __syncthreads();
    }
    if (warp == kMmaWarpAttn) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ---------------------------------------------------------------- attention, one query tile per CTA
// The second form of the kernel: bit-identical to the two-tile form and, with the SMs full for several rounds,
// about 9 % slower, because four softmax warps -- one per scheduler -- cannot keep the exponential unit and the
// issue slots as busy as eight do.  Its CTAs are half as long, so the launcher takes it where that saves rounds
// over the SMs (few query rows); KREA2_ATTENTION_FORM=0 / 1 forces a form.
// A CTA owns ONE query tile of 128 rows and gives it everything the first form splits between two tiles.  Tensor memory (512 columns): S twice (2 x 128), O (128), P (64), Q (64).
//  - Q sits in tensor memory (f16 pairs, the A-operand layout), so S = Q K^T reads only K from shared memory;
//  - S is double-buffered and P has columns of its own, which breaks the chain S -> softmax -> P V -> next S of
//    the two-tile form: the scores of tile j + 1 are computed while the softmax works on tile j, and P V of
//    tile j runs under the softmax of tile j + 1.  The softmax warps never wait for the tensor pipe as long as
//    two products take less time than one softmax.
// Four softmax warps (one row per thread, the whole row of scores in registers: with 256 threads per CTA the
// register file allows it), a K loader, a V loader, and TWO issuing threads, one for the score products and
// one for P V: the two streams of products do not depend on each other except through the barriers, and each
// round of waits and commits costs an issuing thread several hundred cycles during which a single issuer
// would leave the tensor pipe idle.  Three K and V stages.
constexpr int kSingleThreads = 256;  // warps 0-3 softmax, 4 K loads, 5 issues the score products, 6 V loads, 7 issues P V
constexpr int kSingleKWarp = 4, kSingleMmaWarp = 5, kSingleVWarp = 6, kSingleValuesWarp = 7;
constexpr int kSingleStages = 3;
constexpr int kSingleSmemBytes = 2 * kSingleStages * kOperandBytes + 1024 + 1024;
constexpr uint32_t kColS = 0, kColO = 256, kColP = 384, kColQ = 448;

// S (+)= Q K^T with Q in tensor memory: eight K = 16 steps, eight columns of Q each.
__device__ __forceinline__ void issue_scores_tmem_q(uint32_t tmem_d, uint32_t tmem_q, uint32_t k_addr) {
#pragma unroll
    for (int sub = 0; sub < 2; sub++) {
        const uint64_t b_desc = smem_descriptor(k_addr + sub * kSubtileBytes);
#pragma unroll
        for (int k = 0; k < 4; k++)
            umma_f16_tmem_a(tmem_d, tmem_q + (sub * 4 + k) * 8, b_desc + 2 * k, kIdescF16, (sub != 0 || k != 0) ? 1u : 0u);
    }
}

__global__ void __launch_bounds__(kSingleThreads, 1)
attention_single_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const uint16_t *__restrict__ q, uint32_t q_stride, const AttnArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *k_smem = smem, *v_smem = smem + kSingleStages * kOperandBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(v_smem + kSingleStages * kOperandBytes);
    uint64_t *k_full = bars, *k_empty = k_full + kSingleStages, *v_full = k_empty + kSingleStages, *v_empty = v_full + kSingleStages;
    uint64_t *s_full = v_empty + kSingleStages;  // [2] the scores of a tile are in buffer b
    uint64_t *s_free = s_full + 2;               // [2] the softmax has read buffer b into registers
    uint64_t *p_full = s_free + 2;               // P of a tile is written (and O rescaled where needed)
    uint64_t *p_free = p_full + 1;               // P V of a tile has completed: P may be rewritten, O holds the tile
    uint64_t *q_ready = p_free + 1, *o_done = q_ready + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(o_done + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t q0 = blockIdx.x * kTile, head = blockIdx.y, kv_head = head / g.q_heads_per_kv;
    const uint32_t tiles = (g.tokens + kTile - 1) / kTile;
    uint32_t k_issued = 0, v_issued = 0;  // loader threads: tiles requested so far

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSingleStages; s++) {
            mbar_init(k_full + s, 1);
            mbar_init(k_empty + s, 1);
            mbar_init(v_full + s, 1);
            mbar_init(v_empty + s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(s_full + b, 1);
            mbar_init(s_free + b, kGroupWarps);
        }
        mbar_init(p_full, kGroupWarps);
        mbar_init(p_free, 1);
        mbar_init(q_ready, kGroupWarps);
        mbar_init(o_done, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kSingleMmaWarp) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    chain_wait();  // everything above touched only this CTA's shared and tensor memory

    if (warp == kSingleKWarp) {
        if (lane == 0) {
            for (uint32_t j = 0; j < tiles; j++) {
                const uint32_t s = j % kSingleStages, phase = (j / kSingleStages) & 1u;
                if (!mbar_wait(k_empty + s, phase ^ 1u, abort_flag)) break;
                mbar_expect_tx(k_full + s, kOperandBytes);
                uint8_t *dst = k_smem + s * kOperandBytes;
                tma_load_2d(dst, &map_k, k_full + s, static_cast<int>(kv_head * kTile), static_cast<int>(j * kTile));
                tma_load_2d(dst + kSubtileBytes, &map_k, k_full + s, static_cast<int>(kv_head * kTile + 64), static_cast<int>(j * kTile));
                k_issued = j + 1;
            }
        }
    } else if (warp == kSingleVWarp) {
        if (lane == 0) {
            for (uint32_t j = 0; j < tiles; j++) {
                const uint32_t s = j % kSingleStages, phase = (j / kSingleStages) & 1u;
                if (!mbar_wait(v_empty + s, phase ^ 1u, abort_flag)) break;
                mbar_expect_tx(v_full + s, kOperandBytes);
                uint8_t *dst = v_smem + s * kOperandBytes;
                tma_load_2d(dst, &map_v, v_full + s, static_cast<int>(j * kTile), static_cast<int>(kv_head * kTile));
                tma_load_2d(dst + kSubtileBytes, &map_v, v_full + s, static_cast<int>(j * kTile + 64), static_cast<int>(kv_head * kTile));
                v_issued = j + 1;
            }
        }
    } else if (warp == kSingleMmaWarp) {
        if (lane == 0) {
            bool alive = mbar_wait(q_ready, 0, abort_flag) && mbar_wait(k_full, 0, abort_flag);
            if (alive) {
                tc_fence_after();
                issue_scores_tmem_q(tmem_base + kColS, tmem_base + kColQ, smem_u32(k_smem));
                umma_commit(s_full);
                umma_commit(k_empty);
            }
            for (uint32_t n = 1; alive && n < tiles; n++) {
                // The scores of tile n, into the buffer whose previous scores (tile n - 2) the softmax has taken
                // into registers: issued as soon as that is so, ready long before the softmax of tile n - 1 ends.
                const uint32_t s = n % kSingleStages, b = n & 1u;
                alive = mbar_wait(k_full + s, (n / kSingleStages) & 1u, abort_flag) &&
                        (n < 2 || mbar_wait(s_free + b, ((n - 2) >> 1) & 1u, abort_flag));
                if (!alive) break;
                tc_fence_after();
                issue_scores_tmem_q(tmem_base + kColS + b * kTile, tmem_base + kColQ, smem_u32(k_smem + s * kOperandBytes));
                umma_commit(s_full + b);
                umma_commit(k_empty + s);
            }
        }
    } else if (warp == kSingleValuesWarp) {
        if (lane == 0) {
            bool alive = true;
            for (uint32_t j = 0; alive && j < tiles; j++) {
                const uint32_t s = j % kSingleStages;
                alive = mbar_wait(v_full + s, (j / kSingleStages) & 1u, abort_flag) && mbar_wait(p_full, j & 1u, abort_flag);
                if (!alive) break;
                tc_fence_after();
                issue_values(tmem_base + kColO, tmem_base + kColP, smem_u32(v_smem + s * kOperandBytes), j > 0);
                umma_commit(p_free);
                umma_commit(v_empty + s);
            }
            if (alive) umma_commit(o_done);
        }
    } else if (warp < kGroupWarps) {
        const uint32_t lane_bits = static_cast<uint32_t>(warp * 32) << 16;
        const uint32_t row = q0 + warp * 32 + lane;
        const uint32_t o_addr = tmem_base + kColO + lane_bits, p_addr = tmem_base + kColP + lane_bits;
        // Q of this row into tensor memory: its 128 channels are 64 f16x2 words, channel 2c in the low half of
        // column c, the layout an A operand in tensor memory has.
        {
            uint32_t words[64];
            const uint4 *src = reinterpret_cast<const uint4 *>(q + static_cast<size_t>(row) * q_stride + head * kTile);
#pragma unroll
            for (int i = 0; i < 16; i++) {
                uint4 v4 = make_uint4(0u, 0u, 0u, 0u);
                if (row < g.q_rows) v4 = __ldg(src + i);
                words[4 * i] = v4.x, words[4 * i + 1] = v4.y, words[4 * i + 2] = v4.z, words[4 * i + 3] = v4.w;
            }
            tmem_store_32_async(tmem_base + kColQ + lane_bits, words);
            tmem_store_32_async(tmem_base + kColQ + 32 + lane_bits, words + 32);
            tmem_wait_store();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(q_ready);
        }
        float reference = -INFINITY, sum = 0.0f;  // in units of log2: scores are scaled by scale * log2(e)
        bool alive = true;
        for (uint32_t j = 0; j < tiles; j++) {
            const uint32_t b = j & 1u;
            const bool ready = mbar_wait(s_full + b, (j >> 1) & 1u, abort_flag);
            if (!__all_sync(kFull, ready)) {
                alive = false;
                break;
            }
            tc_fence_after();
            const uint32_t s_addr = tmem_base + kColS + b * kTile + lane_bits;
            const uint32_t valid = g.tokens - j * kTile;  // keys of this tile before the end of the sequence
            float v[kTile];
#pragma unroll
            for (int c = 0; c < 4; c++) tmem_load_32_async(s_addr + c * 32, v + c * 32);
            tmem_wait_load();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(s_free + b);  // the buffer may take the scores of tile j + 2
            if (valid < static_cast<uint32_t>(kTile)) {  // the last tile: keys past the sequence score -inf
#pragma unroll
                for (int i = 0; i < kTile; i++)
                    if (static_cast<uint32_t>(i) >= valid) v[i] = -INFINITY;
            }
            float part[8];
#pragma unroll
            for (int i = 0; i < 8; i++) part[i] = max3(v[i], v[i + 8], v[i + 16]);
#pragma unroll
            for (int i = 24; i < kTile - 8; i += 16)
#pragma unroll
                for (int k = 0; k < 8; k++) part[k] = max3(part[k], v[i + k], v[i + 8 + k]);
#pragma unroll
            for (int k = 0; k < 8; k++) part[k] = fmaxf(part[k], v[kTile - 8 + k]);
            float tile_max = fmaxf(max3(part[0], part[1], part[2]), max3(max3(part[3], part[4], part[5]), part[6], part[7]));
            tile_max *= g.scale_log2;
            // The exponent reference moves only when the maximum has grown by more than 2^8.
            float alpha = 1.0f;
            const bool move = tile_max > reference + 8.0f;
            if (move) {
                alpha = fast_exp2(reference - tile_max);  // 0 on the first tile
                reference = tile_max;
                sum *= alpha;
            }
            const F2 scale2 = {g.scale_log2, g.scale_log2}, shift2 = {-reference, -reference};
            F2 partial[4] = {{0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}, {0.0f, 0.0f}};
            uint32_t packed[64];
#pragma unroll
            for (int i = 0; i < kTile; i += 2) {
                const F2 x = fma2(F2{v[i], v[i + 1]}, scale2, shift2);
                F2 pr;
                if ((i >> 1) % (kUnitPairs + kFmaPairs) < kUnitPairs) {
                    pr = F2{fast_exp2(x.a), fast_exp2(x.b)};
                } else {
                    pr = exp2_on_fma(x);
                }
                partial[(i >> 1) & 3] = add2(partial[(i >> 1) & 3], pr);
                const __half2 h = __floats2half2_rn(pr.a, pr.b);
                packed[i / 2] = *reinterpret_cast<const uint32_t *>(&h);
            }
            const F2 total = add2(add2(partial[0], partial[1]), add2(partial[2], partial[3]));
            sum += total.a + total.b;
            // P V of tile j - 1 must have completed before P is rewritten, and before O (which then holds the
            // tiles up to j - 1) is rescaled.  It was issued a whole softmax ago.
            if (j > 0) {
                const bool done = mbar_wait(p_free, (j - 1) & 1u, abort_flag);
                if (!__all_sync(kFull, done)) {
                    alive = false;
                    break;
                }
                tc_fence_after();
                if (__any_sync(kFull, move)) {
#pragma unroll 1
                    for (int c = 0; c < 4; c++) {
                        float o[32];
                        tmem_load_32(o_addr + c * 32, o);
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] *= alpha;
                        tmem_store_32(o_addr + c * 32, o);
                    }
                }
            }
            tmem_store_32_async(p_addr, packed);
            tmem_store_32_async(p_addr + 32, packed + 32);
            tmem_wait_store();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
        }
        const bool finished = alive && mbar_wait(o_done, 0, abort_flag);
        if (__all_sync(kFull, finished)) {
            tc_fence_after();
            const float inv = 1.0f / sum;
            uint16_t *dst = g.out + static_cast<size_t>(row) * g.out_stride + head * kTile;
#pragma unroll 1
            for (int c = 0; c < 4; c++) {
                float o[32];
                tmem_load_32(o_addr + c * 32, o);
                if (row < g.q_rows) {
#pragma unroll
                    for (int qd = 0; qd < 4; qd++) {
                        uint32_t w[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int e = 8 * qd + 2 * i;
                            const __half2 h = __floats2half2_rn(o[e] * inv, o[e + 1] * inv);
                            w[i] = *reinterpret_cast<const uint32_t *>(&h);
                        }
                        *reinterpret_cast<uint4 *>(dst + c * 32 + qd * 8) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();  // every role is done: the abort flag is final
    tc_fence_after();
    if (*abort_flag) {
        // No load may still be writing this CTA's shared memory when it exits: each loader waits (bounded) for
        // the last load it issued into every stage.
        const uint64_t start = timer_ns();
        if ((warp == kSingleKWarp || warp == kSingleVWarp) && lane == 0) {
            const uint32_t issued = warp == kSingleKWarp ? k_issued : v_issued;
            uint64_t *full = warp == kSingleKWarp ? k_full : v_full;
            for (uint32_t i = issued > static_cast<uint32_t>(kSingleStages) ? issued - kSingleStages : 0u; i < issued; i++)
                while (!mbar_try_wait(full + i % kSingleStages, (i / kSingleStages) & 1u))
                    if (timer_ns() - start > kAttnWaitLimitNs) break;
        }
        __syncthreads();
    }
    if (warp == kSingleMmaWarp) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

using EncodeTiled = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

// f16 [rows][pitch] as a 2-D tensor (inner x rows) with boxes of 64 x 128 elements, 128-byte swizzle.
int make_f16_map(CUtensorMap *map, const void *base, size_t inner, size_t rows, size_t pitch) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return fail(KREA2_RUNTIME, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {pitch * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t element_strides[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), dims, strides, box, element_strides,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KREA2_RUNTIME, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
    return KREA2_OK;
}

int launch_check(const char *what, cudaError_t launched = cudaSuccess) {
    cudaError_t status = launched != cudaSuccess ? launched : cudaGetLastError();
    if (status != cudaSuccess) return fail(KREA2_RUNTIME, "%s launch failed: %s", what, cudaGetErrorString(status));
    return KREA2_OK;
}

int ensure_attention() {
    static std::once_flag once[64];
    static cudaError_t attr_status[64];
    int device = 0;
    KREA2_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(KREA2_INTERNAL, "device index %d out of range", device);
    std::call_once(once[device], [&] {
        attr_status[device] =
            cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmemBytes);
        if (attr_status[device] == cudaSuccess)
            attr_status[device] = cudaFuncSetAttribute(attention_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                       kSingleSmemBytes);
    });
    if (attr_status[device] != cudaSuccess)
        return fail(KREA2_RUNTIME, "cannot reserve %d bytes of shared memory: %s", kAttnSmemBytes,
                    cudaGetErrorString(attr_status[device]));
    return encode_tiled() ? KREA2_OK : fail(KREA2_RUNTIME, "cuTensorMapEncodeTiled is not available from this driver");
}

}  // namespace

int prepare_attention_device() { return ensure_attention(); }

// Reads and clears the attention kernel's status word (the device is already synchronised).
int take_attention_status(int *value) {
    KREA2_CUDA(cudaMemcpyFromSymbol(value, g_attention_status, sizeof(int)));
    if (*value != 0) {
        int zero = 0;
        KREA2_CUDA(cudaMemcpyToSymbol(g_attention_status, &zero, sizeof(int)));
    }
    return KREA2_OK;
}

}  // namespace krea2

using namespace krea2;

extern "C" int krea2_rope_qknorm_f16(krea2_stream stream, size_t tokens, const void *qkv, const float *q_scale,
                                     const float *k_scale, const float *cos_table, const float *sin_table, void *q_out,
                                     void *k_out, void *v_out, size_t row_stride, size_t q_heads, size_t kv_heads,
                                     size_t k_offset, float eps) {
    clear_error();
    KREA2_REQUIRE(tokens >= 1 && tokens <= 1048576, "rope_qknorm_f16: tokens %zu outside 1..1048576", tokens);
    KREA2_REQUIRE(row_stride >= 128 && row_stride <= 65536 && row_stride % 128 == 0,
                  "rope_qknorm_f16: row_stride %zu must be a multiple of 128 up to 65536", row_stride);
    KREA2_REQUIRE(q_heads >= 1 && q_heads <= 256 && kv_heads >= 1 && kv_heads <= 256, "rope_qknorm_f16: heads outside 1..256");
    KREA2_REQUIRE(k_offset >= 128 && k_offset % 128 == 0 && k_offset >= q_heads * 128 &&
                      k_offset + 2 * kv_heads * 128 <= row_stride,
                  "rope_qknorm_f16: k_offset %zu must be a multiple of 128 past the q heads with k and v inside the row",
                  k_offset);
    KREA2_REQUIRE(qkv && q_scale && k_scale && cos_table && sin_table && q_out && k_out && v_out, "rope_qknorm_f16: null buffer");
    KREA2_REQUIRE(aligned16(qkv) && aligned16(q_scale) && aligned16(k_scale) && aligned16(cos_table) && aligned16(sin_table) &&
                      aligned16(q_out) && aligned16(k_out) && aligned16(v_out),
                  "rope_qknorm_f16: buffers must be 16-byte aligned");
    const cudaError_t launched = launch_chain_kernel(
        rope_qknorm_kernel<false>, dim3(static_cast<unsigned>(tokens)), dim3(256), 0, static_cast<cudaStream_t>(stream),
        static_cast<const uint16_t *>(qkv), q_scale, k_scale, cos_table, sin_table, static_cast<uint16_t *>(q_out),
        static_cast<uint16_t *>(k_out), static_cast<uint16_t *>(v_out), static_cast<uint32_t>(row_stride),
        static_cast<uint32_t>(q_heads), static_cast<uint32_t>(kv_heads), static_cast<uint32_t>(k_offset), eps, RowPush{});
    return launch_check("rope_qknorm_f16", launched);
}

namespace {
int fill_push(const char *name, const krea2_row_shard *shard, bool with_rows, RowPush *push) {
    KREA2_REQUIRE(shard, "%s: shard description is null", name);
    KREA2_REQUIRE(shard->world >= 1 && shard->world <= 8 && shard->rank < shard->world, "%s: world %u / rank %u outside 1..8",
                  name, shard->world, shard->rank);
    KREA2_REQUIRE(shard->first_row <= 0xffffffffull, "%s: first_row too large", name);
    *push = RowPush{};
    push->world = shard->world, push->rank = shard->rank, push->first_row = static_cast<uint32_t>(shard->first_row);
    push->epoch = shard->epoch, push->counter = shard->counter, push->epoch_base = shard->epoch_base;
    bool any_flag = false;
    for (uint32_t d = 0; d < shard->world; d++) {
        if (with_rows)
            KREA2_REQUIRE(shard->k_dest[d] && shard->v_dest[d] && aligned16(shard->k_dest[d]) && aligned16(shard->v_dest[d]),
                          "%s: destination %u is null or unaligned", name, d);
        push->k_dest[d] = static_cast<uint16_t *>(shard->k_dest[d]);
        push->v_dest[d] = static_cast<uint16_t *>(shard->v_dest[d]);
        push->flags[d] = shard->flags[d];
        any_flag = any_flag || shard->flags[d] != nullptr;
    }
    KREA2_REQUIRE(!with_rows || !any_flag || shard->counter, "%s: flags need the launch counter", name);
    return KREA2_OK;
}
}  // namespace

extern "C" int krea2_rope_qknorm_f16_sharded(krea2_stream stream, size_t tokens, const void *qkv, const float *q_scale,
                                             const float *k_scale, const float *cos_table, const float *sin_table,
                                             void *q_out, size_t row_stride, size_t q_heads, size_t kv_heads,
                                             size_t k_offset, float eps, const krea2_row_shard *shard) {
    clear_error();
    KREA2_REQUIRE(tokens >= 1 && tokens <= 1048576, "rope_qknorm_f16_sharded: tokens %zu outside 1..1048576", tokens);
    KREA2_REQUIRE(row_stride >= 128 && row_stride <= 65536 && row_stride % 128 == 0,
                  "rope_qknorm_f16_sharded: row_stride %zu must be a multiple of 128 up to 65536", row_stride);
    KREA2_REQUIRE(q_heads >= 1 && q_heads <= 256 && kv_heads >= 1 && kv_heads <= 256,
                  "rope_qknorm_f16_sharded: heads outside 1..256");
    KREA2_REQUIRE(k_offset >= 128 && k_offset % 128 == 0 && k_offset >= q_heads * 128 &&
                      k_offset + 2 * kv_heads * 128 <= row_stride,
                  "rope_qknorm_f16_sharded: k_offset %zu must be a multiple of 128 past the q heads with k and v inside the row",
                  k_offset);
    KREA2_REQUIRE(qkv && q_scale && k_scale && cos_table && sin_table && q_out, "rope_qknorm_f16_sharded: null buffer");
    KREA2_REQUIRE(aligned16(qkv) && aligned16(q_scale) && aligned16(k_scale) && aligned16(cos_table) && aligned16(sin_table) &&
                      aligned16(q_out),
                  "rope_qknorm_f16_sharded: buffers must be 16-byte aligned");
    RowPush push;
    if (int status = fill_push("rope_qknorm_f16_sharded", shard, true, &push)) return status;
    rope_qknorm_kernel<true><<<static_cast<unsigned>(tokens), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t *>(qkv), q_scale, k_scale, cos_table, sin_table, static_cast<uint16_t *>(q_out), nullptr,
        nullptr, static_cast<uint32_t>(row_stride), static_cast<uint32_t>(q_heads), static_cast<uint32_t>(kv_heads),
        static_cast<uint32_t>(k_offset), eps, push);
    return launch_check("rope_qknorm_f16_sharded");
}

extern "C" int krea2_shard_signal(krea2_stream stream, const krea2_row_shard *shard) {
    clear_error();
    RowPush push;
    if (int status = fill_push("shard_signal", shard, false, &push)) return status;
    shard_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(push);
    return launch_check("shard_signal");
}

extern "C" int krea2_v_transpose(krea2_stream stream, size_t rows, const void *x, void *out, size_t width,
                                 size_t row_capacity) {
    clear_error();
    KREA2_REQUIRE(width >= 32 && width <= 65536 && width % 32 == 0, "v_transpose: width %zu must be a multiple of 32", width);
    KREA2_REQUIRE(row_capacity >= 32 && row_capacity <= 1048576 && row_capacity % 32 == 0,
                  "v_transpose: row_capacity %zu must be a multiple of 32", row_capacity);
    KREA2_REQUIRE(rows >= 1 && rows <= row_capacity, "v_transpose: rows %zu outside 1..row_capacity", rows);
    KREA2_REQUIRE(x && out, "v_transpose: null buffer");
    dim3 grid(static_cast<unsigned>((rows + 31) / 32), static_cast<unsigned>(width / 32), 1);
    const cudaError_t launched = launch_chain_kernel(
        v_transpose_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const uint16_t *>(x),
        static_cast<uint16_t *>(out), static_cast<uint32_t>(rows), static_cast<uint32_t>(width),
        static_cast<uint32_t>(row_capacity));
    return launch_check("v_transpose", launched);
}

extern "C" int krea2_attention_gqa_f16_rows(krea2_stream stream, size_t q_rows, size_t tokens, size_t kv_heads, const void *q,
                                            const void *k, const void *v_transposed, void *out, size_t q_stride,
                                            size_t kv_stride, size_t out_stride, size_t token_capacity, float scale) {
    clear_error();
    KREA2_REQUIRE(tokens >= 16 && tokens <= 65536, "attention: tokens %zu outside 16..65536", tokens);
    KREA2_REQUIRE(q_rows >= 1 && q_rows <= tokens, "attention: q_rows %zu outside 1..tokens", q_rows);
    KREA2_REQUIRE(q_stride >= 128 && q_stride <= 32768 && q_stride % 128 == 0 && kv_stride >= 128 && kv_stride <= 32768 &&
                      kv_stride % 128 == 0 && out_stride >= 128 && out_stride <= 32768 && out_stride % 128 == 0,
                  "attention: strides must be multiples of 128 up to 32768");
    KREA2_REQUIRE(kv_heads >= 1 && kv_heads * 128 == kv_stride, "attention: kv_heads %zu does not match kv_stride %zu", kv_heads,
                  kv_stride);
    KREA2_REQUIRE(q_stride % kv_stride == 0 && out_stride == q_stride,
                  "attention: q heads must be a whole multiple of kv heads and out_stride must equal q_stride");
    KREA2_REQUIRE(token_capacity >= 32 && token_capacity <= 1048576 && token_capacity % 16 == 0 && token_capacity >= tokens,
                  "attention: token_capacity %zu must be a multiple of 16 and at least tokens", token_capacity);
    KREA2_REQUIRE(scale == scale && scale > 0.0f, "attention: scale must be positive");
    KREA2_REQUIRE(q && k && v_transposed && out && aligned16(q) && aligned16(k) && aligned16(v_transposed) && aligned16(out),
                  "attention: buffers must be non-null and 16-byte aligned");
    if (int status = ensure_attention()) return status;
    CUtensorMap map_q, map_k, map_v;
    if (int status = make_f16_map(&map_q, q, q_stride, q_rows, q_stride)) return status;
    if (int status = make_f16_map(&map_k, k, kv_stride, tokens, kv_stride)) return status;
    if (int status = make_f16_map(&map_v, v_transposed, token_capacity, kv_stride, token_capacity)) return status;
    AttnArgs args;
    args.tokens = static_cast<uint32_t>(tokens);
    args.q_rows = static_cast<uint32_t>(q_rows);
    args.q_heads_per_kv = static_cast<uint32_t>(q_stride / kv_stride);
    args.out_stride = static_cast<uint32_t>(out_stride);
    args.scale_log2 = scale * 1.4426950408889634f;
    args.out = static_cast<uint16_t *>(out);
    // Two forms of the kernel give the same bits (same products, same softmax, same order).  With two query tiles
    // per CTA a launch is shorter when the SMs are full for several rounds (measured at 4608 tokens: 0.477 ms
    // against 0.518 ms, 0.534 J against 0.581 J); with one tile per CTA the CTAs are half as long, which wins when
    // that saves rounds over the SMs -- few query rows, e.g. a device's share of a token-sharded sequence
    // (1152 rows of 4608, 48 heads: 3 half-length rounds instead of 2 full ones, 0.135 ms against 0.163 ms).
    // KREA2_ATTENTION_FORM=0 / 1 forces the two-tile / one-tile form.
    static const int forced_form = [] {
        const char *v = getenv("KREA2_ATTENTION_FORM");
        return v && (v[0] == '0' || v[0] == '1') ? v[0] - '0' : -1;
    }();
    bool single_tile = forced_form == 1;
    if (forced_form < 0) {
        static int sm_counts[64] = {};  // per device, read once (benign race: every writer stores the same value)
        int device = 0, sms = 0;
        if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < 64) {
            sms = sm_counts[device];
            if (sms == 0 && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess)
                sm_counts[device] = sms;
        }
        if (sms > 0) {
            const size_t heads = q_stride / 128;
            const size_t pair_rounds = ((q_rows + 2 * kTile - 1) / (2 * kTile) * heads + sms - 1) / sms;
            const size_t tile_rounds = ((q_rows + kTile - 1) / kTile * heads + sms - 1) / sms;
            single_tile = tile_rounds * 543 < pair_rounds * 970;  // a one-tile CTA takes 0.543 of a two-tile CTA's time
        }
    }
    if (single_tile) {
        dim3 grid(static_cast<unsigned>((q_rows + kTile - 1) / kTile), static_cast<unsigned>(q_stride / 128), 1);
        const cudaError_t launched =
            launch_chain_kernel(attention_single_kernel, grid, dim3(kSingleThreads), kSingleSmemBytes, static_cast<cudaStream_t>(stream),
                                map_k, map_v, static_cast<const uint16_t *>(q), static_cast<uint32_t>(q_stride), args);
        return launch_check("attention", launched);
    }
    dim3 grid(static_cast<unsigned>((q_rows + 2 * kTile - 1) / (2 * kTile)), static_cast<unsigned>(q_stride / 128), 1);
    const cudaError_t launched = launch_chain_kernel(attention_kernel, grid, dim3(kAttnThreads), kAttnSmemBytes,
                                                     static_cast<cudaStream_t>(stream), map_q, map_k, map_v, args);
    return launch_check("attention", launched);
}

extern "C" int krea2_attention_gqa_lds_f16_wmma(krea2_stream stream, size_t tokens, size_t kv_heads, const void *q,
                                                const void *k, const void *v_transposed, void *out, size_t q_stride,
                                                size_t kv_stride, size_t out_stride, size_t token_capacity, float scale) {
    return krea2_attention_gqa_f16_rows(stream, tokens, tokens, kv_heads, q, k, v_transposed, out, q_stride, kv_stride,
                                        out_stride, token_capacity, scale);
}

extern "C" int krea2_attention_gqa_lds_f16_wmma_q32(krea2_stream stream, size_t tokens, size_t kv_heads, const void *q,
                                                    const void *k, const void *v_transposed, void *out, size_t q_stride,
                                                    size_t kv_stride, size_t out_stride, size_t token_capacity,
                                                    float scale) {
    return krea2_attention_gqa_lds_f16_wmma(stream, tokens, kv_heads, q, k, v_transposed, out, q_stride, kv_stride, out_stride,
                                            token_capacity, scale);
}
