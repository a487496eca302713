// The W8A8 GEMM family of krea2-hrx for sm_100a:
//   krea2_gemm_i8_256, krea2_gemm_i8_resid_256, krea2_gemm_i8_resid_256x256,
//   krea2_gemm_i8_swiglu_256  (kernels/gemm_i8_*.loom), plus the raw-accumulator variant.
//
// One persistent, warp-specialised kernel, templated on the epilogue and the N tile:
//   warp 8      TMA producer: int8 A [128 x 128B] and W [BN x 128B] tiles, 128-byte swizzle,
//               into a ring of shared-memory stages, completion on mbarriers
//   warp 9      one thread issues tcgen05.mma kind::i8 (128 x BN x 32 per instruction),
//               accumulating i32 in tensor memory; tcgen05.commit frees the stage
//   warps 0-7   epilogue: tcgen05.ld of the 128 x BN accumulator (one row per thread),
//               i32 -> f32, weight-channel and token scales, the bf16 rounding points of
//               the reference and the residual / SwiGLU / plain store
// Two accumulators alternate in tensor memory, so the epilogue of one tile runs under the
// main loop of the next.  The default variant for N a multiple of 256 pairs two CTAs in a cluster
// on one 256 x 256 tile (tcgen05.mma.cta_group::2, each CTA loading its own halves of A and W);
// no load is multicast.
//
// Every wait on an mbarrier is bounded in time; a wait that runs out raises a CTA-wide
// abort flag and a device status word, the roles fall through to the common teardown, the
// producer drains its loads in flight, tensor memory is released and the kernel returns.
#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace krea2 {

__device__ int g_device_status = 0;

namespace {

constexpr int kBlockM = 128;        // accumulator rows = TMEM lanes
constexpr int kBlockK = 128;        // bytes of K per stage = one 128-byte swizzle row
constexpr int kUmmaK = 32;          // K of one kind::i8 instruction
constexpr int kEpilogueWarps = 8;   // two warps per 32-lane quarter of tensor memory, alternating column chunks
constexpr int kProducerWarp = kEpilogueWarps;
constexpr int kMmaWarp = kEpilogueWarps + 1;
constexpr int kGemmThreads = (kEpilogueWarps + 2) * 32;
constexpr int kStagingBytes = 4096;  // per epilogue warp: 32 rows x 128 bytes of output on their way out
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // every wait gives up after two seconds

enum class Epi { Plain, Resid, Swiglu, Acc, SwigluRot, PlainRope };

enum StatusBits { kProducerTimedOut = 1, kMmaTimedOut = 2, kEpilogueTimedOut = 4, kDrainTimedOut = 8, kShardWaitTimedOut = 16 };

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
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
// Waits for the phase of `parity` to complete.  Returns false when the CTA is aborting or
// when the wait ran out of time (in which case it raises the abort flag and `bit`).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int bit) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = global_timer_ns();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 63u) == 0u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - start > kWaitLimitNs) {
                *abort_flag = 1;
                atomicOr(&g_device_status, bit);
                return false;
            }
        }
    }
}
// Accounts for `bytes` of a transaction that will never arrive (teardown only).
__device__ __forceinline__ void mbar_complete_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.complete_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Teardown after an abort: waits (bounded) for the given phase of a stage's `full` barrier, i.e. until the
// loads armed on it have landed; a wait that runs out is recorded in the status word.
__device__ __forceinline__ void drain_stage(uint64_t *bar, uint32_t parity, uint64_t start) {
    while (!mbar_try_wait(bar, parity)) {
        if (global_timer_ns() - start > kWaitLimitNs) {
            atomicOr(&g_device_status, kDrainTimedOut);
            return;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t *dst, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base + i).
__device__ __forceinline__ void tmem_load_32(uint32_t address, int32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- two-CTA (cta_group::2) forms: a pair of CTAs in one cluster drives both SMs' tensor cores
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The shared::cluster address of `p` (an address in this CTA's shared memory) inside CTA `rank`.
__device__ __forceinline__ uint32_t map_to_cta(const void *p, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
    return out;
}
__device__ __forceinline__ void store_cluster_u32(uint32_t cluster_address, uint32_t value) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_address), "r"(value) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_address) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}
// TMA tile load whose completion is counted on a barrier that may live in the peer CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void *dst, const CUtensorMap *map, uint32_t bar_cluster_address,
                                                 int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
        "l"(map), "r"(bar_cluster_address), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *dst, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)),
                 "r"(columns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t address, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}
__device__ __forceinline__ void umma_i8_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives, once the MMAs issued so far have completed, on the barrier at this offset in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint64_t *bar) {
    const uint16_t both = 3;
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
            smem_u32(bar)),
        "h"(both)
        : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte
// swizzled, eight rows (1024 bytes) per swizzle atom: start address, leading offset 1
// (unused by this layout), stride 1024 between atoms, descriptor version 1, swizzle mode 2.
__device__ __forceinline__ uint64_t smem_descriptor(uint32_t address) {
    return static_cast<uint64_t>((address & 0x3ffffu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(1024 >> 4) << 32) |
           (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::i8: i32 accumulate (2 at bit 4), signed 8-bit A and B
// (1 at bits 7 and 10), both K-major, N/8 at bit 17, M/16 at bit 24.
__host__ __device__ constexpr uint32_t instruction_descriptor(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
           (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------- kernel
template <int BN>
struct Tile {
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kABytes = kBlockM * kBlockK;
    static constexpr int kBBytes = BN * kBlockK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemColumns = 2 * BN;
    // stages, then barriers (full, empty per stage; full, empty per accumulator), the TMEM
    // base and the abort flag; 1024 spare bytes to align the stages.
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kEpilogueWarps * kStagingBytes;
};

struct GemmArgs {
    uint32_t m, n, k_blocks;
    uint32_t n_group;      // pair kernel: output tile columns walked together (0: all rows of a column first)
    uint32_t serpentine;   // pair kernel, grouped order: every other tile of a cluster walks K backwards
    const float *scale;    // [n] per output channel
    const float *a_scale;  // [m] per token
    const float *gate;     // [n], residual epilogue only
    void *c;               // f16 [m][n] | bf16 [m][n] in/out | f16 [m][n/2] | i32 [m][n]
    // Column-sharded launches (template flag S): this launch owns output columns c_offset.. of rows
    // that are c_pitch elements long, and stores every finished vector into `world` destination
    // buffers -- its own (`c`, also the source of the residual) and the peers' copies of the same
    // tensor, reached through peer-mapped pointers.  When the last CTA has finished, slot `rank` of
    // every destination's flag array receives `epoch`.
    uint32_t world, rank, c_pitch, c_offset, epoch;
    void *dest[8];
    uint32_t *flags[8];
    uint32_t *done_counter;
    const uint32_t *epoch_base;  // optional device word added to `epoch` (lets a replayed graph count on)
    // Epi::PlainRope: the q|k|v|gate product whose epilogue also does the QK-norm + RoPE launch's work.  Columns
    // are heads of 128 channels: q_heads query heads, then kv_heads key heads, then kv_heads value heads, the
    // rest (the attention gate) stays in `c`.
    const float *rope_cos, *rope_sin;  // f32 [m][128]
    const float *q_norm, *k_norm;      // f32 [128]
    uint16_t *q_out, *k_out, *v_out;   // f16 [m][q_heads*128], [m][kv_heads*128], [m][kv_heads*128]
    uint32_t q_heads, kv_heads;
    float rope_eps;
};

// Stores one 16-byte vector at byte offset `at` of the output: into `c` alone, or into every
// destination of a sharded launch.
template <bool S>
__device__ __forceinline__ void store_out(const GemmArgs &g, size_t at, uint4 value) {
    if constexpr (S) {
#pragma unroll
        for (int d = 0; d < 8; d++)
            if (d < static_cast<int>(g.world)) *reinterpret_cast<uint4 *>(static_cast<uint8_t *>(g.dest[d]) + at) = value;
    } else {
        *reinterpret_cast<uint4 *>(static_cast<uint8_t *>(g.c) + at) = value;
    }
}

__device__ __forceinline__ float dequant(int32_t acc, float ws, float as) {
    // kernels/gemm_i8_256.loom:610-620: sitofp, times the channel scale, times the token scale, bf16.
    return bf_round(__fmul_rn(__fmul_rn(__int2float_rn(acc), ws), as));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __halves2half2(__float2half_rn(lo), __float2half_rn(hi));
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t pack_bf162(float lo, float hi) {
    __nv_bfloat162 b = __halves2bfloat162(__float2bfloat16_rn(lo), __float2bfloat16_rn(hi));
    return *reinterpret_cast<uint32_t *>(&b);
}

// Output of one thread's 32 accumulator columns: 16-byte vectors per chunk and bytes per element.
template <Epi E>
struct Out {
    static constexpr int kVectors = E == Epi::Acc ? 8 : ((E == Epi::Swiglu || E == Epi::SwigluRot) ? 2 : 4);  // PlainRope as Plain
    static constexpr int kElementBytes = E == Epi::Acc ? 4 : 2;
};

// ---- the SwiGLU epilogue that also starts the next prologue's rotation (Epi::SwigluRot)
// prepare_plain_i8 rotates every aligned group of 256 SwiGLU outputs with four radix-4 stages (strides 1, 4, 16,
// 64), each followed by a quarter and an f16 rounding (kernels/prepare_plain_i8.loom:112-167, 213-232, 259-278).
// An epilogue thread owns 64 consecutive outputs of one row, an aligned quarter of such a group, so the first
// three stages touch nothing but its own registers and can run here, under the next tile's main loop; what
// reaches memory is the f16 row after three stages, and the prologue that follows does the last stage, the
// row maximum and the codes.  Same operations in the same order with the same roundings: the int8 codes and
// scales equal those of the unfused pair bit for bit.
struct Pair2 {
    float a, b;
};
__device__ __forceinline__ Pair2 add2(Pair2 x, Pair2 y) { return Pair2{__fadd_rn(x.a, y.a), __fadd_rn(x.b, y.b)}; }
__device__ __forceinline__ Pair2 sub2(Pair2 x, Pair2 y) { return Pair2{__fsub_rn(x.a, y.a), __fsub_rn(x.b, y.b)}; }
// One radix-4 butterfly on both lanes of the pairs (kernels/prepare_plain_i8.loom:121-128).
__device__ __forceinline__ void butterfly2(Pair2 &e0, Pair2 &e1, Pair2 &e2, Pair2 &e3) {
    const Pair2 s01 = add2(e0, e1), s23 = add2(e2, e3), d01 = sub2(e0, e1), d23 = sub2(e2, e3);
    e0 = add2(s01, d23);
    e1 = sub2(s01, d23);
    e2 = add2(d01, s23);
    e3 = sub2(s23, d01);
}
// f32(h) * 0.25 for both halves of an f16x2 word.  The stage's quarter is applied to its inputs: a power of two
// commutes with the f32 additions and with the f16 rounding that follows (nothing is near the f32 underflow).
__device__ __forceinline__ Pair2 unpack_quarter(uint32_t w) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w));
    return Pair2{__fmul_rn(f.x, 0.25f), __fmul_rn(f.y, 0.25f)};
}
__device__ __forceinline__ uint32_t pack_pair(Pair2 v) { return pack_half2(v.a, v.b); }
// Strides 1 and 4 inside 16 consecutive f16-valued outputs o[0..15]; leaves them as eight f16x2 words in order.
__device__ __forceinline__ void rotate16(const float (&o)[16], uint32_t *words) {
    uint32_t w[8];
#pragma unroll
    for (int half = 0; half < 2; half++) {  // quads 2*half and 2*half + 1 ride in the two lanes of a pair
        Pair2 e[4];
#pragma unroll
        for (int i = 0; i < 4; i++) e[i] = Pair2{__fmul_rn(o[8 * half + i], 0.25f), __fmul_rn(o[8 * half + 4 + i], 0.25f)};
        butterfly2(e[0], e[1], e[2], e[3]);
        w[4 * half + 0] = pack_half2(e[0].a, e[1].a);
        w[4 * half + 1] = pack_half2(e[2].a, e[3].a);
        w[4 * half + 2] = pack_half2(e[0].b, e[1].b);
        w[4 * half + 3] = pack_half2(e[2].b, e[3].b);
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {  // word i holds outputs 2i, 2i+1; its quad partners are words i+2, i+4, i+6
        Pair2 e0 = unpack_quarter(w[i]), e1 = unpack_quarter(w[i + 2]), e2 = unpack_quarter(w[i + 4]), e3 = unpack_quarter(w[i + 6]);
        butterfly2(e0, e1, e2, e3);
        w[i] = pack_pair(e0), w[i + 2] = pack_pair(e1), w[i + 4] = pack_pair(e2), w[i + 6] = pack_pair(e3);
    }
#pragma unroll
    for (int i = 0; i < 8; i++) words[i] = w[i];
}

// One thread's 32 consecutive accumulator columns of one row, starting at (shard-local) column n,
// turned into that row's output vectors.  `prior` points at the same columns of the residual row.
template <Epi E>
__device__ __forceinline__ void epilogue_math(const int32_t (&acc)[32], const GemmArgs &g, uint32_t n, float as,
                                              const uint4 *prior, uint4 (&out)[Out<E>::kVectors]) {
    float ws[32];
    if constexpr (E != Epi::Acc) {
#pragma unroll
        for (int i = 0; i < 8; i++)
            *reinterpret_cast<float4 *>(ws + 4 * i) = __ldg(reinterpret_cast<const float4 *>(g.scale + n) + i);
    }
    if constexpr (E == Epi::Plain || E == Epi::PlainRope) {
#pragma unroll
        for (int v = 0; v < 4; v++) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++)
                w[i] = pack_half2(dequant(acc[8 * v + 2 * i], ws[8 * v + 2 * i], as),
                                  dequant(acc[8 * v + 2 * i + 1], ws[8 * v + 2 * i + 1], as));
            out[v] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else if constexpr (E == Epi::Resid) {
        // kernels/gemm_i8_resid_256.loom:622-635: bf16(lin), bf16(lin * gate), bf16(prior + gated).
        float gt[32];
#pragma unroll
        for (int i = 0; i < 8; i++)
            *reinterpret_cast<float4 *>(gt + 4 * i) = __ldg(reinterpret_cast<const float4 *>(g.gate + n) + i);
#pragma unroll
        for (int v = 0; v < 4; v++) {
            const uint4 before = prior[v];
            const uint32_t pw[4] = {before.x, before.y, before.z, before.w};
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int c = 8 * v + 2 * i;
                float lo = bf_round(__fmul_rn(dequant(acc[c], ws[c], as), gt[c]));
                float hi = bf_round(__fmul_rn(dequant(acc[c + 1], ws[c + 1], as), gt[c + 1]));
                lo = __fadd_rn(__uint_as_float(pw[i] << 16), lo);
                hi = __fadd_rn(__uint_as_float(pw[i] & 0xffff0000u), hi);
                w[i] = pack_bf162(lo, hi);
            }
            out[v] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else if constexpr (E == Epi::Swiglu || E == Epi::SwigluRot) {
        // kernels/gemm_i8_swiglu_256.loom:612-660: columns n..n+15 are gate rows, n+16..n+31 the
        // matching up rows; 16 outputs at column n/2.
#pragma unroll
        for (int v = 0; v < 2; v++) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float r[2];
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int o = 8 * v + 2 * i + h;
                    float gv = dequant(acc[o], ws[o], as);
                    float uv = dequant(acc[o + 16], ws[o + 16], as);
                    float silu = bf_round(__fmul_rn(gv, sigmoid_f32(gv)));
                    r[h] = bf_round(__fmul_rn(silu, uv));
                }
                w[i] = pack_half2(r[0], r[1]);
            }
            out[v] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
#pragma unroll
        for (int v = 0; v < 8; v++) out[v] = make_uint4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
    }
}

// ---- the q|k|v|gate epilogue that also normalises and rotates q and k (Epi::PlainRope)
// rope_qknorm_f16 (kernels/rope_qknorm_f16.loom:78-157) reads the f16 q and k heads this GEMM writes, normalises
// each head of 128 channels (RMS with 1 + scale, bf16), rotates channel pairs by the token's angles (bf16) and
// writes f16 q and k; v is copied.  An epilogue thread owns one row and 128 consecutive accumulator columns,
// exactly one head, so all of it can happen here on the values the plain epilogue would have stored: the sum of
// squares in the order the standalone kernel uses (four channels per partial, the 32 partials by the xor tree
// 16, 8, 4, 2, 1), the same operations and roundings, hence the same bits.  The head's accumulators are read
// from tensor memory twice, once for the sum and once for the outputs.
__device__ __forceinline__ void dequant_chunk(const int32_t (&acc)[32], const GemmArgs &g, uint32_t n, float as, float (&x)[32]) {
    float ws[32];
#pragma unroll
    for (int i = 0; i < 8; i++) *reinterpret_cast<float4 *>(ws + 4 * i) = __ldg(reinterpret_cast<const float4 *>(g.scale + n) + i);
#pragma unroll
    for (int i = 0; i < 32; i++) x[i] = __half2float(__float2half_rn(dequant(acc[i], ws[i], as)));  // what gemm_i8_256 stores
}

template <int kChunks>
__device__ __forceinline__ void epilogue_tile_rope(const GemmArgs &g, uint32_t tmem_lane_base, uint32_t row_base, uint32_t n0,
                                                   int first_chunk, uint8_t *stage, int lane) {
    static_assert(kChunks == 4, "a thread owns 128 accumulator columns: one head");
    const uint32_t row = row_base + lane;
    const bool in_range = row < g.m;
    const uint32_t column = n0 + first_chunk * 32, head = column / 128;  // the same for the whole warp
    const bool is_q = head < g.q_heads, is_k = !is_q && head < g.q_heads + g.kv_heads;
    const bool is_v = !is_q && !is_k && head < g.q_heads + 2 * g.kv_heads;
    // Where this head's 128 columns go: element pointer of row 0 and the row pitch in elements.
    uint16_t *dest;
    size_t pitch;
    if (is_q) dest = g.q_out + head * 128, pitch = static_cast<size_t>(g.q_heads) * 128;
    else if (is_k) dest = g.k_out + (head - g.q_heads) * 128, pitch = static_cast<size_t>(g.kv_heads) * 128;
    else if (is_v) dest = g.v_out + (head - g.q_heads - g.kv_heads) * 128, pitch = static_cast<size_t>(g.kv_heads) * 128;
    else dest = static_cast<uint16_t *>(g.c) + column, pitch = g.n;
    const float as = in_range ? __ldg(g.a_scale + row) : 0.0f;
    float rinv = 0.0f;
    if (is_q || is_k) {
        float partial[32];  // partial[l]: the four channels 4l .. 4l + 3, as lane l of the standalone kernel sums them
#pragma unroll
        for (int cc = 0; cc < 4; cc++) {
            int32_t acc[32];
            tmem_load_32(tmem_lane_base + (first_chunk + cc) * 32, acc);
            float x[32];
            dequant_chunk(acc, g, column + cc * 32, as, x);
#pragma unroll
            for (int l = 0; l < 8; l++)
                partial[8 * cc + l] = __fadd_rn(__fadd_rn(__fmul_rn(x[4 * l], x[4 * l]), __fmul_rn(x[4 * l + 1], x[4 * l + 1])),
                                                __fadd_rn(__fmul_rn(x[4 * l + 2], x[4 * l + 2]), __fmul_rn(x[4 * l + 3], x[4 * l + 3])));
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
            for (int l = 0; l < off; l++) partial[l] = __fadd_rn(partial[l], partial[l + off]);
        rinv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(partial[0], 0.0078125f), g.rope_eps)));
    }
    const float *norm = is_q ? g.q_norm : g.k_norm;
    int slot = 0;
#pragma unroll 1
    for (int cc = 0; cc < 4; cc++) {
        int32_t acc[32];
        tmem_load_32(tmem_lane_base + (first_chunk + cc) * 32, acc);
        uint4 out[4];
        if (in_range) {
            if (is_q || is_k) {
                float x[32];
                dequant_chunk(acc, g, column + cc * 32, as, x);
                const float *cos_row = g.rope_cos + static_cast<size_t>(row) * 128 + cc * 32;
                const float *sin_row = g.rope_sin + static_cast<size_t>(row) * 128 + cc * 32;
#pragma unroll
                for (int v = 0; v < 4; v++) {
                    uint32_t w[4];
#pragma unroll
                    for (int h = 0; h < 2; h++) {  // four channels at a time, as one lane of the standalone kernel
                        const int c0 = 8 * v + 4 * h;
                        const float4 sc = __ldg(reinterpret_cast<const float4 *>(norm + cc * 32 + c0));
                        const float4 cs = __ldg(reinterpret_cast<const float4 *>(cos_row + c0));
                        const float4 sn = __ldg(reinterpret_cast<const float4 *>(sin_row + c0));
                        const float x0 = bf_round(__fmul_rn(__fmul_rn(x[c0], rinv), __fadd_rn(sc.x, 1.0f)));
                        const float x1 = bf_round(__fmul_rn(__fmul_rn(x[c0 + 1], rinv), __fadd_rn(sc.y, 1.0f)));
                        const float x2 = bf_round(__fmul_rn(__fmul_rn(x[c0 + 2], rinv), __fadd_rn(sc.z, 1.0f)));
                        const float x3 = bf_round(__fmul_rn(__fmul_rn(x[c0 + 3], rinv), __fadd_rn(sc.w, 1.0f)));
                        const float o0 = bf_round(__fadd_rn(__fmul_rn(x0, cs.x), __fmul_rn(__fsub_rn(0.0f, x1), sn.x)));
                        const float o1 = bf_round(__fadd_rn(__fmul_rn(x1, cs.y), __fmul_rn(x0, sn.y)));
                        const float o2 = bf_round(__fadd_rn(__fmul_rn(x2, cs.z), __fmul_rn(__fsub_rn(0.0f, x3), sn.z)));
                        const float o3 = bf_round(__fadd_rn(__fmul_rn(x3, cs.w), __fmul_rn(x2, sn.w)));
                        w[2 * h] = pack_half2(o0, o1);
                        w[2 * h + 1] = pack_half2(o2, o3);
                    }
                    out[v] = make_uint4(w[0], w[1], w[2], w[3]);
                }
            } else {
                epilogue_math<Epi::PlainRope>(acc, g, column + cc * 32, as, nullptr, out);  // value and gate heads: as gemm_i8_256
            }
        }
#pragma unroll
        for (int v = 0; v < 4; v++)
            *reinterpret_cast<uint4 *>(stage + lane * 128 + (((slot + v) ^ (lane & 7)) * 16)) = out[v];
        slot += 4;
        if (slot == 8) {
            __syncwarp();
            const size_t out_column = static_cast<size_t>(cc - 1) * 32;  // the flush covers chunks cc - 1 and cc
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int r = j * 4 + lane / 8, piece = lane % 8;
                const uint4 value = *reinterpret_cast<const uint4 *>(stage + r * 128 + ((piece ^ (r & 7)) * 16));
                const uint32_t out_row = row_base + r;
                if (out_row < g.m)
                    *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(dest + out_row * pitch + out_column) + piece * 16) = value;
            }
            __syncwarp();
            slot = 0;
        }
    }
}

// One epilogue warp's share of a finished accumulator tile: 32 rows (its TMEM lane quarter) by
// kChunks consecutive 32-column chunks starting at chunk `first_chunk`.  Every thread computes the
// output vectors of its own row; they go through a 4 KB per-warp staging area in shared memory
// (16-byte pieces xor-swizzled by row, so both the row-wise writes and the piece-wise reads are
// conflict-free) and leave as stores in which P lanes cover P*16 contiguous bytes of one row:
// 128-byte row segments instead of 16-byte pieces scattered over 32 rows, which is what the
// memory system -- and a peer GPU's NVLink port in a sharded launch -- wants.
template <Epi E, bool S, int kChunks>
__device__ __forceinline__ void epilogue_tile(const GemmArgs &g, uint32_t tmem_lane_base, uint32_t row_base,
                                              uint32_t n0, int first_chunk, uint8_t *stage, int lane) {
    constexpr int NV = Out<E>::kVectors;
    constexpr int EB = Out<E>::kElementBytes;
    constexpr int P = (kChunks * NV) < 8 ? (kChunks * NV) : 8;  // pieces of 16 bytes per row and flush
    static_assert(P == 4 || P == 8, "a flush covers 64 or 128 bytes of a row");
    constexpr int kRowsPerStore = 32 / P;
    const uint32_t row = row_base + lane;
    const bool in_range = row < g.m;
    // Output geometry in elements: row pitch, and the column of this launch's first output.
    const size_t pitch = S ? g.c_pitch : ((E == Epi::Swiglu || E == Epi::SwigluRot) ? g.n / 2 : g.n);
    const size_t column0 = (S ? g.c_offset : 0);
    float as = 0.0f;
    if constexpr (E != Epi::Acc) as = in_range ? __ldg(g.a_scale + row) : 0.0f;
    if constexpr (E == Epi::SwigluRot) {
        static_assert(kChunks == 4 && P == 8 && !S, "a thread owns 128 accumulator columns = 64 outputs of its row");
        uint32_t words[32];  // the thread's 64 outputs as f16x2 words, in order
#pragma unroll
        for (int cc = 0; cc < 4; cc++) {
            const uint32_t n = n0 + (first_chunk + cc) * 32;
            int32_t acc[32];
            tmem_load_32(tmem_lane_base + (first_chunk + cc) * 32, acc);
            float o[16];
            if (in_range) {
                uint4 plain[2];
                epilogue_math<E>(acc, g, n, as, nullptr, plain);  // the 16 f16 outputs of gemm_i8_swiglu_256
                const uint32_t pw[8] = {plain[0].x, plain[0].y, plain[0].z, plain[0].w, plain[1].x, plain[1].y, plain[1].z, plain[1].w};
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&pw[i]));
                    o[2 * i] = f.x, o[2 * i + 1] = f.y;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 16; i++) o[i] = 0.0f;
            }
            rotate16(o, words + 8 * cc);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {  // stride 16: word i of each 16-output block
            Pair2 e0 = unpack_quarter(words[i]), e1 = unpack_quarter(words[8 + i]), e2 = unpack_quarter(words[16 + i]),
                  e3 = unpack_quarter(words[24 + i]);
            butterfly2(e0, e1, e2, e3);
            words[i] = pack_pair(e0), words[8 + i] = pack_pair(e1), words[16 + i] = pack_pair(e2), words[24 + i] = pack_pair(e3);
        }
#pragma unroll
        for (int v = 0; v < 8; v++)
            *reinterpret_cast<uint4 *>(stage + lane * 128 + ((v ^ (lane & 7)) * 16)) =
                make_uint4(words[4 * v], words[4 * v + 1], words[4 * v + 2], words[4 * v + 3]);
        __syncwarp();
        const size_t out_column = (n0 + first_chunk * 32) / 2;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int r = j * 4 + lane / 8, piece = lane % 8;
            const uint4 value = *reinterpret_cast<const uint4 *>(stage + r * 128 + ((piece ^ (r & 7)) * 16));
            const uint32_t out_row = row_base + r;
            if (out_row < g.m) store_out<false>(g, (out_row * pitch + out_column) * 2 + piece * 16, value);
        }
        __syncwarp();
        return;
    }
    int slot = 0;
    uint32_t flush_n = n0 + first_chunk * 32;  // accumulator column of the first piece awaiting a flush
#pragma unroll 1
    for (int cc = 0; cc < kChunks; cc++) {
        const uint32_t n = n0 + (first_chunk + cc) * 32;
        int32_t acc[32];
        tmem_load_32(tmem_lane_base + (first_chunk + cc) * 32, acc);
        uint4 out[NV];
        if (in_range) {
            const uint4 *prior = nullptr;
            if constexpr (E == Epi::Resid)
                prior = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(g.c) + row * pitch + column0 + n);
            epilogue_math<E>(acc, g, n, as, prior, out);
        }
#pragma unroll
        for (int v = 0; v < NV; v++)
            *reinterpret_cast<uint4 *>(stage + lane * (P * 16) + (((slot + v) ^ (lane & (P - 1))) * 16)) = out[v];
        slot += NV;
        if (slot == P) {
            __syncwarp();
            const size_t out_column = column0 + (E == Epi::Swiglu ? flush_n / 2 : flush_n);
#pragma unroll
            for (int j = 0; j < P; j++) {
                const int r = j * kRowsPerStore + lane / P, piece = lane % P;
                const uint4 value = *reinterpret_cast<const uint4 *>(stage + r * (P * 16) + ((piece ^ (r & (P - 1))) * 16));
                const uint32_t out_row = row_base + r;
                if (out_row < g.m) store_out<S>(g, (out_row * pitch + out_column) * EB + piece * 16, value);
            }
            __syncwarp();
            slot = 0;
            flush_n = n + 32;
        }
    }
}

// After the CTA-wide (or cluster-wide) barrier that follows the last tile: the last CTA of a sharded
// launch to get here publishes `epoch` in every destination's flag slot.  Each storing thread has
// already fenced at system scope, so whoever observes the flag observes the stores.
__device__ __forceinline__ void publish_shard(const GemmArgs &g) {
    if (threadIdx.x != 0 || g.done_counter == nullptr) return;
    __threadfence_system();
    const uint32_t finished = atomicAdd(g.done_counter, 1u);
    if (finished != gridDim.x - 1) return;
    *g.done_counter = 0;  // ready for the next launch on this stream
    const uint32_t value = g.epoch + (g.epoch_base ? *g.epoch_base : 0u);
    __threadfence_system();
#pragma unroll
    for (int d = 0; d < 8; d++)
        if (d < static_cast<int>(g.world) && g.flags[d] != nullptr)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(g.flags[d] + g.rank), "r"(value) : "memory");
}

template <Epi E, int BN, bool S>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const GemmArgs g) {
    using T = Tile<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + T::kStages * T::kStageBytes);
    uint64_t *empty = full + T::kStages;
    uint64_t *acc_full = empty + T::kStages;
    uint64_t *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    uint8_t *staging = smem + T::kStages * T::kStageBytes + 256;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t m_tiles = (g.m + kBlockM - 1) / kBlockM;
    const uint32_t tiles = m_tiles * (g.n / BN);
    uint32_t armed = 0, armed_parity = 0;  // producer thread: stages with a load issued, and the phase of the last one

    if (threadIdx.x == 0) {
        for (int s = 0; s < T::kStages; s++) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(acc_full + a, 1);
            mbar_init(acc_empty + a, kEpilogueWarps * 32);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        __syncwarp();
        tmem_alloc(tmem_slot, T::kTmemColumns);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    chain_wait();  // everything above touched only this CTA's shared and tensor memory

    if (warp == kProducerWarp) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool alive = true;
            for (uint32_t tile = blockIdx.x; alive && tile < tiles; tile += gridDim.x) {
                const int m0 = static_cast<int>(tile % m_tiles) * kBlockM;
                const int n0 = static_cast<int>(tile / m_tiles) * BN;
                for (uint32_t kb = 0; kb < g.k_blocks; kb++) {
                    if (!mbar_wait(empty + stage, phase ^ 1u, abort_flag, kProducerTimedOut)) {
                        alive = false;
                        break;
                    }
                    uint8_t *a_dst = smem + stage * T::kStageBytes;
                    mbar_expect_tx(full + stage, T::kStageBytes);
                    tma_load_2d(a_dst, &map_a, full + stage, static_cast<int>(kb) * kBlockK, m0);
                    tma_load_2d(a_dst + T::kABytes, &map_w, full + stage, static_cast<int>(kb) * kBlockK, n0);
                    armed |= 1u << stage;
                    armed_parity = (armed_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == T::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            constexpr uint32_t idesc = instruction_descriptor(kBlockM, BN);
            uint32_t stage = 0, phase = 0, local = 0;
            bool alive = true;
            for (uint32_t tile = blockIdx.x; alive && tile < tiles; tile += gridDim.x, local++) {
                const uint32_t a = local & 1u, a_phase = (local >> 1) & 1u;
                if (!mbar_wait(acc_empty + a, a_phase ^ 1u, abort_flag, kMmaTimedOut)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + a * BN;
                for (uint32_t kb = 0; kb < g.k_blocks; kb++) {
                    if (!mbar_wait(full + stage, phase, abort_flag, kMmaTimedOut)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + stage * T::kStageBytes);
                    const uint64_t a_desc = smem_descriptor(a_addr);
                    const uint64_t b_desc = smem_descriptor(a_addr + T::kABytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / kUmmaK; k++) {
                        // 32 bytes further along K inside the swizzled row: +2 in 16-byte units.
                        umma_i8(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                    umma_commit(empty + stage);
                    if (++stage == T::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (alive) umma_commit(acc_full + a);
            }
        }
    } else {
        // Epilogue warps: warp w may read TMEM lanes 32*(w%4)..+31 only, one accumulator row per
        // thread; the warps that share a quarter take alternate 32-column chunks.
        constexpr int kColumnGroups = kEpilogueWarps / 4;
        const int quarter = warp & 3, group = warp >> 2;
        uint32_t local = 0;
        for (uint32_t tile = blockIdx.x; tile < tiles; tile += gridDim.x, local++) {
            const uint32_t a = local & 1u, a_phase = (local >> 1) & 1u;
            const uint32_t m0 = (tile % m_tiles) * kBlockM, n0 = (tile / m_tiles) * BN;
            const bool ready = mbar_wait(acc_full + a, a_phase, abort_flag, kEpilogueTimedOut);
            if (!__all_sync(0xffffffffu, ready)) break;
            tc_fence_after();
            const uint32_t lane_base = tmem_base + a * BN + (static_cast<uint32_t>(quarter * 32) << 16);
            constexpr int kChunks = BN / 32 / kColumnGroups;
            if constexpr (E == Epi::PlainRope)
                epilogue_tile_rope<kChunks>(g, lane_base, m0 + quarter * 32, n0, group * kChunks, staging + warp * kStagingBytes, lane);
            else
                epilogue_tile<E, S, kChunks>(g, lane_base, m0 + quarter * 32, n0, group * kChunks, staging + warp * kStagingBytes,
                                             lane);
            tc_fence_before();
            mbar_arrive(acc_empty + a);
        }
        if constexpr (S) __threadfence_system();
    }

    tc_fence_before();
    __syncthreads();  // every role is done: the abort flag is final
    tc_fence_after();
    if (*abort_flag) {
        // Drain: no load of this CTA may still be writing shared memory when it exits.  Whichever role gave
        // up, the producer thread waits here for the last load it issued into every stage.
        if (warp == kProducerWarp && lane == 0) {
            const uint64_t start = global_timer_ns();
            for (int s = 0; s < T::kStages; s++)
                if (armed & (1u << s)) drain_stage(full + s, (armed_parity >> s) & 1u, start);
        }
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        __syncwarp();
        tmem_dealloc(tmem_base, T::kTmemColumns);
    }
    if constexpr (S) publish_shard(g);
}

// ---------------------------------------------------------------- two-CTA kernel
// A cluster of two CTAs computes a 256 x 256 tile: CTA r holds rows r*128.. of A and rows
// r*128.. of the W tile in its own shared memory (32 KB per stage instead of 48), the leader's
// MMA thread issues tcgen05.mma.cta_group::2 (256 x 256 x 32) that reads both halves, and each
// CTA ends up with its 128 accumulator rows x 256 columns in its own tensor memory.  Per SM this
// moves a third less operand data than the single-CTA tile and leaves six stages in flight.
// Barriers: each CTA's loads complete on the LEADER's full[s]; the leader's commit arrives on
// empty[s] and acc_full[a] of both CTAs; one lane per epilogue warp of both CTAs arrives on the
// leader's acc_empty[a].
struct PairTile {
    static constexpr int kStages = 6;
    static constexpr int kBN = 256;
    static constexpr int kABytes = kBlockM * kBlockK;
    static constexpr int kBBytes = (kBN / 2) * kBlockK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemColumns = 2 * kBN;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + kEpilogueWarps * kStagingBytes;
};

template <Epi E, bool S>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_i8_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const GemmArgs g) {
    using T = PairTile;
    constexpr int BN = T::kBN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + T::kStages * T::kStageBytes);
    uint64_t *empty = full + T::kStages;
    uint64_t *acc_full = empty + T::kStages;
    uint64_t *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    // Teardown exchange: [0], [1] the loads each CTA's producer issued (kept in the leader), [2], [3] each CTA's
    // abort flag (kept in both CTAs).
    volatile uint32_t *exchange = reinterpret_cast<volatile uint32_t *>(tmem_slot + 2);
    uint8_t *staging = smem + T::kStages * T::kStageBytes + 256;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    uint32_t issued = 0;  // producer thread: stage loads issued by this CTA
    const bool leader = rank == 0;
    const uint32_t pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const uint32_t m_tiles = (g.m + 2 * kBlockM - 1) / (2 * kBlockM);
    const uint32_t tiles = m_tiles * (g.n / BN);
    // Tile order.  By default a column of tiles is walked top to bottom before the next one, so the tiles
    // in flight (74 pairs) share all of A and a few column panels of W: right while A stays in L2.  When A
    // is larger than that (the down projection: 76 MB), `n_group` column panels are walked row by row
    // instead, so that this group's W panels stay resident while A streams through once per group.
    const uint32_t n_tiles = g.n / BN;
    auto tile_origin = [&](uint32_t tile, uint32_t &tile_m, uint32_t &tile_n) {
        if (g.n_group == 0) {
            tile_m = tile % m_tiles;
            tile_n = tile / m_tiles;
        } else {
            const uint32_t per_group = m_tiles * g.n_group, group = tile / per_group, t = tile % per_group;
            const uint32_t first = group * g.n_group, width = n_tiles - first < g.n_group ? n_tiles - first : g.n_group;
            tile_m = t / width;
            tile_n = first + t % width;
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < T::kStages; s++) {
            mbar_init(full + s, 1);
            mbar_init(empty + s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(acc_full + a, 1);
            mbar_init(acc_empty + a, 2 * kEpilogueWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        __syncwarp();
        tmem_alloc_pair(tmem_slot, T::kTmemColumns);
    }
    tc_fence_before();
    cluster_sync_all();  // barriers of both CTAs are initialised and the allocation is visible
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    chain_wait();  // everything above touched only the pair's shared and tensor memory

    if (warp == kProducerWarp) {
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, local = 0;
            bool alive = true;
            for (uint32_t tile = pair; alive && tile < tiles; tile += pairs, local++) {
                uint32_t tile_m, tile_n;
                tile_origin(tile, tile_m, tile_n);
                const int m0 = static_cast<int>(tile_m * 2 * kBlockM + rank * kBlockM);
                const int n0 = static_cast<int>(tile_n * BN + rank * (BN / 2));
                // In the grouped order every other tile of a cluster walks K backwards.  All clusters are on
                // the same local tile at about the same time, so a wave that ends at the high end of K is
                // followed by one that starts there, on W panels whose high end is the part of them most
                // recently in L2.  The accumulators are integer sums: the order of the K steps changes no bit.
                const bool backwards = g.serpentine != 0 && (local & 1u) != 0;
                for (uint32_t kb = 0; kb < g.k_blocks; kb++) {
                    if (!mbar_wait(empty + stage, phase ^ 1u, abort_flag, kProducerTimedOut)) {
                        alive = false;
                        break;
                    }
                    uint8_t *a_dst = smem + stage * T::kStageBytes;
                    const uint32_t leader_full = map_to_cta(full + stage, 0);
                    if (leader) mbar_expect_tx(full + stage, 2 * T::kStageBytes);
                    const int k0 = static_cast<int>(backwards ? g.k_blocks - 1 - kb : kb) * kBlockK;
                    tma_load_2d_pair(a_dst, &map_a, leader_full, k0, m0);
                    tma_load_2d_pair(a_dst + T::kABytes, &map_w, leader_full, k0, n0);
                    issued++;
                    if (++stage == T::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
    } else if (warp == kMmaWarp) {
        if (leader && lane == 0) {
            constexpr uint32_t idesc = instruction_descriptor(2 * kBlockM, BN);
            uint32_t stage = 0, phase = 0, local = 0;
            bool alive = true;
            for (uint32_t tile = pair; alive && tile < tiles; tile += pairs, local++) {
                const uint32_t a = local & 1u, a_phase = (local >> 1) & 1u;
                if (!mbar_wait(acc_empty + a, a_phase ^ 1u, abort_flag, kMmaTimedOut)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + a * BN;
                for (uint32_t kb = 0; kb < g.k_blocks; kb++) {
                    if (!mbar_wait(full + stage, phase, abort_flag, kMmaTimedOut)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + stage * T::kStageBytes);
                    const uint64_t a_desc = smem_descriptor(a_addr);
                    const uint64_t b_desc = smem_descriptor(a_addr + T::kABytes);
#pragma unroll
                    for (int k = 0; k < kBlockK / kUmmaK; k++)
                        umma_i8_pair(tmem_d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit_pair(empty + stage);
                    if (++stage == T::kStages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (alive) umma_commit_pair(acc_full + a);
            }
        }
    } else {
        constexpr int kColumnGroups = kEpilogueWarps / 4;
        const int quarter = warp & 3, group = warp >> 2;
        uint32_t local = 0;
        for (uint32_t tile = pair; tile < tiles; tile += pairs, local++) {
            const uint32_t a = local & 1u, a_phase = (local >> 1) & 1u;
            uint32_t tile_m, tile_n;
            tile_origin(tile, tile_m, tile_n);
            const uint32_t m0 = tile_m * 2 * kBlockM + rank * kBlockM, n0 = tile_n * BN;
            const bool ready = mbar_wait(acc_full + a, a_phase, abort_flag, kEpilogueTimedOut);
            if (!__all_sync(0xffffffffu, ready)) break;
            tc_fence_after();
            const uint32_t lane_base = tmem_base + a * BN + (static_cast<uint32_t>(quarter * 32) << 16);
            constexpr int kChunks = BN / 32 / kColumnGroups;
            if constexpr (E == Epi::PlainRope)
                epilogue_tile_rope<kChunks>(g, lane_base, m0 + quarter * 32, n0, group * kChunks, staging + warp * kStagingBytes, lane);
            else
                epilogue_tile<E, S, kChunks>(g, lane_base, m0 + quarter * 32, n0, group * kChunks, staging + warp * kStagingBytes,
                                             lane);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(acc_empty + a, 0));
        }
        if constexpr (S) __threadfence_system();
    }

    tc_fence_before();
    __syncthreads();  // every role of this CTA is done: its abort flag is final
    if (threadIdx.x == 0) {
        const uint32_t mine = *abort_flag ? 1u : 0u;
        store_cluster_u32(map_to_cta(const_cast<uint32_t *>(exchange) + 2 + rank, 0), mine);
        store_cluster_u32(map_to_cta(const_cast<uint32_t *>(exchange) + 2 + rank, 1), mine);
    }
    if (warp == kProducerWarp && lane == 0) store_cluster_u32(map_to_cta(const_cast<uint32_t *>(exchange) + rank, 0), issued);
    __syncwarp();
    cluster_sync_all();  // neither CTA frees tensor memory or exits while the other may still use it
    tc_fence_after();
    if (exchange[2] | exchange[3]) {
        // One of the CTAs gave up on a wait.  No load may still be writing either CTA's shared memory when the
        // cluster exits, and every load of the pair completes on the LEADER's `full` barriers: the leader's
        // producer thread waits for the last load into every stage.  Where only one CTA issued that load (they
        // can be up to a ring apart when a wait runs out) the barrier's byte count is first put right: the
        // peer's missing half is accounted as complete, or the peer's lone half is armed.
        if (leader && warp == kProducerWarp && lane == 0) {
            const uint32_t issued_leader = exchange[0], issued_peer = exchange[1];
            const uint32_t high = issued_leader > issued_peer ? issued_leader : issued_peer;
            const uint32_t low = high > static_cast<uint32_t>(T::kStages) ? high - T::kStages : 0u;
            const uint64_t start = global_timer_ns();
            for (uint32_t i = low; i < high; i++) {
                const uint32_t s = i % T::kStages, parity = (i / T::kStages) & 1u;
                const bool by_leader = i < issued_leader, by_peer = i < issued_peer;
                if (by_leader && !by_peer) mbar_complete_tx(full + s, T::kStageBytes);
                if (!by_leader && by_peer) mbar_expect_tx(full + s, T::kStageBytes);
                drain_stage(full + s, parity, start);
            }
        }
        __syncwarp();
        cluster_sync_all();  // the peer stays until the leader has seen its loads land
    }
    if (warp == kMmaWarp) {
        __syncwarp();
        tmem_dealloc_pair(tmem_base, T::kTmemColumns);
    }
    if constexpr (S) publish_shard(g);
}

// ---------------------------------------------------------------- host side
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

// int8 [rows][k_stride] viewed as a 2-D tensor (k_size x rows), boxes of 128 bytes x box_rows,
// 128-byte swizzle; out-of-range rows and K read as zero.
int make_operand_map(CUtensorMap *map, const void *base, size_t rows, size_t k_size, size_t k_stride,
                     uint32_t box_rows) {
    EncodeTiled encode = encode_tiled();
    if (!encode) return fail(KREA2_RUNTIME, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[2] = {k_size, rows};
    cuuint64_t strides[1] = {k_stride};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(kBlockK), box_rows};
    cuuint32_t element_strides[2] = {1, 1};
    CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box,
                        element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KREA2_RUNTIME, "cuTensorMapEncodeTiled failed with code %d", static_cast<int>(r));
    return KREA2_OK;
}

int sm_count() {
    static int cached[64];
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (cached[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        cached[device] = n;
    }
    return cached[device];
}

// Raises the kernel's dynamic shared-memory limit once per device.
template <Epi E, int BN, bool S = false>
int ensure_instance() {
    static std::once_flag once[64];
    static cudaError_t attr_status[64];
    int device = 0;
    KREA2_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(KREA2_INTERNAL, "device index %d out of range", device);
    std::call_once(once[device], [&] {
        attr_status[device] = cudaFuncSetAttribute(gemm_i8_kernel<E, BN, S>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   Tile<BN>::kSmemBytes);
    });
    if (attr_status[device] != cudaSuccess)
        return fail(KREA2_RUNTIME, "cannot reserve %d bytes of shared memory: %s", Tile<BN>::kSmemBytes,
                    cudaGetErrorString(attr_status[device]));
    return KREA2_OK;
}

template <Epi E, int BN, bool S = false>
int launch_instance(cudaStream_t stream, const CUtensorMap &map_a, const CUtensorMap &map_w, const GemmArgs &args) {
    if (int status = ensure_instance<E, BN, S>()) return status;
    const uint32_t tiles = ((args.m + kBlockM - 1) / kBlockM) * (args.n / BN);
    const unsigned grid = tiles < static_cast<uint32_t>(sm_count()) ? tiles : static_cast<unsigned>(sm_count());
    cudaError_t status = launch_chain_kernel(gemm_i8_kernel<E, BN, S>, dim3(grid), dim3(kGemmThreads), Tile<BN>::kSmemBytes, stream,
                                             map_a, map_w, args);
    if (status == cudaSuccess) status = cudaGetLastError();
    if (status != cudaSuccess) return fail(KREA2_RUNTIME, "gemm_i8 launch failed: %s", cudaGetErrorString(status));
    return KREA2_OK;
}

// Shared-memory limit and the number of two-CTA clusters this device can hold at once.
template <Epi E, bool S = false>
int ensure_pair_instance(int *clusters) {
    static std::once_flag once[64];
    static cudaError_t attr_status[64];
    static int max_clusters[64];
    int device = 0;
    KREA2_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return fail(KREA2_INTERNAL, "device index %d out of range", device);
    std::call_once(once[device], [&] {
        attr_status[device] = cudaFuncSetAttribute(gemm_i8_pair_kernel<E, S>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   PairTile::kSmemBytes);
        if (attr_status[device] != cudaSuccess) return;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(2 * static_cast<unsigned>(sm_count()), 1, 1);
        config.blockDim = dim3(kGemmThreads, 1, 1);
        config.dynamicSmemBytes = PairTile::kSmemBytes;
        cudaLaunchAttribute attribute;
        attribute.id = cudaLaunchAttributeClusterDimension;
        attribute.val.clusterDim.x = 2;
        attribute.val.clusterDim.y = 1;
        attribute.val.clusterDim.z = 1;
        config.attrs = &attribute;
        config.numAttrs = 1;
        int n = 0;
        attr_status[device] = cudaOccupancyMaxActiveClusters(&n, gemm_i8_pair_kernel<E, S>, &config);
        max_clusters[device] = n;
    });
    if (attr_status[device] != cudaSuccess)
        return fail(KREA2_RUNTIME, "cannot prepare the two-CTA GEMM: %s", cudaGetErrorString(attr_status[device]));
    if (max_clusters[device] < 1) return fail(KREA2_RUNTIME, "this device cannot hold a two-CTA cluster of the GEMM");
    *clusters = max_clusters[device];
    return KREA2_OK;
}

template <Epi E, bool S = false>
int launch_pair(cudaStream_t stream, const CUtensorMap &map_a, const CUtensorMap &map_w, const GemmArgs &args) {
    int clusters = 0;
    if (int status = ensure_pair_instance<E, S>(&clusters)) return status;
    const uint32_t tiles = ((args.m + 2 * kBlockM - 1) / (2 * kBlockM)) * (args.n / PairTile::kBN);
    const unsigned pairs = tiles < static_cast<uint32_t>(clusters) ? tiles : static_cast<unsigned>(clusters);
    cudaError_t status = launch_chain_kernel(gemm_i8_pair_kernel<E, S>, dim3(2 * pairs), dim3(kGemmThreads), PairTile::kSmemBytes,
                                             stream, map_a, map_w, args);
    if (status == cudaSuccess) status = cudaGetLastError();
    if (status != cudaSuccess) return fail(KREA2_RUNTIME, "gemm_i8 (two-CTA) launch failed: %s", cudaGetErrorString(status));
    return KREA2_OK;
}

// KREA2_GEMM_PAIR=0 keeps every launch on the single-CTA kernel (for A/B measurements).
bool pair_enabled() {
    static const bool enabled = [] {
        const char *v = getenv("KREA2_GEMM_PAIR");
        return !(v && v[0] == '0');
    }();
    return enabled;
}

// The `config.decl` ranges of the GEMM kernels (kernels/gemm_i8_256.loom:14-22,
// gemm_i8_resid_256x256.loom:16-27) and the row-count bound (:97).
int check_gemm(const char *name, size_t m, size_t k_size, size_t k_stride, size_t n_size, size_t m_group,
               size_t k_multiple, size_t n_multiple) {
    KREA2_REQUIRE(m >= 1 && m <= 16777216, "%s: m %zu outside 1..16777216", name, m);
    KREA2_REQUIRE(k_size >= k_multiple && k_size <= 65536 && k_size % k_multiple == 0,
                  "%s: k_size %zu must be a multiple of %zu up to 65536", name, k_size, k_multiple);
    KREA2_REQUIRE(n_size >= n_multiple && n_size <= 32768 && n_size % n_multiple == 0,
                  "%s: n_size %zu must be a multiple of %zu up to 32768", name, n_size, n_multiple);
    KREA2_REQUIRE(k_stride >= 64 && k_stride <= 65536 && k_stride % 64 == 0 && k_stride >= k_size,
                  "%s: k_stride %zu must be a multiple of 64 up to 65536 and at least k_size", name, k_stride);
    KREA2_REQUIRE(m_group >= 1 && m_group <= 4, "%s: m_group %zu outside 1..4", name, m_group);
    return KREA2_OK;
}

// Bounded wait of one device for the flag slots its peers (and itself) publish.
__global__ void shard_advance_kernel(uint32_t *epoch_base, uint32_t delta) { *epoch_base += delta; }

__global__ void shard_wait_kernel(const uint32_t *flags, uint32_t world, uint32_t epoch, const uint32_t *epoch_base) {
    const uint32_t r = threadIdx.x;
    if (r >= world) return;
    if (epoch_base) epoch += *epoch_base;
    const uint64_t start = global_timer_ns();
    for (;;) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + r) : "memory");
        if (static_cast<int32_t>(seen - epoch) >= 0) return;
        if (global_timer_ns() - start > kWaitLimitNs) {
            atomicOr(&g_device_status, kShardWaitTimedOut);
            return;
        }
    }
}

int check_shard(const char *name, const krea2_shard *shard, size_t out_columns) {
    KREA2_REQUIRE(shard->world >= 1 && shard->world <= 8 && shard->rank < shard->world,
                  "%s: world %u / rank %u outside 1..8", name, shard->world, shard->rank);
    KREA2_REQUIRE(shard->pitch % 16 == 0 && shard->offset % 16 == 0 && shard->offset + out_columns <= shard->pitch,
                  "%s: columns %zu..%zu do not fit rows of %zu (both multiples of 16)", name, shard->offset,
                  shard->offset + out_columns, shard->pitch);
    KREA2_REQUIRE(shard->pitch <= 0xffffffffull, "%s: pitch too large", name);
    bool any_flag = false;
    for (uint32_t d = 0; d < shard->world; d++) {
        KREA2_REQUIRE(shard->dest[d] && aligned16(shard->dest[d]), "%s: destination %u is null or unaligned", name, d);
        any_flag = any_flag || shard->flags[d] != nullptr;
    }
    KREA2_REQUIRE(!any_flag || shard->counter, "%s: flags need the launch counter", name);
    return KREA2_OK;
}

// How many 256-column tile panels of W the two-CTA kernel walks together (0 = one column of tiles at a
// time).  With the default order the tiles in flight share all of A; once A is larger than what stays in
// L2 beside the streaming W (measured: the down projection, 76 MB of A, read 626 MB from DRAM instead of
// 233 MB) the panels of a group are kept resident instead and A streams through once per group.
uint32_t tile_column_group(size_t m, size_t k_size, size_t n_size) {
    static const long forced = [] {
        const char *text = std::getenv("KREA2_GEMM_NGROUP");
        return text ? std::strtol(text, nullptr, 10) : -1L;
    }();
    if (forced >= 0) return static_cast<uint32_t>(forced);
    const size_t a_bytes = m * k_size, panel_bytes = 256 * k_size;
    if (a_bytes <= (size_t(48) << 20)) return 0;
    const size_t group = (size_t(48) << 20) / panel_bytes;
    const size_t panels = n_size / 256;
    return static_cast<uint32_t>(group < 1 ? 1 : (group >= panels ? 0 : group));
}

// Whether 128-row tiles on single CTAs need clearly fewer rounds over the SMs than 256-row tiles on CTA pairs.
// Both kinds of round do the same work (one 128 x 256 tile per SM), and the pair kernel's are the faster ones
// (each CTA stages half of W); but when the row count leaves the last 256-row tile half empty -- an odd number
// of 128-row halves, as with 1043 or 1152 rows -- the pairs can pay a whole extra round for it.  The single-CTA
// kernel is taken when it saves at least one round in thirteen.  Integer sums: the choice changes no bit.
bool fewer_rounds_in_halves(size_t m, size_t n_size) {
    static const bool enabled = [] {  // KREA2_GEMM_HALVES=0 keeps the pair kernel (for A/B runs)
        const char *v = std::getenv("KREA2_GEMM_HALVES");
        return !(v && v[0] == '0');
    }();
    if (!enabled) return false;
    const size_t sms = static_cast<size_t>(sm_count()), columns = n_size / 256;
    if (sms < 2) return false;
    const size_t pair_rounds = ((m + 255) / 256 * columns + sms / 2 - 1) / (sms / 2);
    const size_t half_rounds = ((m + 127) / 128 * columns + sms - 1) / sms;
    return half_rounds * 13 <= pair_rounds * 12;
}

// What the PlainRope epilogue needs beyond the plain one's arguments.
struct RopeArgs {
    const float *cos, *sin, *q_norm, *k_norm;
    void *q_out, *k_out, *v_out;
    size_t q_heads, kv_heads;
    float eps;
};

template <Epi E>
int run_gemm(const char *name, cudaStream_t stream, size_t m, const void *a, const void *w, const float *scale,
             const float *a_scale, void *c, const float *gate, size_t k_size, size_t k_stride, size_t n_size,
             const krea2_shard *shard = nullptr, const RopeArgs *rope = nullptr) {
    KREA2_REQUIRE(a && w && c, "%s: null buffer", name);
    KREA2_REQUIRE(aligned16(a) && aligned16(w) && aligned16(c), "%s: buffers must be 16-byte aligned", name);
    if constexpr (E != Epi::Acc) {
        KREA2_REQUIRE(scale && a_scale && aligned16(scale), "%s: scale vectors missing or not 16-byte aligned", name);
    }
    if constexpr (E == Epi::Resid) {
        KREA2_REQUIRE(gate && aligned16(gate), "%s: gate vector missing or not 16-byte aligned", name);
    }
    GemmArgs args;
    args.m = static_cast<uint32_t>(m);
    args.n = static_cast<uint32_t>(n_size);
    args.k_blocks = static_cast<uint32_t>((k_size + kBlockK - 1) / kBlockK);
    args.n_group = tile_column_group(m, k_size, n_size);
    static const bool serpentine_enabled = [] {  // KREA2_GEMM_SERPENTINE=0 keeps every tile walking K forwards (for A/B runs)
        const char *v = std::getenv("KREA2_GEMM_SERPENTINE");
        return !(v && v[0] == '0');
    }();
    args.serpentine = (args.n_group != 0 && serpentine_enabled) ? 1u : 0u;
    args.scale = scale;
    args.a_scale = a_scale;
    args.gate = gate;
    args.c = c;
    args.world = 1, args.rank = 0, args.c_pitch = 0, args.c_offset = 0, args.epoch = 0, args.done_counter = nullptr;
    args.epoch_base = nullptr;
    for (int d = 0; d < 8; d++) args.dest[d] = nullptr, args.flags[d] = nullptr;
    args.rope_cos = args.rope_sin = args.q_norm = args.k_norm = nullptr;
    args.q_out = args.k_out = args.v_out = nullptr;
    args.q_heads = args.kv_heads = 0, args.rope_eps = 0.0f;
    if constexpr (E == Epi::PlainRope) {
        args.rope_cos = rope->cos, args.rope_sin = rope->sin, args.q_norm = rope->q_norm, args.k_norm = rope->k_norm;
        args.q_out = static_cast<uint16_t *>(rope->q_out), args.k_out = static_cast<uint16_t *>(rope->k_out);
        args.v_out = static_cast<uint16_t *>(rope->v_out);
        args.q_heads = static_cast<uint32_t>(rope->q_heads), args.kv_heads = static_cast<uint32_t>(rope->kv_heads);
        args.rope_eps = rope->eps;
    }
    if (shard) {
        args.world = shard->world, args.rank = shard->rank, args.epoch = shard->epoch;
        args.c_pitch = static_cast<uint32_t>(shard->pitch), args.c_offset = static_cast<uint32_t>(shard->offset);
        args.done_counter = shard->counter;
        args.epoch_base = shard->epoch_base;
        for (uint32_t d = 0; d < shard->world; d++) args.dest[d] = shard->dest[d], args.flags[d] = shard->flags[d];
    }
    const bool wide = n_size % 256 == 0;
    // The two-CTA kernel wants whole 256-column tiles and more than one 128-row half to fill.
    const bool pair = wide && m > kBlockM && pair_enabled() && !fewer_rounds_in_halves(m, n_size);
    CUtensorMap map_a, map_w;
    if (int status = make_operand_map(&map_a, a, m, k_size, k_stride, kBlockM)) return status;
    if (int status = make_operand_map(&map_w, w, n_size, k_size, k_stride, (wide && !pair) ? 256 : 128)) return status;
    if constexpr (E != Epi::Acc && E != Epi::SwigluRot && E != Epi::PlainRope) {
        if (shard) {
            if (pair) return launch_pair<E, true>(stream, map_a, map_w, args);
            return wide ? launch_instance<E, 256, true>(stream, map_a, map_w, args)
                        : launch_instance<E, 128, true>(stream, map_a, map_w, args);
        }
    }
    if (pair) return launch_pair<E>(stream, map_a, map_w, args);
    if constexpr (E == Epi::SwigluRot || E == Epi::PlainRope) {
        KREA2_REQUIRE(wide, "%s: n_size %zu must be a multiple of 256", name, n_size);
        return launch_instance<E, 256>(stream, map_a, map_w, args);
    } else {
        return wide ? launch_instance<E, 256>(stream, map_a, map_w, args)
                    : launch_instance<E, 128>(stream, map_a, map_w, args);
    }
}

}  // namespace

// Everything a later launch would otherwise do on first use (driver entry point, shared
// memory limits), so that a launch inside a stream capture issues nothing but the kernel.
int prepare_gemm_device() {
    if (!encode_tiled()) return fail(KREA2_RUNTIME, "cuTensorMapEncodeTiled is not available from this driver");
    sm_count();
    if (int s = ensure_instance<Epi::Plain, 128>()) return s;
    if (int s = ensure_instance<Epi::Plain, 256>()) return s;
    if (int s = ensure_instance<Epi::Resid, 128>()) return s;
    if (int s = ensure_instance<Epi::Resid, 256>()) return s;
    if (int s = ensure_instance<Epi::Swiglu, 128>()) return s;
    if (int s = ensure_instance<Epi::Swiglu, 256>()) return s;
    if (int s = ensure_instance<Epi::SwigluRot, 256>()) return s;
    if (int s = ensure_instance<Epi::PlainRope, 256>()) return s;
    if (int s = ensure_instance<Epi::Acc, 128>()) return s;
    if (int s = ensure_instance<Epi::Acc, 256>()) return s;
    int clusters = 0;
    if (int s = ensure_pair_instance<Epi::Plain>(&clusters)) return s;
    if (int s = ensure_pair_instance<Epi::Resid>(&clusters)) return s;
    if (int s = ensure_pair_instance<Epi::Swiglu>(&clusters)) return s;
    if (int s = ensure_pair_instance<Epi::SwigluRot>(&clusters)) return s;
    if (int s = ensure_pair_instance<Epi::PlainRope>(&clusters)) return s;
    if (int s = ensure_pair_instance<Epi::Acc>(&clusters)) return s;
    return KREA2_OK;
}

}  // namespace krea2

using namespace krea2;

extern "C" int krea2_gemm_i8_256(krea2_stream stream, size_t m, const void *a, const void *w, const float *scale,
                                 const float *a_scale, void *c, size_t k_size, size_t k_stride, size_t n_size,
                                 size_t m_group) {
    clear_error();
    if (int status = check_gemm("gemm_i8_256", m, k_size, k_stride, n_size, m_group, 128, 128)) return status;
    return run_gemm<Epi::Plain>("gemm_i8_256", static_cast<cudaStream_t>(stream), m, a, w, scale, a_scale, c, nullptr,
                                k_size, k_stride, n_size);
}

extern "C" int krea2_gemm_i8_resid_256(krea2_stream stream, size_t m, const void *a, const void *w,
                                       const float *scale, const float *a_scale, void *c, const float *gate,
                                       size_t k_size, size_t k_stride, size_t n_size, size_t m_group) {
    clear_error();
    if (int status = check_gemm("gemm_i8_resid_256", m, k_size, k_stride, n_size, m_group, 128, 128)) return status;
    return run_gemm<Epi::Resid>("gemm_i8_resid_256", static_cast<cudaStream_t>(stream), m, a, w, scale, a_scale, c,
                                gate, k_size, k_stride, n_size);
}

extern "C" int krea2_gemm_i8_resid_256x256(krea2_stream stream, size_t m, const void *a, const void *w,
                                           const float *scale, const float *a_scale, void *c, const float *gate,
                                           size_t k_size, size_t k_stride, size_t n_size, size_t m_group,
                                           size_t schedule_rows) {
    clear_error();
    if (int status = check_gemm("gemm_i8_resid_256x256", m, k_size, k_stride, n_size, m_group, 64, 256))
        return status;
    KREA2_REQUIRE(schedule_rows <= 1, "gemm_i8_resid_256x256: schedule_rows %zu outside 0..1", schedule_rows);
    return run_gemm<Epi::Resid>("gemm_i8_resid_256x256", static_cast<cudaStream_t>(stream), m, a, w, scale, a_scale,
                                c, gate, k_size, k_stride, n_size);
}

extern "C" int krea2_gemm_i8_swiglu_256(krea2_stream stream, size_t m, const void *a, const void *w,
                                        const float *scale, const float *a_scale, void *c, size_t k_size,
                                        size_t k_stride, size_t n_size, size_t m_group) {
    clear_error();
    if (int status = check_gemm("gemm_i8_swiglu_256", m, k_size, k_stride, n_size, m_group, 128, 128)) return status;
    return run_gemm<Epi::Swiglu>("gemm_i8_swiglu_256", static_cast<cudaStream_t>(stream), m, a, w, scale, a_scale, c,
                                 nullptr, k_size, k_stride, n_size);
}

extern "C" int krea2_gemm_i8_swiglu_rotated_256(krea2_stream stream, size_t m, const void *a, const void *w,
                                                const float *scale, const float *a_scale, void *c, size_t k_size,
                                                size_t k_stride, size_t n_size, size_t m_group) {
    clear_error();
    if (int status = check_gemm("gemm_i8_swiglu_rotated_256", m, k_size, k_stride, n_size, m_group, 128, 256)) return status;
    return run_gemm<Epi::SwigluRot>("gemm_i8_swiglu_rotated_256", static_cast<cudaStream_t>(stream), m, a, w, scale, a_scale,
                                    c, nullptr, k_size, k_stride, n_size);
}

extern "C" int krea2_gemm_i8_rope_256(krea2_stream stream, size_t m, const void *a, const void *w, const float *scale,
                                      const float *a_scale, void *c, const float *q_norm, const float *k_norm,
                                      const float *cos_table, const float *sin_table, void *q_out, void *k_out, void *v_out,
                                      size_t k_size, size_t k_stride, size_t n_size, size_t m_group, size_t q_heads,
                                      size_t kv_heads, float eps) {
    clear_error();
    if (int status = check_gemm("gemm_i8_rope_256", m, k_size, k_stride, n_size, m_group, 128, 256)) return status;
    KREA2_REQUIRE(q_heads >= 1 && q_heads <= 256 && kv_heads >= 1 && kv_heads <= 256 && (q_heads + 2 * kv_heads) * 128 <= n_size,
                  "gemm_i8_rope_256: %zu query and 2 x %zu key/value heads of 128 channels do not fit %zu columns", q_heads,
                  kv_heads, n_size);
    KREA2_REQUIRE(q_norm && k_norm && cos_table && sin_table && q_out && k_out && v_out, "gemm_i8_rope_256: null buffer");
    KREA2_REQUIRE(aligned16(q_norm) && aligned16(k_norm) && aligned16(cos_table) && aligned16(sin_table) && aligned16(q_out) &&
                      aligned16(k_out) && aligned16(v_out),
                  "gemm_i8_rope_256: buffers must be 16-byte aligned");
    const RopeArgs rope{cos_table, sin_table, q_norm, k_norm, q_out, k_out, v_out, q_heads, kv_heads, eps};
    return run_gemm<Epi::PlainRope>("gemm_i8_rope_256", static_cast<cudaStream_t>(stream), m, a, w, scale, a_scale, c, nullptr,
                                    k_size, k_stride, n_size, nullptr, &rope);
}

extern "C" int krea2_gemm_i8_acc(krea2_stream stream, size_t m, const void *a, const void *w, int32_t *acc,
                                 size_t k_size, size_t k_stride, size_t n_size) {
    clear_error();
    if (int status = check_gemm("gemm_i8_acc", m, k_size, k_stride, n_size, 1, 64, 128)) return status;
    return run_gemm<Epi::Acc>("gemm_i8_acc", static_cast<cudaStream_t>(stream), m, a, w, nullptr, nullptr, acc,
                              nullptr, k_size, k_stride, n_size);
}

extern "C" int krea2_gemm_i8_sharded(krea2_stream stream, int kind, size_t m, const void *a, const void *w,
                                     const float *scale, const float *a_scale, const float *gate, size_t k_size,
                                     size_t k_stride, size_t n_size, const krea2_shard *shard) {
    clear_error();
    KREA2_REQUIRE(shard, "gemm_i8_sharded: shard description is null");
    KREA2_REQUIRE(kind >= KREA2_SHARD_PLAIN && kind <= KREA2_SHARD_SWIGLU, "gemm_i8_sharded: unknown kind %d", kind);
    if (int status = check_gemm("gemm_i8_sharded", m, k_size, k_stride, n_size, 1, 128, 128)) return status;
    const size_t out_columns = kind == KREA2_SHARD_SWIGLU ? n_size / 2 : n_size;
    if (int status = check_shard("gemm_i8_sharded", shard, out_columns)) return status;
    void *own = shard->dest[shard->rank];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (kind == KREA2_SHARD_PLAIN)
        return run_gemm<Epi::Plain>("gemm_i8_sharded", st, m, a, w, scale, a_scale, own, nullptr, k_size, k_stride, n_size,
                                    shard);
    if (kind == KREA2_SHARD_SWIGLU)
        return run_gemm<Epi::Swiglu>("gemm_i8_sharded", st, m, a, w, scale, a_scale, own, nullptr, k_size, k_stride, n_size,
                                     shard);
    return run_gemm<Epi::Resid>("gemm_i8_sharded", st, m, a, w, scale, a_scale, own, gate, k_size, k_stride, n_size, shard);
}

extern "C" int krea2_shard_advance(krea2_stream stream, uint32_t *epoch_base, uint32_t delta) {
    clear_error();
    KREA2_REQUIRE(epoch_base, "shard_advance: epoch word is null");
    shard_advance_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(epoch_base, delta);
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return fail(KREA2_RUNTIME, "shard_advance launch failed: %s", cudaGetErrorString(status));
    return KREA2_OK;
}

extern "C" int krea2_shard_wait(krea2_stream stream, const uint32_t *flags, uint32_t world, uint32_t epoch,
                                const uint32_t *epoch_base) {
    clear_error();
    KREA2_REQUIRE(flags && world >= 1 && world <= 8, "shard_wait: flags null or world outside 1..8");
    shard_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, world, epoch, epoch_base);
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return fail(KREA2_RUNTIME, "shard_wait launch failed: %s", cudaGetErrorString(status));
    return KREA2_OK;
}

extern "C" int krea2_device_status(int *host_status) {
    clear_error();
    KREA2_REQUIRE(host_status, "device_status: null output");
    KREA2_CUDA(cudaDeviceSynchronize());
    int value = 0;
    KREA2_CUDA(cudaMemcpyFromSymbol(&value, g_device_status, sizeof(int)));
    if (value != 0) {
        int zero = 0;
        KREA2_CUDA(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    }
    int attention = 0;
    if (int status = take_attention_status(&attention)) return status;
    *host_status = value | attention;
    return KREA2_OK;
}
