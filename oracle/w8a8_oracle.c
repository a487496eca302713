/*
 * CPU restatement of krea2-hrx's W8A8 linear-layer arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or calls
 * this file; it exists so the tests, the smoke check and the benchmark's CPU
 * baseline have an independent statement of what the CUDA kernels must produce.
 *
 * Every function cites the reference source it follows (paths are relative to the
 * krea2-hrx repository).  Where the reference leaves an f32 evaluation order to its
 * compiler (the 8-wide and 32-lane sum reductions, the approximate exp, rsqrt) this
 * file fixes ONE order, documented at the function, and the CUDA kernels are held
 * to that order bit for bit.  Those spots are "parity unpinned" against the
 * reference's kernels at the ulp level; the reference's own tests tolerate +-1 code
 * there.  Each of them feeds a bf16 rounding, and against the reference's torch code
 * (scripts/quantized_reference.py, imported by the scripts under tests/golden/) the
 * bf16 results are equal on every fixture value: RMSNorm + adaLN, the attention gate,
 * QK-norm + RoPE, the SwiGLU product, the residual update.
 * Everything else (the Hadamard butterflies, bf16/f16 rounding points, quantisation,
 * the i32 dot, the three epilogues) is pinned by the reference's tests, restated in
 * tests/test_oracle_pins.py.
 *
 * Build: see oracle/Makefile (-O2 -ffp-contract=off, no fast-math; every f32
 * operation below is meant to be exactly one IEEE operation).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---------------------------------------------------------------- conversions */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* bf16 -> f32 is exact (src/numerics.rs:11-13). */
static inline float bf16_to_f32(uint16_t b) { return bits_f32((uint32_t)b << 16); }

/* f32 -> bf16, round to nearest even, NaN quieted (src/numerics.rs:18-26). */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
static inline float bf(float x) { return bf16_to_f32(f32_to_bf16(x)); }

/* f16 -> f32, exact. */
static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
    if (e == 0) {
        if (m == 0) return bits_f32(sign);
        /* subnormal: m * 2^-24 */
        float v = (float)m * 5.9604644775390625e-08f;
        return (sign ? -v : v);
    }
    if (e == 31) return bits_f32(sign | 0x7f800000u | (m << 13));
    return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
}

/* f32 -> f16, IEEE round to nearest even with subnormals and overflow to inf: the
 * `fptrunc ... to f16` of kernels/prepare_plain_i8.loom:121 and the GEMM epilogues. */
static inline uint16_t f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    x &= 0x7fffffffu;
    if (x > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (x >= 0x38800000u) { /* >= 2^-14: normal half (or overflow) */
        uint32_t m = x - 0x38000000u;
        uint32_t r = (m + 0xfffu + ((m >> 13) & 1u)) >> 13;
        if (r >= 0x7c00u) r = 0x7c00u;
        return (uint16_t)(sign | r);
    }
    if (x <= 0x33000000u) return sign; /* <= 2^-25 rounds to zero (tie goes to even) */
    {
        uint32_t e = x >> 23, mant = (x & 0x7fffffu) | 0x800000u;
        uint32_t shift = 126u - e; /* 14..24 */
        uint32_t q = mant >> shift, rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1u);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
}
static inline float hf(float x) { return f16_to_f32(f32_to_f16(x)); }

/* Exported so the tests can check the conversions against numpy. */
void oracle_f32_to_f16(const float *src, uint16_t *dst, size_t n) { for (size_t i = 0; i < n; i++) dst[i] = f32_to_f16(src[i]); }
void oracle_f16_to_f32(const uint16_t *src, float *dst, size_t n) { for (size_t i = 0; i < n; i++) dst[i] = f16_to_f32(src[i]); }
void oracle_f32_to_bf16(const float *src, uint16_t *dst, size_t n) { for (size_t i = 0; i < n; i++) dst[i] = f32_to_bf16(src[i]); }

/* ---------------------------------------------------------------- canonical exp
 * The reference calls an approximate exp (`expf<afn>`, kernels/prepare_gated_i8.loom:99,
 * kernels/gemm_i8_swiglu_256.loom:650) whose bits depend on its compiler and GPU.
 * The canonical replacement: Cody-Waite reduction by ln2 in two pieces and the
 * classic degree-6 minimax polynomial (the published Cephes expf), every step a
 * single f32 operation or a fused multiply-add, so that a CPU and a GPU produce the
 * same bits.  Accurate to about 1 ulp; callers round the result to bf16 right away.
 * The quotient 1/(1+e) that follows is a correctly rounded reciprocal. */
float oracle_exp(float x) {
    /* Clamped, not branched: above 89 the scaled result overflows to +inf by itself, below
     * -104 it underflows to zero or the smallest subnormal; a NaN passes through. */
    float xc = fminf(fmaxf(x, -104.0f), 89.0f);
    float t = xc * 1.44269502162933349609375f;
    float n = rintf(t);
    float r = fmaf(n, -0.693359375f, xc);
    r = fmaf(n, 2.12194440e-4f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float r2 = r * r;
    float y = fmaf(p, r2, r);
    y = y + 1.0f;
    int ni = (int)n;
    int h1 = ni >> 1, h2 = ni - h1; /* floor(n/2) and the rest: both exponents stay in range */
    float a = bits_f32((uint32_t)(h1 + 127) << 23);
    float b = bits_f32((uint32_t)(h2 + 127) << 23);
    float result = (y * a) * b;
    return x != x ? x : result;
}

/* sigma(g) = 1 / (1 + exp(0 - g)) in f32, unrounded (kernels/prepare_gated_i8.loom:98-101). */
static inline float sigmoid_f32(float g) {
    float neg = 0.0f - g;
    float e = oracle_exp(neg);
    float den = 1.0f + e;
    return 1.0f / den;
}

/* ---------------------------------------------------------------- Hadamard
 * One radix-4 butterfly (kernels/prepare_norm_i8.loom:194-201): every line is one f32 op. */
static inline void butterfly(float e0, float e1, float e2, float e3, float *o) {
    float s01 = e0 + e1, s23 = e2 + e3, d01 = e0 - e1, d23 = e2 - e3;
    o[0] = s01 + d23;
    o[1] = s01 - d23;
    o[2] = d01 + s23;
    o[3] = s23 - d01;
}

/* Four stages of strides 1, 4, 16, 64 inside every aligned 256-group, f32 throughout,
 * unnormalised (kernels/prepare_norm_i8.loom:174-309). */
static void hadamard256_f32(float *x, size_t width) {
    for (size_t s = 1; s <= 64; s *= 4)
        for (size_t block = 0; block < width; block += 4 * s)
            for (size_t c = 0; c < s; c++) {
                float o[4];
                float *p = x + block + c;
                butterfly(p[0], p[s], p[2 * s], p[3 * s], o);
                p[0] = o[0]; p[s] = o[1]; p[2 * s] = o[2]; p[3 * s] = o[3];
            }
}

/* The plain prologue's rotation: the same butterflies, but each stage's result is
 * multiplied by 1/4 and rounded to f16 (kernels/prepare_plain_i8.loom:112-167 for
 * strides 1 and 4, :213-232 and :259-278 for strides 16 and 64). */
static void hadamard256_f16(float *x, size_t width) {
    for (size_t s = 1; s <= 64; s *= 4)
        for (size_t block = 0; block < width; block += 4 * s)
            for (size_t c = 0; c < s; c++) {
                float o[4];
                float *p = x + block + c;
                butterfly(p[0], p[s], p[2 * s], p[3 * s], o);
                p[0] = hf(o[0] * 0.25f); p[s] = hf(o[1] * 0.25f);
                p[2 * s] = hf(o[2] * 0.25f); p[3 * s] = hf(o[3] * 0.25f);
            }
}

/* absmax -> scale -> codes (kernels/prepare_norm_i8.loom:312-372, prepare_plain_i8.loom:283-346).
 * `rotation` is 1/16 for the f32 rotation and 16 for the f16 one.  Only the first
 * `width` bytes of the output row are written. */
static void quantise_row(const float *x, size_t width, float rotation, int8_t *q, float *q_scale) {
    float amax = 0.0f;
    for (size_t i = 0; i < width; i++) amax = fmaxf(amax, fabsf(x[i]));
    float row_max = amax * rotation;
    float safe = fmaxf(row_max, 1.0000000000000001e-30f);
    float s = safe / 127.0f;
    float inv = rotation / s;
    for (size_t i = 0; i < width; i++) {
        float r = x[i] * inv;
        float f = rintf(r);
        f = fmaxf(f, -127.0f);
        f = fminf(f, 127.0f);
        q[i] = (int8_t)(int32_t)f;
    }
    *q_scale = s;
}

/* ---------------------------------------------------------------- prologues */

/* kernels/prepare_norm_i8.loom:18-374.
 * Sum of squares (:90-138): lane l of 256 owns chunks j*256+l of 8 elements and keeps
 * an 8-wide accumulator added to in j order.  Canonical choices for the two orders
 * the reference leaves open: the 8-wide accumulator folds as
 * ((a0+a1)+(a2+a3))+((a4+a5)+(a6+a7)); the 32 lanes of a wave fold by the xor
 * butterfly 16, 8, 4, 2, 1.  The eight wave sums combine as the reference writes:
 * ((p0+p4)+(p2+p6)) + ((p1+p5)+(p3+p7)).  rsqrt is 1/sqrt, both correctly rounded. */
/* The front half of prepare_norm_i8 for one row: RMSNorm with `1 + norm_scale`, then adaLN, every product and the
 * sum rounded to bf16 (kernels/prepare_norm_i8.loom:120-172); x receives the bf16 values as f32. */
static void norm_modulate_row(const uint16_t *row, const float *norm_scale, const float *mod_scale,
                              const float *mod_shift, float *x, size_t width, float eps) {
    size_t chunks_per_lane = width / 2048;
    float lane_sum[256];
    for (size_t l = 0; l < 256; l++) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (size_t j = 0; j < chunks_per_lane; j++) {
            const uint16_t *c = row + (j * 256 + l) * 8;
            for (int e = 0; e < 8; e++) {
                float v = bf16_to_f32(c[e]);
                float sq = v * v;
                acc[e] = acc[e] + sq;
            }
        }
        lane_sum[l] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
    }
    float p[8];
    for (size_t w = 0; w < 8; w++) {
        float v[32], n[32];
        memcpy(v, lane_sum + w * 32, sizeof v);
        for (int off = 16; off >= 1; off >>= 1) {
            for (int i = 0; i < 32; i++) n[i] = v[i] + v[i ^ off];
            memcpy(v, n, sizeof v);
        }
        p[w] = v[0];
    }
    float total = ((p[0] + p[4]) + (p[2] + p[6])) + ((p[1] + p[5]) + (p[3] + p[7]));
    float mean = total / (float)(int32_t)width;
    float mean_eps = mean + eps;
    float rinv = 1.0f / sqrtf(mean_eps);
    for (size_t i = 0; i < width; i++) {
        float v = bf16_to_f32(row[i]);
        float n = v * rinv;
        float ns1 = norm_scale[i] + 1.0f;
        float normed = bf(n * ns1);
        float ms1 = bf(mod_scale[i] + 1.0f);
        float scaled = bf(normed * ms1);
        x[i] = bf(scaled + mod_shift[i]);
    }
}

/* The same for `tokens` rows, as bf16 bits: what the Hadamard rotation of prepare_norm_i8 receives.  Test
 * infrastructure for holding that stage to the reference's torch statement of it. */
void oracle_norm_modulate(size_t tokens, const uint16_t *h, const float *norm_scale, const float *mod_scale,
                          const float *mod_shift, uint16_t *out, size_t width, float eps) {
    float *x = (float *)malloc(width * sizeof(float));
    for (size_t t = 0; t < tokens; t++) {
        norm_modulate_row(h + t * width, norm_scale, mod_scale, mod_shift, x, width, eps);
        for (size_t i = 0; i < width; i++) out[t * width + i] = f32_to_bf16(x[i]);
    }
    free(x);
}

void oracle_prepare_norm_i8(size_t tokens, const uint16_t *h, const float *norm_scale,
                            const float *mod_scale, const float *mod_shift, int8_t *q,
                            float *q_scale, size_t width, size_t out_stride, float eps) {
    float *x = (float *)malloc(width * sizeof(float));
    for (size_t t = 0; t < tokens; t++) {
        norm_modulate_row(h + t * width, norm_scale, mod_scale, mod_shift, x, width, eps);
        hadamard256_f32(x, width);
        quantise_row(x, width, 0.0625f, q + t * out_stride, q_scale + t);
    }
    free(x);
}

/* kernels/prepare_gated_i8.loom:18-313: a = bf16(attn), sigma = bf16(1/(1+exp(-g))),
 * o = bf16(a*sigma) (:86-108), then the f32 rotation and quantisation of the norm kernel. */
/* The front half of prepare_gated_i8 for one row: the attention output times the sigmoid of the gate, the
 * sigmoid and the product rounded to bf16 (kernels/prepare_gated_i8.loom:86-108). */
static void gate_row(const uint16_t *attn, const uint16_t *gate, float *x, size_t width) {
    for (size_t i = 0; i < width; i++) {
        float a = bf(f16_to_f32(attn[i]));
        float g = f16_to_f32(gate[i]);
        float sig = bf(sigmoid_f32(g));
        x[i] = bf(a * sig);
    }
}

/* The same for `tokens` rows, as bf16 bits: what the Hadamard rotation of prepare_gated_i8 receives.  Test
 * infrastructure for holding that stage to the reference's torch statement of it. */
void oracle_gate_attention(size_t tokens, const uint16_t *attn, const uint16_t *gate, uint16_t *out, size_t width,
                           size_t gate_stride) {
    float *x = (float *)malloc(width * sizeof(float));
    for (size_t t = 0; t < tokens; t++) {
        gate_row(attn + t * width, gate + t * gate_stride, x, width);
        for (size_t i = 0; i < width; i++) out[t * width + i] = f32_to_bf16(x[i]);
    }
    free(x);
}

void oracle_prepare_gated_i8(size_t tokens, const uint16_t *attn, const uint16_t *gate, int8_t *q,
                             float *q_scale, size_t width, size_t out_stride, size_t gate_stride) {
    float *x = (float *)malloc(width * sizeof(float));
    for (size_t t = 0; t < tokens; t++) {
        gate_row(attn + t * width, gate + t * gate_stride, x, width);
        hadamard256_f32(x, width);
        quantise_row(x, width, 0.0625f, q + t * out_stride, q_scale + t);
    }
    free(x);
}

/* kernels/prepare_plain_i8.loom:15-348. */
void oracle_prepare_plain_i8(size_t tokens, const uint16_t *h, int8_t *q, float *q_scale,
                             size_t width, size_t out_stride) {
    float *x = (float *)malloc(width * sizeof(float));
    for (size_t t = 0; t < tokens; t++) {
        for (size_t i = 0; i < width; i++) x[i] = f16_to_f32(h[t * width + i]);
        hadamard256_f16(x, width);
        quantise_row(x, width, 16.0f, q + t * out_stride, q_scale + t);
    }
    free(x);
}

/* ---------------------------------------------------------------- GEMM core
 * acc[m][n] = sum_k a[m][k] * w[n][k] in i32, exact (kernels/gemm_i8_256.loom:261-556).
 * Bytes k_size..k_stride of a row are never read. */
void oracle_gemm_i8_acc(size_t m, const int8_t *a, const int8_t *w, int32_t *acc, size_t k_size,
                        size_t k_stride, size_t n_size) {
    /* Integer sums are exact in any order, so the loop nest is free: two rows by four columns per pass over
     * k keep eight independent sums going and reuse every loaded byte four or two times. */
#pragma omp parallel for schedule(static)
    for (ptrdiff_t nb = 0; nb < (ptrdiff_t)n_size; nb += 16) {
        const size_t n_end = (size_t)nb + 16 < n_size ? (size_t)nb + 16 : n_size;
        size_t r = 0;
        for (; r + 2 <= m; r += 2) {
            const int8_t *a0 = a + r * k_stride, *a1 = a0 + k_stride;
            size_t n = (size_t)nb;
            for (; n + 4 <= n_end; n += 4) {
                const int8_t *w0 = w + n * k_stride, *w1 = w0 + k_stride, *w2 = w1 + k_stride, *w3 = w2 + k_stride;
                int32_t s00 = 0, s01 = 0, s02 = 0, s03 = 0, s10 = 0, s11 = 0, s12 = 0, s13 = 0;
                for (size_t k = 0; k < k_size; k++) {
                    const int32_t x0 = a0[k], x1 = a1[k], y0 = w0[k], y1 = w1[k], y2 = w2[k], y3 = w3[k];
                    s00 += x0 * y0, s01 += x0 * y1, s02 += x0 * y2, s03 += x0 * y3;
                    s10 += x1 * y0, s11 += x1 * y1, s12 += x1 * y2, s13 += x1 * y3;
                }
                int32_t *o0 = acc + r * n_size + n, *o1 = o0 + n_size;
                o0[0] = s00, o0[1] = s01, o0[2] = s02, o0[3] = s03;
                o1[0] = s10, o1[1] = s11, o1[2] = s12, o1[3] = s13;
            }
            for (; n < n_end; n++) {
                const int8_t *wr = w + n * k_stride;
                int32_t s0 = 0, s1 = 0;
                for (size_t k = 0; k < k_size; k++) s0 += (int32_t)a0[k] * wr[k], s1 += (int32_t)a1[k] * wr[k];
                acc[r * n_size + n] = s0, acc[(r + 1) * n_size + n] = s1;
            }
        }
        for (; r < m; r++) {
            const int8_t *ar = a + r * k_stride;
            for (size_t n = (size_t)nb; n < n_end; n++) {
                const int8_t *wr = w + n * k_stride;
                int32_t s = 0;
                for (size_t k = 0; k < k_size; k++) s += (int32_t)ar[k] * (int32_t)wr[k];
                acc[r * n_size + n] = s;
            }
        }
    }
}

/* lin = bf16((f32(acc) * ws[n]) * as[m])  (kernels/gemm_i8_256.loom:610-620). */
static inline float dequant(int32_t acc, float ws, float as) {
    float f = (float)acc;
    float s0 = f * ws;
    return bf(s0 * as);
}

/* Plain epilogue: C = f16(lin) (kernels/gemm_i8_256.loom:558-628). */
void oracle_epilogue_plain(size_t m, const int32_t *acc, const float *scale, const float *a_scale,
                           uint16_t *c, size_t n_size) {
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)m; r++)
        for (size_t n = 0; n < n_size; n++)
            c[r * n_size + n] = f32_to_f16(dequant(acc[r * n_size + n], scale[n], a_scale[r]));
}

/* Residual epilogue, in place on bf16 x: x = bf16(x + bf16(lin * gate[n]))
 * (kernels/gemm_i8_resid_256.loom:613-635; the 256x256 sibling is identical, :394-475). */
void oracle_epilogue_resid(size_t m, const int32_t *acc, const float *scale, const float *a_scale,
                           uint16_t *c, const float *gate, size_t n_size) {
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)m; r++)
        for (size_t n = 0; n < n_size; n++) {
            float lin = dequant(acc[r * n_size + n], scale[n], a_scale[r]);
            float gated = bf(lin * gate[n]);
            float prior = bf16_to_f32(c[r * n_size + n]);
            c[r * n_size + n] = f32_to_bf16(prior + gated);
        }
}

/* SwiGLU epilogue over 16-row interleaved gate|up columns: output o takes gate column
 * 32*(o/16) + o%16 and up column 16 further; C = f16(bf16(bf16(g*sigma(g)) * u)),
 * sigma unrounded f32 (kernels/gemm_i8_swiglu_256.loom:612-660). */
void oracle_epilogue_swiglu(size_t m, const int32_t *acc, const float *scale, const float *a_scale,
                            uint16_t *c, size_t n_size) {
    size_t half = n_size / 2;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t r = 0; r < (ptrdiff_t)m; r++)
        for (size_t o = 0; o < half; o++) {
            size_t gc = 32 * (o / 16) + (o % 16), uc = gc + 16;
            float g = dequant(acc[r * n_size + gc], scale[gc], a_scale[r]);
            float u = dequant(acc[r * n_size + uc], scale[uc], a_scale[r]);
            float silu = bf(g * sigmoid_f32(g));
            c[r * half + o] = f32_to_f16(bf(silu * u));
        }
}

/* The four kernels as the reference exports them (binding order of each launch(...)). */
void oracle_gemm_i8_256(size_t m, const int8_t *a, const int8_t *w, const float *scale,
                        const float *a_scale, uint16_t *c, size_t k_size, size_t k_stride, size_t n_size) {
    int32_t *acc = (int32_t *)malloc(m * n_size * sizeof(int32_t));
    oracle_gemm_i8_acc(m, a, w, acc, k_size, k_stride, n_size);
    oracle_epilogue_plain(m, acc, scale, a_scale, c, n_size);
    free(acc);
}
void oracle_gemm_i8_resid_256(size_t m, const int8_t *a, const int8_t *w, const float *scale,
                              const float *a_scale, uint16_t *c, const float *gate, size_t k_size,
                              size_t k_stride, size_t n_size) {
    int32_t *acc = (int32_t *)malloc(m * n_size * sizeof(int32_t));
    oracle_gemm_i8_acc(m, a, w, acc, k_size, k_stride, n_size);
    oracle_epilogue_resid(m, acc, scale, a_scale, c, gate, n_size);
    free(acc);
}
void oracle_gemm_i8_swiglu_256(size_t m, const int8_t *a, const int8_t *w, const float *scale,
                               const float *a_scale, uint16_t *c, size_t k_size, size_t k_stride, size_t n_size) {
    int32_t *acc = (int32_t *)malloc(m * n_size * sizeof(int32_t));
    oracle_gemm_i8_acc(m, a, w, acc, k_size, k_stride, n_size);
    oracle_epilogue_swiglu(m, acc, scale, a_scale, c, n_size);
    free(acc);
}

/* f16 <-> bf16 transport of src/training/quantized.rs:63-72,102-110 (`lora_transport`
 * reverse=1: bf16 -> f16, reverse=2: f16 -> bf16), value-preserving where representable. */
void oracle_transport_bf16_to_f16(const uint16_t *src, uint16_t *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = f32_to_f16(bf16_to_f32(src[i]));
}
void oracle_transport_f16_to_bf16(const uint16_t *src, uint16_t *dst, size_t n) {
    for (size_t i = 0; i < n; i++) dst[i] = f32_to_bf16(f16_to_f32(src[i]));
}

/* Sets the number of OpenMP threads later calls use, whatever OMP_NUM_THREADS said at load time
 * (a launcher such as torchrun exports OMP_NUM_THREADS=1 to its ranks). */
void oracle_set_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int oracle_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------- the rest of a block
 * Not W8A8 products; restated so that the session's full block can be checked. */

/* kernels/rope_qknorm_f16.loom:78-157.  Canonical orders for the two sums the reference leaves
 * open: four squares per lane fold as (s0+s1)+(s2+s3), the 32 lanes by xor butterfly 16..1. */
void oracle_rope_qknorm_f16(size_t tokens, const uint16_t *qkv, const float *q_scale, const float *k_scale,
                            const float *cos_table, const float *sin_table, uint16_t *q_out, uint16_t *k_out,
                            uint16_t *v_out, size_t row_stride, size_t q_heads, size_t kv_heads, size_t k_offset,
                            float eps) {
    for (size_t t = 0; t < tokens; t++) {
        const uint16_t *row = qkv + t * row_stride;
        memcpy(v_out + t * kv_heads * 128, row + k_offset + kv_heads * 128, kv_heads * 128 * 2);
        for (size_t head = 0; head < q_heads + kv_heads; head++) {
            int is_q = head < q_heads;
            const uint16_t *h = row + (is_q ? head * 128 : k_offset + (head - q_heads) * 128);
            const float *scale = is_q ? q_scale : k_scale;
            float v[128], lane[32], next[32], x[128];
            for (int c = 0; c < 128; c++) v[c] = f16_to_f32(h[c]);
            for (int l = 0; l < 32; l++) {
                float s0 = v[4 * l] * v[4 * l], s1 = v[4 * l + 1] * v[4 * l + 1];
                float s2 = v[4 * l + 2] * v[4 * l + 2], s3 = v[4 * l + 3] * v[4 * l + 3];
                lane[l] = (s0 + s1) + (s2 + s3);
            }
            for (int off = 16; off >= 1; off >>= 1) {
                for (int l = 0; l < 32; l++) next[l] = lane[l] + lane[l ^ off];
                memcpy(lane, next, sizeof lane);
            }
            float mean = lane[0] * 0.0078125f;
            float rinv = 1.0f / sqrtf(mean + eps);
            for (int c = 0; c < 128; c++) {
                float normed = v[c] * rinv;
                x[c] = bf(normed * (scale[c] + 1.0f));
            }
            uint16_t *dst = is_q ? q_out + t * q_heads * 128 + head * 128 : k_out + t * kv_heads * 128 + (head - q_heads) * 128;
            for (int c = 0; c < 128; c++) {
                float rot = (c % 2 == 0) ? (0.0f - x[c + 1]) : x[c - 1];
                float xc = x[c] * cos_table[t * 128 + c];
                float rs = rot * sin_table[t * 128 + c];
                dst[c] = f32_to_f16(bf(xc + rs));
            }
        }
    }
}

/* kernels/native/v_transpose.loom: x [rows][width] -> out [width][capacity]; inside the last 32-row
 * tile the columns past `rows` are written as zero, everything further right is left alone. */
void oracle_v_transpose(size_t rows, const uint16_t *x, uint16_t *out, size_t width, size_t capacity) {
    size_t padded = (rows + 31) / 32 * 32;
    if (padded > capacity) padded = capacity;
    for (size_t c = 0; c < width; c++)
        for (size_t r = 0; r < padded; r++) out[c * capacity + r] = r < rows ? x[r * width + c] : 0;
}

/* Grouped-query attention in f64 (the CPU softmax the reference's own test compares with,
 * tests/quantized.rs:314-338): a tolerance reference, not a bit reference. */
void oracle_attention_gqa(size_t queries, size_t tokens, size_t q_heads, size_t kv_heads, const uint16_t *q,
                          const uint16_t *k, const uint16_t *v, double *out, double scale) {
    size_t group = q_heads / kv_heads;
#pragma omp parallel for schedule(dynamic) collapse(2)
    for (ptrdiff_t t = 0; t < (ptrdiff_t)queries; t++)
        for (ptrdiff_t head = 0; head < (ptrdiff_t)q_heads; head++) {
            size_t kvh = (size_t)head / group;
            double *scores = (double *)malloc(tokens * sizeof(double));
            double qv[128], mx = -INFINITY, sum = 0.0, acc[128];
            for (int c = 0; c < 128; c++) qv[c] = f16_to_f32(q[((size_t)t * q_heads + head) * 128 + c]), acc[c] = 0.0;
            for (size_t j = 0; j < tokens; j++) {
                double s = 0.0;
                for (int c = 0; c < 128; c++) s += qv[c] * f16_to_f32(k[(j * kv_heads + kvh) * 128 + c]);
                scores[j] = s * scale;
                if (scores[j] > mx) mx = scores[j];
            }
            for (size_t j = 0; j < tokens; j++) {
                double w = exp(scores[j] - mx);
                sum += w;
                for (int c = 0; c < 128; c++) acc[c] += w * f16_to_f32(v[(j * kv_heads + kvh) * 128 + c]);
            }
            for (int c = 0; c < 128; c++) out[((size_t)t * q_heads + head) * 128 + c] = acc[c] / sum;
            free(scores);
        }
}

/* ---------------------------------------------------------------- the outer step
 * The three pointwise kernels around the block chain and the sigma schedule.  All
 * pinned: the reference tests state euler and guidance exactly (tests/arithmetic.rs:38-84)
 * and hold the schedule to recorded scheduler bits (tests/schedule.rs). */

/* kernels/native/modulation.loom:30-43: y[i] = bf16(x[i % xsize] + tables[i]) widened to f32. */
void oracle_modulation(size_t count, const uint16_t *x, const uint16_t *tables, float *y, size_t xsize) {
    for (size_t i = 0; i < count; i++) y[i] = bf(bf16_to_f32(x[i % xsize]) + bf16_to_f32(tables[i]));
}

/* kernels/native/euler.loom:28-41: sample = bf16(sample + bf16(bf16(delta) * velocity)). */
void oracle_euler(size_t count, float delta, uint16_t *sample, const uint16_t *velocity) {
    const float dt = bf(delta);
    for (size_t i = 0; i < count; i++) {
        float product = bf(dt * bf16_to_f32(velocity[i]));
        sample[i] = f32_to_bf16(bf16_to_f32(sample[i]) + product);
    }
}

/* kernels/native/guidance.loom:28-43: cond = bf16(cond + bf16(scale * bf16(cond - uncond))). */
void oracle_guidance(size_t count, float scale, uint16_t *cond, const uint16_t *uncond) {
    for (size_t i = 0; i < count; i++) {
        float c = bf16_to_f32(cond[i]);
        float difference = bf(c - bf16_to_f32(uncond[i]));
        cond[i] = f32_to_bf16(c + bf(scale * difference));
    }
}

/* src/pipeline/schedule.rs:11-14 */
double oracle_dynamic_mu(size_t image_tokens) {
    double slope = (1.15 - 0.5) / (6400.0 - 256.0);
    return (double)image_tokens * slope + (0.5 - slope * 256.0);
}

/* src/pipeline/schedule.rs:17-27: the linspace value in f32, exp(mu) in double then f32. */
float oracle_sigma(size_t step, size_t steps, double mu) {
    if (step == steps) return 0.0f;
    float raw = (float)(1.0 - (double)step / (double)steps);
    float shift = (float)exp(mu);
    float offset = 1.0f / raw - 1.0f;
    return shift / (shift + offset);
}

/* src/pipeline/schedule.rs:33-35 */
float oracle_next_sigma(size_t step, size_t last, size_t steps, double mu) {
    return step + 1 >= last ? 0.0f : oracle_sigma(step + 1, steps, mu);
}
