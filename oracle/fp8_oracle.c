/*
 * TEST INFRASTRUCTURE ONLY -- CPU oracle for the FP8 fine-grained-scaled GEMM path.
 *
 * PARITY UNPINNED: the reference (zoheth/yan) ships no finished FP8 GEMM, no
 * quantizer, no torch reference and no golden vectors for this path
 * (yan/jit_kernels/gemm.py:1-31 is a template string only;
 * yan/include/gemm/fp8_gemm.cuh:187-197 stops mid-statement).  This file restates
 * the arithmetic that the reference's fragments and the workload definition fix:
 *
 *   - operand granularity and layouts: A scales are one fp32 per (row, 128-wide
 *     k-block), consumed M-contiguous per k-block
 *     (yan/include/gemm/fp8_gemm.cuh:59 `SMEM_SCALES_A_SIZE_PER_STAGE = BLOCK_M*4`,
 *     yan/jit_kernels/gemm.py:25 `make_2d_tma_scales_a_desc(lhs_scales, m)`);
 *     B scales are one fp32 per 128x128 block, [N/128, K/128] row-major
 *     (yan/include/gemm/fp8_gemm.cuh:41,55,60-61);
 *     B is [N, K] K-major ("NT"), D is [M, N] bf16 (fp8_gemm.cuh:56,87).
 *   - arithmetic: scale = amax/448, e4m3 round-to-nearest-even, fp32 accumulation,
 *     bf16 output (the CPU-runnable configuration of the workload list).
 *
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may load
 * this file; the product path never does.
 *
 * Build: see oracle/Makefile  (gcc -O2 -fno-fast-math -ffp-contract=off).
 * No FMA contraction and no fast-math: every operation below is one IEEE fp32
 * round-to-nearest operation, which is what the CUDA kernels reproduce with
 * __fdiv_rn / __fmul_rn.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GROUP 128

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* fp32 -> bf16, round-to-nearest-even; NaN stays NaN. */
static inline uint16_t f32_to_bf16_rne(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* e4m3fn (1-4-3, bias 7, no inf, 0x7f/0xff = NaN, max 448) -> fp32. */
float yan_oracle_e4m3_decode(uint8_t c) {
    uint32_t s = (c >> 7) & 1u, e = (c >> 3) & 0xfu, m = c & 7u;
    float v;
    if (e == 0xf && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m, -9);           /* subnormal: m * 2^-9 */
    else        v = ldexpf(1.0f + (float)m / 8.0f, (int)e - 7);
    return s ? -v : v;
}

/*
 * fp32 -> e4m3fn, round-to-nearest-even.
 * saturate != 0 : results beyond 448 clamp to 448 (the CUDA cvt.rn.satfinite form).
 * saturate == 0 : results that round beyond 448 become NaN (torch CPU semantics:
 *                 464 -> 448 because the tie goes to the even mantissa, 465 -> NaN).
 * The pinned quantizer never produces |v| > 448*(1+2^-23), so both agree on its inputs.
 */
uint8_t yan_oracle_e4m3_encode(float f, int saturate) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(sign | 0x7f);              /* NaN */
    if (a == 0x7f800000u) return (uint8_t)(sign | (saturate ? 0x7e : 0x7f));
    float af;
    memcpy(&af, &a, 4);
    if (af < 0.015625f) {                                             /* below 2^-6: subnormal grid of 2^-9 */
        float q = nearbyintf(af * 512.0f);                            /* exact scaling, RNE (default mode) */
        return (uint8_t)(sign | (uint8_t)q);                          /* q == 8 is the first normal code 0x08 */
    }
    int32_t exp = (int32_t)(a >> 23) - 127;
    uint32_t mant = a & 0x7fffffu;
    uint32_t lsb = (mant >> 20) & 1u;
    mant += 0x7ffffu + lsb;                                           /* RNE to 3 mantissa bits */
    if (mant & 0x800000u) { mant = 0; exp += 1; }
    uint32_t m3 = mant >> 20;
    if (exp > 8 || (exp == 8 && m3 == 7)) return (uint8_t)(sign | (saturate ? 0x7e : 0x7f));
    return (uint8_t)(sign | ((uint32_t)(exp + 7) << 3) | m3);
}

/*
 * Per-token-group activation quantizer (1 x 128 groups).
 *   a      : [M, K] bf16 bits, row-major, K % 128 == 0
 *   q      : [M, K] e4m3 codes
 *   scales : K-block-major, scales[kb * M + m]   (M contiguous per k-block: the
 *            layout the GEMM consumes, fp8_gemm.cuh:59)
 * Pinned operation sequence per group (each one fp32 RN op):
 *   amax  = max |x|;  amax_c = max(amax, 1e-4f)
 *   inv   = 448.0f / amax_c
 *   q     = e4m3_rne(x * inv)
 *   scale = amax_c / 448.0f
 */
void yan_oracle_per_token_cast_to_fp8(const uint16_t *a, int64_t M, int64_t K,
                                      uint8_t *q, float *scales) {
    int64_t KB = K / GROUP;
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t kb = 0; kb < KB; ++kb) {
            const uint16_t *src = a + m * K + kb * GROUP;
            float amax = 0.0f;
            for (int i = 0; i < GROUP; ++i) {
                float v = fabsf(bf16_to_f32(src[i]));
                if (v > amax) amax = v;
            }
            float amax_c = amax > 1e-4f ? amax : 1e-4f;
            volatile float inv = 448.0f / amax_c;
            for (int i = 0; i < GROUP; ++i) {
                volatile float p = bf16_to_f32(src[i]) * inv;
                q[m * K + kb * GROUP + i] = yan_oracle_e4m3_encode(p, 1);
            }
            scales[kb * M + m] = amax_c / 448.0f;
        }
    }
}

/*
 * Per-block weight quantizer (128 x 128 blocks).  b: [N, K] bf16 bits; N, K % 128 == 0.
 * scales: [N/128, K/128] row-major.  Same operation sequence as above with the
 * amax taken over the whole block.
 */
void yan_oracle_per_block_cast_to_fp8(const uint16_t *b, int64_t N, int64_t K,
                                      uint8_t *q, float *scales) {
    int64_t NB = N / GROUP, KB = K / GROUP;
    for (int64_t nb = 0; nb < NB; ++nb) {
        for (int64_t kb = 0; kb < KB; ++kb) {
            float amax = 0.0f;
            for (int r = 0; r < GROUP; ++r)
                for (int c = 0; c < GROUP; ++c) {
                    float v = fabsf(bf16_to_f32(b[(nb * GROUP + r) * K + kb * GROUP + c]));
                    if (v > amax) amax = v;
                }
            float amax_c = amax > 1e-4f ? amax : 1e-4f;
            volatile float inv = 448.0f / amax_c;
            for (int r = 0; r < GROUP; ++r)
                for (int c = 0; c < GROUP; ++c) {
                    int64_t idx = (nb * GROUP + r) * K + kb * GROUP + c;
                    volatile float p = bf16_to_f32(b[idx]) * inv;
                    q[idx] = yan_oracle_e4m3_encode(p, 1);
                }
            scales[nb * KB + kb] = amax_c / 448.0f;
        }
    }
}

/*
 * Reference GEMM: D = bf16( dequant(A) . dequant(B)^T ), fp32 accumulation.
 *   qa [M,K] e4m3, sa K-block-major [K/128][M];  qb [N,K] e4m3, sb [N/128][K/128]
 *   d  [M,N] bf16 bits, row stride ldd elements.
 * Dequantized values are fp32(code) * scale (one RN multiply); the dot product is a
 * plain left-to-right fp32 sum over k (no FMA contraction).  The GPU kernel sums in
 * a different order, so D is compared with a tolerance, never bit-for-bit.
 */
void yan_oracle_ref_gemm(const uint8_t *qa, const float *sa, const uint8_t *qb, const float *sb,
                         int64_t M, int64_t N, int64_t K, uint16_t *d, int64_t ldd) {
    int64_t KB = K / GROUP;
    float lut[256];
    for (int i = 0; i < 256; ++i) lut[i] = yan_oracle_e4m3_decode((uint8_t)i);
    for (int64_t m = 0; m < M; ++m) {
        float *da = (float *)malloc((size_t)K * sizeof(float));
        for (int64_t k = 0; k < K; ++k) {
            volatile float t = lut[qa[m * K + k]] * sa[(k / GROUP) * M + m];
            da[k] = t;
        }
        for (int64_t n = 0; n < N; ++n) {
            float sum = 0.0f;
            for (int64_t k = 0; k < K; ++k) {
                volatile float db = lut[qb[n * K + k]] * sb[(n / GROUP) * KB + k / GROUP];
                volatile float p = da[k] * db;
                sum = sum + p;
            }
            d[m * ldd + n] = f32_to_bf16_rne(sum);
        }
        free(da);
    }
}

/* Dequantize helpers used by tests that want the fp32 operands themselves. */
void yan_oracle_dequant_a(const uint8_t *qa, const float *sa, int64_t M, int64_t K, float *out) {
    int64_t KB = K / GROUP;
    for (int64_t m = 0; m < M; ++m)
        for (int64_t k = 0; k < K; ++k) {
            volatile float t = yan_oracle_e4m3_decode(qa[m * K + k]) * sa[(k / GROUP) * M + m];
            out[m * K + k] = t;
        }
    (void)KB;
}

void yan_oracle_dequant_b(const uint8_t *qb, const float *sb, int64_t N, int64_t K, float *out) {
    int64_t KB = K / GROUP;
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) {
            volatile float t = yan_oracle_e4m3_decode(qb[n * K + k]) * sb[(n / GROUP) * KB + k / GROUP];
            out[n * K + k] = t;
        }
}

void yan_oracle_f32_to_bf16(const float *in, int64_t n, uint16_t *out) {
    for (int64_t i = 0; i < n; ++i) out[i] = f32_to_bf16_rne(in[i]);
}
