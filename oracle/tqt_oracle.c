/*
 * CPU oracle for the quantized GEMM micro-kernel path of TORQ-Tile.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic the
 * reference defines for the path, so that the CUDA kernels can be compared with it
 * on identical inputs.  Nothing in the shipped library links, loads or calls it;
 * only the test-suite, the smoke check and the benchmark's CPU-baseline leg do.
 *
 * Parity status of each function ("pinned" = checked against code of the reference
 * compiled from its own sources, see ref_shim.cpp and tests/test_oracle_pins.py):
 *   tqo_gemm_clamp_i32_i8_i8        pinned  (reference_gemm_i32_i8)
 *   tqo_gemm_w4a16                   pinned  (reference_gemm_quantized_weight_mixed)
 *   tqo_quantize_fp16_to_int4        pinned  (quantize_fp16_to_int4)
 *   tqo_quantize_multiplier          pinned  (tqt_quantize_multiplier, incl. the known
 *                                            answer 0.0025 -> (1374389535, -8))
 *   tqo_quantize_i8 / fuse_zp        pinned  (quantize_i8, fuse_zp_to_bias)
 *   f32<->f16/bf16 conversions       pinned  (g++ static_cast on _Float16 / __bf16)
 *   tqo_quantize_a_per_row_asym,
 *   tqo_quantize_b_per_channel_sym_int4,
 *   tqo_gemm_w4a8                    restated from a gtest translation unit that cannot
 *                                    be compiled off RISC-V; integer core pinned through
 *                                    reference_gemm_i32_i8 on the unpacked nibbles,
 *                                    per-element quantiser pinned through quantize_i8.
 *   tqo_gemm_reqi32toi8              restated from RVV instruction semantics; no C
 *                                    version exists in the reference.  Multiplier pinned;
 *                                    the integer tail (mulh / sra / add / two saturating
 *                                    narrows / clamp) is "parity unpinned" beyond the
 *                                    reference's own +-1 LSB dequantised tolerance.
 *
 * Build: see oracle/Makefile (gcc -O3 -ffp-contract=off [-fopenmp]).
 * -ffp-contract=off matters: the reference's epilogues are separate multiply and add
 * instructions, never fused.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define TQO_TD_F32 0
#define TQO_TD_F16 1
#define TQO_TD_BF16 2

int tqo_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void tqo_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* 16-bit float conversions (round-to-nearest-even), bit-level.              */
/* They stand for static_cast<float16_t>/<bfloat16_t> in the reference's     */
/* portable code (src/common/tqt_common.h:27-28 typedefs __bf16/_Float16).   */
/* ------------------------------------------------------------------------- */
static inline uint32_t f32_bits(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}
static inline float bits_f32(uint32_t u)
{
    float f;
    memcpy(&f, &u, 4);
    return f;
}

uint16_t tqo_f32_to_bf16(float f)
{
    uint32_t u = f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) { /* NaN: keep quiet */
        return (uint16_t)((u >> 16) | 0x0040u);
    }
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

float tqo_bf16_to_f32(uint16_t h)
{
    return bits_f32((uint32_t)h << 16);
}

uint16_t tqo_f32_to_f16(float f)
{
    uint32_t u = f32_bits(f);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((a >> 13) & 0x3ffu)); /* NaN */
    if (a >= 0x477ff000u) {                     /* >= 65520 rounds to inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (a < 0x33000001u) {                      /* <= 2^-25: rounds to zero (tie at 2^-25 -> even = 0) */
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(a >> 23) - 127;
    uint32_t man = (a & 0x7fffffu) | 0x800000u; /* 24-bit significand */
    uint32_t shift;
    uint32_t base_exp;
    if (exp < -14) {                            /* subnormal half */
        shift = (uint32_t)(13 + (-14 - exp));
        base_exp = 0;
    } else {
        shift = 13;
        base_exp = (uint32_t)(exp + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    uint32_t out;
    if (base_exp == 0) {
        out = q;                                /* may carry into exponent 1: correct */
    } else {
        out = ((base_exp - 1) << 10) + q;       /* q includes the hidden bit (0x400) */
    }
    return (uint16_t)(sign | out);
}

float tqo_f16_to_f32(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    if (exp == 0) {
        if (man == 0) return bits_f32(sign);
        float v = (float)man * 5.9604644775390625e-8f; /* 2^-24 */
        return sign ? -v : v;
    }
    if (exp == 31) return bits_f32(sign | 0x7f800000u | (man << 13));
    return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

static inline float td_load(const void *p, size_t i, int td)
{
    switch (td) {
        case TQO_TD_F16: return tqo_f16_to_f32(((const uint16_t *)p)[i]);
        case TQO_TD_BF16: return tqo_bf16_to_f32(((const uint16_t *)p)[i]);
        default: return ((const float *)p)[i];
    }
}

static inline void td_store(void *p, size_t i, int td, float v)
{
    switch (td) {
        case TQO_TD_F16: ((uint16_t *)p)[i] = tqo_f32_to_f16(v); break;
        case TQO_TD_BF16: ((uint16_t *)p)[i] = tqo_f32_to_bf16(v); break;
        default: ((float *)p)[i] = v; break;
    }
}

/* ------------------------------------------------------------------------- */
/* gemm_clamp_i32_i8_i8: D = clamp(C + A*B).                                  */
/* Follows test/common/reference_gemm.cpp:92-129 (reference_gemm_i32_i8).     */
/* b_transposed != 0: B is [n,k] (ldb = row length); else B is [k,n].         */
/* ------------------------------------------------------------------------- */
void tqo_gemm_clamp_i32_i8_i8(size_t m, size_t n, size_t k, const int8_t *A, size_t lda,
                              const int8_t *B, size_t ldb, int b_transposed, const int32_t *C,
                              size_t ldc, int32_t *D, size_t ldd, int32_t clamp_min,
                              int32_t clamp_max)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            int32_t acc = 0;
            if (b_transposed) {
                const int8_t *a = A + i * lda;
                const int8_t *b = B + j * ldb;
                for (size_t p = 0; p < k; ++p) acc += (int32_t)a[p] * (int32_t)b[p];
            } else {
                for (size_t p = 0; p < k; ++p)
                    acc += (int32_t)A[i * lda + p] * (int32_t)B[p * ldb + j];
            }
            if (C) acc = (int32_t)((uint32_t)acc + (uint32_t)C[i * ldc + j]);
            if (acc < clamp_min) acc = clamp_min;
            if (acc > clamp_max) acc = clamp_max;
            D[i * ldd + j] = acc;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Scalar int8 quantiser: clamp(nearbyintf(val/scale) + zp, -128, 127).       */
/* Follows test/common/test_common.h:232-240 (quantize_i8).                   */
/* ------------------------------------------------------------------------- */
int8_t tqo_quantize_i8(float val, float scale, int32_t zp)
{
    float q = nearbyintf(val / scale) + (float)zp;
    if (q > 127.0f) q = 127.0f;
    if (q < -128.0f) q = -128.0f;
    return (int8_t)q;
}

/* fused[ch] = bias[ch] - zp * sum(data[ch, :]); test/common/test_common.h:280-290. */
void tqo_fuse_zp_to_bias(int32_t *fused, const int32_t *bias, const int8_t *data, int32_t zp,
                         size_t channels, size_t channel_size)
{
    for (size_t ch = 0; ch < channels; ++ch) {
        int32_t s = 0;
        for (size_t i = 0; i < channel_size; ++i) s += (int32_t)data[ch * channel_size + i];
        fused[ch] = bias[ch] - zp * s;
    }
}

/* ------------------------------------------------------------------------- */
/* qai8dx: dynamic per-row asymmetric int8 quantisation of activations.       */
/* Follows test/gemm/test_gemm_i8_i4_rvv.cpp:40-77 (quantize_a_per_row_asym). */
/* The input may be f32, f16 or bf16 (widened exactly to f32 first).          */
/* ------------------------------------------------------------------------- */
void tqo_quantize_a_per_row_asym(const void *A, int ta, size_t m, size_t k, size_t lda,
                                 int8_t *A_i8, size_t ldq, float *scale_a, int32_t *zp_a)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t row = 0; row < (ptrdiff_t)m; ++row) {
        float fmin = FLT_MAX;
        float fmax = -FLT_MAX;
        for (size_t i = 0; i < k; ++i) {
            float v = td_load(A, row * lda + i, ta);
            if (v < fmin) fmin = v;
            if (v > fmax) fmax = v;
        }
        fmax = fmax > 0.0f ? fmax : 0.0f;
        fmin = fmin < 0.0f ? fmin : 0.0f;
        float s = (fmax - fmin) / 255.0f;
        if (s == 0.0f) {
            scale_a[row] = 1.0f;
            zp_a[row] = 0;
            for (size_t i = 0; i < k; ++i) A_i8[row * ldq + i] = 0;
            continue;
        }
        float zp_tmp = -128.0f - fmin / s;
        int32_t zp = (int32_t)nearbyintf(zp_tmp);
        if (zp < -128) zp = -128;
        if (zp > 127) zp = 127;
        scale_a[row] = s;
        zp_a[row] = zp;
        for (size_t i = 0; i < k; ++i)
            A_i8[row * ldq + i] = tqo_quantize_i8(td_load(A, row * lda + i, ta), s, zp);
    }
}

/* ------------------------------------------------------------------------- */
/* qsi4cx: per-channel symmetric int4 weight quantisation, two nibbles/byte,  */
/* stored value = q + 8, low nibble = even k.                                 */
/* Follows test/gemm/test_gemm_i8_i4_rvv.cpp:82-118.                          */
/* ------------------------------------------------------------------------- */
void tqo_quantize_b_per_channel_sym_int4(const float *B, size_t n, size_t k, uint8_t *B_nib,
                                         float *scale_b)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t row = 0; row < (ptrdiff_t)n; ++row) {
        const float *r = B + row * k;
        float abs_max = 0.0f;
        for (size_t i = 0; i < k; ++i) {
            float v = fabsf(r[i]);
            if (v > abs_max) abs_max = v;
        }
        float s = abs_max / 8.0f;
        if (s == 0.0f) s = 1.0f;
        scale_b[row] = s;
        for (size_t kp = 0; kp < k / 2; ++kp) {
            int32_t q0 = (int32_t)nearbyintf(r[2 * kp + 0] / s);
            int32_t q1 = (int32_t)nearbyintf(r[2 * kp + 1] / s);
            if (q0 < -8) q0 = -8;
            if (q0 > 7) q0 = 7;
            if (q1 < -8) q1 = -8;
            if (q1 > 7) q1 = 7;
            B_nib[row * (k / 2) + kp] = (uint8_t)((uint8_t)(q0 + 8) | ((uint8_t)(q1 + 8) << 4));
        }
    }
}

/* ------------------------------------------------------------------------- */
/* W4A8 GEMM, float output (f32 / f16 / bf16).                                */
/* Follows w4a8_reference_fp32 (test/gemm/test_gemm_i8_i4_rvv.cpp:122-156)    */
/* and the cast through the output type (:296-299).  The multiply order       */
/* ((float)acc * scale_a) * scale_b, "C before bias", clamp in f32 and the    */
/* final round-to-nearest-even narrowing match the RVV kernel                 */
/* (src/gemm/gemm_i8_i4/tqt_kernel_gemm_i8_i4_4x1vl_rvv.h:272-301, 374-397).  */
/* B_nib is [n, k/2] bytes with row stride ldb_bytes.  C and bias are typed   */
/* like D (td).  k must be even.                                              */
/* ------------------------------------------------------------------------- */
void tqo_gemm_w4a8(size_t m, size_t n, size_t k, const int8_t *A, size_t lda, const uint8_t *B_nib,
                   size_t ldb_bytes, const float *scale_a, const int32_t *zp_a,
                   const float *scale_b, const void *C, size_t ldc, const void *bias, void *D,
                   size_t ldd, float clamp_min, float clamp_max, int td)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t mi = 0; mi < (ptrdiff_t)m; ++mi) {
        const int8_t *a = A + mi * lda;
        for (size_t ni = 0; ni < n; ++ni) {
            const uint8_t *b = B_nib + ni * ldb_bytes;
            int32_t acc = 0;
            int32_t b_sum = 0;
            for (size_t kp = 0; kp < k / 2; ++kp) {
                uint8_t byte = b[kp];
                int32_t b_lo = (int32_t)(byte & 0xf) - 8;
                int32_t b_hi = (int32_t)(byte >> 4) - 8;
                acc += (int32_t)a[2 * kp] * b_lo + (int32_t)a[2 * kp + 1] * b_hi;
                b_sum += b_lo + b_hi;
            }
            acc -= zp_a[mi] * b_sum;
            float r = (float)acc * scale_a[mi];
            r = r * scale_b[ni];
            if (C) r += td_load(C, mi * ldc + ni, td);
            if (bias) r += td_load(bias, ni, td);
            if (r < clamp_min) r = clamp_min;
            if (r > clamp_max) r = clamp_max;
            td_store(D, mi * ldd + ni, td, r);
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Requantisation multiplier.                                                 */
/* Follows src/gemm/gemm_i8_i8/tqt_utils_i8_i8.h:16-90 (integer_from_exp) and */
/* :98-132 (tqt_quantize_multiplier): top 30 fraction bits plus the implicit  */
/* one, +1 only when the discarded 22 bits are strictly above half, 2^31      */
/* renormalised, shift < -31 flushed to zero.                                 */
/* ------------------------------------------------------------------------- */
void tqo_quantize_multiplier(double v, int32_t *mult, int32_t *shift)
{
    if (v == 0.) {
        *mult = 0;
        *shift = 0;
        return;
    }
    uint64_t u;
    memcpy(&u, &v, 8);
    int64_t q;
    if ((u & 0x7fffffffffffffffull) == 0) {
        *shift = 0;
        q = 0;
    } else {
        uint32_t e = (uint32_t)((u & 0x7ff0000000000000ull) >> 52);
        if (e == 0x7ff) {
            *shift = 0x7fffffff;
            if (u & 0x000fffffffc00000ull)
                q = 0;
            else
                q = (u >> 63) ? (int64_t)0x8000000000000000ull : (int64_t)0x7fffffffffffffffll;
        } else {
            *shift = (int32_t)(e - 1023) + 1;
            q = 0x40000000 + (int64_t)((u & 0x000fffffffc00000ull) >> 22);
            if ((u & 0x003fffffu) > 0x00200000u) q += 1;
            if (u >> 63) q = -q;
        }
    }
    if (q == (1ll << 31)) {
        q /= 2;
        ++*shift;
    }
    if (*shift < -31) {
        *shift = 0;
        q = 0;
    }
    *mult = (int32_t)q;
}

static inline int32_t sat_narrow_32_16_8(int32_t t)
{
    /* vnclip.wx with shift 0 twice: saturate to int16, then to int8. */
    if (t > 32767) t = 32767;
    if (t < -32768) t = -32768;
    if (t > 127) t = 127;
    if (t < -128) t = -128;
    return t;
}

/* One requantisation step, as the RVV sequence vmulh.vv / vsra.vv / vadd.vx /
 * vnclip / vnclip executes it
 * (src/gemm/gemm_i8_i8/tqt_kernel_gemm_i8_i8_4x1vl_rvv.h:335-408):
 * signed high half of the 64-bit product, arithmetic shift by the low five
 * bits of the shift operand, wrapping add of the zero point, two saturating
 * narrows.  No rounding anywhere. */
int32_t tqo_requantize_one(int32_t acc, int32_t mult, int32_t sh, int32_t zp)
{
    int32_t t = (int32_t)(((int64_t)acc * (int64_t)mult) >> 32);
    t = t >> (sh & 31);
    t = (int32_t)((uint32_t)t + (uint32_t)zp);
    return sat_narrow_32_16_8(t);
}

/* ------------------------------------------------------------------------- */
/* gemm_1xnbias_reqi32toi8_clamp_qai8_*: static W8A8 with int8 output.        */
/* acc = C + A*B + bias[n]; per column real = (double)sa*(double)sb[n]/sd,    */
/* (mult, s) = quantize_multiplier(real), sh = -s-1                           */
/* (src/gemm/gemm_i8_i8/gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp/     */
/*  tqt_gemm_..._4x1vl_rvv.cpp:193-209; quant_channel_b == 1 shares column 0).*/
/* zero_point_a is not applied: callers pre-fuse it into the bias.            */
/* ------------------------------------------------------------------------- */
void tqo_gemm_reqi32toi8(size_t m, size_t n, size_t k, const int8_t *A, size_t lda,
                         const int8_t *B, size_t ldb, int b_transposed, const int32_t *C,
                         size_t ldc, const int32_t *bias, int8_t *D, size_t ldd, int8_t clamp_min,
                         int8_t clamp_max, float scale_a, const float *scale_b,
                         int32_t quant_channel_b, float scale_d, int32_t zp_d)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            int32_t acc = 0;
            if (b_transposed) {
                const int8_t *a = A + i * lda;
                const int8_t *b = B + j * ldb;
                for (size_t p = 0; p < k; ++p) acc += (int32_t)a[p] * (int32_t)b[p];
            } else {
                for (size_t p = 0; p < k; ++p)
                    acc += (int32_t)A[i * lda + p] * (int32_t)B[p * ldb + j];
            }
            uint32_t u = (uint32_t)acc;
            if (C) u += (uint32_t)C[i * ldc + j];
            if (bias) u += (uint32_t)bias[j];
            size_t sj = (quant_channel_b == 1) ? 0 : j;
            double real = (double)scale_a * (double)scale_b[sj] / (double)scale_d;
            int32_t mult, s;
            tqo_quantize_multiplier(real, &mult, &s);
            int32_t sh = -s - 1;
            int32_t t = tqo_requantize_one((int32_t)u, mult, sh, zp_d);
            if (t < clamp_min) t = clamp_min;
            if (t > clamp_max) t = clamp_max;
            D[i * ldd + j] = (int8_t)t;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx[p]_qai8[p]: static W8A8 with a   */
/* per-row scale of A and an Mx1 bias.  acc = C + A*B + bias[m]; per row      */
/* real = (double)sa[m]*(double)sb/sd (row 0 for every row when                */
/* quant_channel_a == 1), then the same integer tail                           */
/* (src/gemm/gemm_i8_i8/gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8/       */
/*  tqt_gemm_..._4x1vl_rvv.cpp:84-118, 141-163; requant                        */
/*  tqt_kernel_gemm_i8_i8_4x1vl_rvv.h:264-330).  A [m,k], B [k,n] row-major.   */
/* zero_point_b is not applied: callers pre-fuse it into the bias.            */
/* Parity unpinned beyond the reference's own +-1 LSB dequantised tolerance,   */
/* like tqo_gemm_reqi32toi8 (same tail).                                       */
/* ------------------------------------------------------------------------- */
void tqo_gemm_mx1bias_reqi32toi8(size_t m, size_t n, size_t k, const int8_t *A, size_t lda,
                                 const int8_t *B, size_t ldb, const int32_t *C, size_t ldc,
                                 const int32_t *bias, int8_t *D, size_t ldd, int8_t clamp_min,
                                 int8_t clamp_max, const float *scale_a, int32_t quant_channel_a,
                                 float scale_b, float scale_d, int32_t zp_d)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
        size_t si = (quant_channel_a == 1) ? 0 : (size_t)i;
        double real = (double)scale_a[si] * (double)scale_b / (double)scale_d;
        int32_t mult, s;
        tqo_quantize_multiplier(real, &mult, &s);
        int32_t sh = -s - 1;
        for (size_t j = 0; j < n; ++j) {
            int32_t acc = 0;
            for (size_t p = 0; p < k; ++p) acc += (int32_t)A[i * lda + p] * (int32_t)B[p * ldb + j];
            uint32_t u = (uint32_t)acc;
            if (C) u += (uint32_t)C[i * ldc + j];
            if (bias) u += (uint32_t)bias[i];
            int32_t t = tqo_requantize_one((int32_t)u, mult, sh, zp_d);
            if (t < clamp_min) t = clamp_min;
            if (t > clamp_max) t = clamp_max;
            D[i * ldd + j] = (int8_t)t;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* qsi4c2: block-wise int4 quantisation of f16 weights with f16 scales.       */
/* Follows test/common/quantize_utils.h:34-70 (quantize_fp16_to_int4):        */
/* scale = signed-absmax / -8, q = min((int8)(v/scale + 8.5), 15).            */
/* ------------------------------------------------------------------------- */
void tqo_quantize_fp16_to_int4(size_t n, size_t k, size_t bl, const uint16_t *src, uint8_t *dst,
                               uint16_t *scale, size_t ld_scale)
{
    memset(dst, 0, n * (k / 2));
    for (size_t j = 0; j < n; ++j) {
        const size_t num_blocks = k / bl;
        for (size_t b = 0; b < num_blocks; ++b) {
            float max_value = 0.0f;
            float abs_max_value = 0.0f;
            for (size_t t = 0; t < bl; ++t) {
                float value = tqo_f16_to_f32(src[j * k + b * bl + t]);
                if (fabsf(value) > abs_max_value) {
                    abs_max_value = fabsf(value);
                    max_value = value;
                }
            }
            float fp32_scale = max_value / -8.0f;
            float inv_scale = (fp32_scale != 0.0f) ? (1.0f / fp32_scale) : 0.0f;
            scale[j * ld_scale + b] = tqo_f32_to_f16(fp32_scale);
            for (size_t t = 0; t < bl; t += 2) {
                float v0 = tqo_f16_to_f32(src[j * k + b * bl + t]);
                float v1 = tqo_f16_to_f32(src[j * k + b * bl + t + 1]);
                uint8_t q0 = (uint8_t)fminf((float)(int8_t)(v0 * inv_scale + 8.5f), 15);
                uint8_t q1 = (uint8_t)fminf((float)(int8_t)(v1 * inv_scale + 8.5f), 15);
                dst[j * (k / 2) + (b * bl + t) / 2] = (uint8_t)(q0 | (uint8_t)(q1 << 4));
            }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* W4A16 block-quant GEMM with f32 accumulation.                              */
/* Follows reference_gemm_quantized_weight_mixed                              */
/* (test/common/reference_gemm.cpp:132-179): acc starts at C, adds            */
/* a * ((nib-8) * scale[n, p/bl]) term by term in f32, then bias, clamp,      */
/* and narrows to the output type.  A and scale_b are f16; C/bias/D are td    */
/* (f16 or f32).  The RVV kernel itself accumulates in f16                    */
/* (src/gemm/gemm_f16_i4/tqt_kernel_gemm_f16_i4_8x2vl_rvv.h:372); the         */
/* reference's tests accept it against this f32-accumulating function.        */
/* ------------------------------------------------------------------------- */
void tqo_gemm_w4a16(size_t m, size_t n, size_t k, size_t bl, const uint16_t *A, size_t lda,
                    const uint8_t *B_nib, size_t ldb, const uint16_t *scale_b, size_t ldsb,
                    const void *C, size_t ldc, void *D, size_t ldd, const void *bias,
                    float clamp_min, float clamp_max, int td)
{
    const size_t b_row_bytes = ldb / 2;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            float acc = 0.0f;
            if (C) acc = td_load(C, i * ldc + j, td);
            for (size_t p = 0; p < k; ++p) {
                float a_val = tqo_f16_to_f32(A[i * lda + p]);
                uint8_t byte_val = B_nib[j * b_row_bytes + p / 2];
                int8_t b_raw = (p % 2 == 0) ? (int8_t)((int8_t)(byte_val & 0x0F) - 8)
                                            : (int8_t)((int8_t)(byte_val >> 4) - 8);
                float scale_val = tqo_f16_to_f32(scale_b[j * ldsb + p / bl]);
                float b_dequant = (float)b_raw * scale_val;
                acc += a_val * b_dequant;
            }
            if (bias) acc += td_load(bias, j, td);
            acc = acc > clamp_min ? acc : clamp_min;
            acc = acc < clamp_max ? acc : clamp_max;
            td_store(D, i * ldd + j, td, acc);
        }
    }
}

/* ------------------------------------------------------------------------- */
/* qai8dx x qsi8cx float-output GEMM (dynamic-A W8A8).                        */
/* Follows src/gemm/gemm_i8_i8/tqt_kernel_gemm_qai8dx_qsi8cx_4x1vl_rvv.h:     */
/* acc = sum (a - zp_a[m]) * b (:95-139); r = (float)acc * (scale_b[n] *      */
/* scale_a[m]) (:167-176); C is ignored.  f32 output: + bias, clamp in f32.   */
/* f16 output: narrow first, then add bias and clamp in f16 (:262-278).       */
/* ------------------------------------------------------------------------- */
void tqo_gemm_qai8dx_qsi8cx(size_t m, size_t n, size_t k, const int8_t *A, size_t lda,
                            const int8_t *B, size_t ldb, int b_transposed, const float *scale_a,
                            const int32_t *zp_a, const float *scale_b, const void *bias, void *D,
                            size_t ldd, float clamp_min, float clamp_max, int td)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            int32_t acc = 0;
            for (size_t p = 0; p < k; ++p) {
                int32_t b = b_transposed ? B[j * ldb + p] : B[p * ldb + j];
                acc += ((int32_t)A[i * lda + p] - zp_a[i]) * b;
            }
            float s = scale_b[j] * scale_a[i];
            float r = (float)acc * s;
            if (td == TQO_TD_F32) {
                if (bias) r += ((const float *)bias)[j];
                if (r < clamp_min) r = clamp_min;
                if (r > clamp_max) r = clamp_max;
                ((float *)D)[i * ldd + j] = r;
            } else {
                /* narrow, then f16 add / max / min, each rounded to f16 */
                float h = tqo_f16_to_f32(tqo_f32_to_f16(r));
                if (bias)
                    h = tqo_f16_to_f32(
                        tqo_f32_to_f16(h + tqo_f16_to_f32(((const uint16_t *)bias)[j])));
                if (h < clamp_min) h = clamp_min;
                if (h > clamp_max) h = clamp_max;
                ((uint16_t *)D)[i * ldd + j] = tqo_f32_to_f16(h);
            }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* im2col of the int8 convolution wrappers.                                   */
/* Follows src/common/tqt_conv.h: channel-first (:52-121) input [C,D,H,W],    */
/* matrix [K, N] with K order (ic, kd, kh, kw) and N = output positions;      */
/* channel-last (:124-196) input [D,H,W,C], matrix [M, K] with M = output     */
/* positions and K order (kd, kh, kw, ic).  Padding positions hold 0.         */
/* geom: the 21 size_t members of tqt_conv_params in declaration order        */
/* (:23-34): input, output, kernel, stride, dilation, pad (3 each),           */
/* input_channel, output_channel, groups.                                     */
/* Written per matrix element (the reference walks the input in nested loops  */
/* and copies channel runs).                                                  */
/* ------------------------------------------------------------------------- */
void tqo_im2col_i8(int channel_first, size_t group_idx, const int8_t *act, int8_t *out,
                   const size_t *geom)
{
    const size_t *in = geom, *o = geom + 3, *ker = geom + 6, *st = geom + 9, *dil = geom + 12,
                 *pad = geom + 15;
    const size_t c_total = geom[18], groups = geom[20];
    const size_t ic_pg = c_total / groups, c_off = group_idx * ic_pg;
    const size_t rows = o[0] * o[1] * o[2], kvol = ker[0] * ker[1] * ker[2], K = kvol * ic_pg;
    const size_t in_vol = in[0] * in[1] * in[2];
    for (size_t pos = 0; pos < rows; ++pos) {
        const size_t ow = pos % o[2], oh = (pos / o[2]) % o[1], od = pos / (o[2] * o[1]);
        for (size_t k = 0; k < K; ++k) {
            size_t ic, kpos;
            if (channel_first) {
                ic = k / kvol;
                kpos = k % kvol;
            } else {
                kpos = k / ic_pg;
                ic = k % ic_pg;
            }
            const size_t kw = kpos % ker[2], kh = (kpos / ker[2]) % ker[1],
                         kd = kpos / (ker[2] * ker[1]);
            const long id = (long)(od * st[0] + kd * dil[0]) - (long)pad[0];
            const long ih = (long)(oh * st[1] + kh * dil[1]) - (long)pad[1];
            const long iw = (long)(ow * st[2] + kw * dil[2]) - (long)pad[2];
            int8_t v = 0;
            if (id >= 0 && id < (long)in[0] && ih >= 0 && ih < (long)in[1] && iw >= 0 &&
                iw < (long)in[2]) {
                const size_t sp = ((size_t)id * in[1] + (size_t)ih) * in[2] + (size_t)iw;
                v = channel_first ? act[(c_off + ic) * in_vol + sp]
                                  : act[sp * c_total + c_off + ic];
            }
            if (channel_first)
                out[k * rows + pos] = v;
            else
                out[pos * K + k] = v;
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Unquantised GEMM families (f32 / f16 / bf16 operands).                     */
/* Follows test/common/reference_gemm.cpp:11-61: f32 accumulation in k order  */
/* (separate multiply and add), + C, + bias (per column, or per row for the   */
/* mx1bias types), clamp in f32, one narrowing to the output type.            */
/* ta / td: TQO_TD_*; b_transposed: B is [n, ldb], else [k, ldb].             */
/* ------------------------------------------------------------------------- */
void tqo_gemm_float(int ta, int td, size_t m, size_t n, size_t k, const void *A, size_t lda,
                    const void *B, size_t ldb, int b_transposed, const void *C, size_t ldc,
                    void *D, size_t ldd, const void *bias, int bias_per_row, float clamp_min,
                    float clamp_max)
{
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)m; ++i) {
        for (size_t j = 0; j < n; ++j) {
            float acc = 0.0f;
            for (size_t p = 0; p < k; ++p) {
                const float a = td_load(A, (size_t)i * lda + p, ta);
                const float b = b_transposed ? td_load(B, j * ldb + p, ta) : td_load(B, p * ldb + j, ta);
                const float prod = a * b;
                acc = acc + prod;
            }
            if (C) acc += td_load(C, (size_t)i * ldc + j, td);
            if (bias) acc += td_load(bias, bias_per_row ? (size_t)i : j, td);
            acc = fmaxf(acc, clamp_min);
            acc = fminf(acc, clamp_max);
            td_store(D, (size_t)i * ldd + j, td, acc);
        }
    }
}
