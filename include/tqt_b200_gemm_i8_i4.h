/*
 * W4A8 GEMM micro-kernels for B200: per-row dynamically quantised int8 activations (qai8dx) times
 * per-channel symmetric int4 weights (qsi4cx), float output.
 *
 *   D = clamp(C + dequant(A) * dequant(B)^T + bias, clamp_min, clamp_max)
 *     acc[m,n]  = sum_k a[m,k] * (nib[n,k] - 8)            (int32, exact)
 *     acc      -= zero_point_a[m] * sum_k (nib[n,k] - 8)
 *     r         = ((float)acc * scale_a[m]) * scale_b[n]   (this order)
 *     r        += C[m,n] (if C), then r += bias[n] (if bias), clamp in f32, narrow (RNE) to TD
 *
 * Each kernel type below replaces the RVV variant of the same name in the reference:
 *   gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp   src/gemm/gemm_i8_i4/gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp/
 *                                            tqt_gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp_4x1vl_rvv.h:33-74
 *                                            (run_gemm: ..._4x1vl_rvv.cpp:196-238)
 *   gemm_1xnbias_clamp_f16_qai8dxp_qsi4cxp   .../gemm_1xnbias_clamp_f16_qai8dxp_qsi4cxp/..._4x1vl_rvv.h
 *                                            (run_gemm: ..._4x1vl_rvv.cpp:206)
 *   gemm_1xnbias_clamp_bf16_qai8dxp_qsi4cxp  .../gemm_1xnbias_clamp_bf16_qai8dxp_qsi4cxp/..._4x1vl_rvv.h:33-76
 *                                            (run_gemm: ..._4x1vl_rvv.cpp:204-248)
 * and the ukernel structs mirror the *_interface.h of each directory.
 *
 * Packed layouts (opaque; sized and addressed only through the helpers):
 *   A_packed  [ceil(m/128)][ceil(k/128)] blocks of 128 rows x 128 int8, each block 16 KiB in the
 *             128-byte-swizzled K-major order that tcgen05.mma reads from shared memory; rows and
 *             columns past m / k are zero.
 *   B_packed  [ceil(n/128)][ceil(k/128)] blocks of 8448 bytes: 128 rows x 128 int4 (two's
 *             complement nibbles, ordered for a two-instruction expansion to int8) followed by
 *             128 int16 partial row sums of the block, which the kernels add up for the
 *             zero-point correction.  Padding nibbles are zero.
 * K-slab packing: run_a_pack / run_bt_pack with k < ld_packed and k_idx a multiple of 128 write
 * the slab into the full buffer when given the destination pointer offset by
 * get_*_packed_offset(idx, k_idx, ld_packed, rows), exactly as with the reference.
 *
 * params->scale_a / zero_point_a / scale_b are indexed from the call's own first row / column
 * (reference ..._4x1vl_rvv.cpp:228-230): a caller that tiles passes offset pointers.
 * The packed-A row stride is k, not lda (reference ..._4x1vl_rvv.cpp:222).
 */
#ifndef TQT_B200_GEMM_I8_I4_H
#define TQT_B200_GEMM_I8_I4_H

#include "tqt_b200_common.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Same layout as the reference's struct (src/gemm/gemm_i8_i4/tqt_params_i8_i4.h:23-28).  The struct
 * lives in host memory; the three arrays are device arrays of m, m and n elements. */
struct tqt_qai8dx_qsi4cx_params {
    const float *scale_a;
    const int32_t *zero_point_a;
    const float *scale_b;
};

#define TQT_B200_DECLARE_W4A8_PACKED(TDNAME, TDTYPE)                                                                    \
    size_t tqt_get_m_step_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(void);                          \
    size_t tqt_get_n_step_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(void);                          \
    size_t tqt_get_a_packed_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                       \
        size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);                                                       \
    size_t tqt_get_b_packed_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                       \
        size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);                                                       \
    size_t tqt_get_c_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t m_idx, size_t n_idx,   \
                                                                                         size_t ldc);                   \
    size_t tqt_get_bias_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t n_idx);             \
    size_t tqt_get_d_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t m_idx, size_t n_idx,   \
                                                                                         size_t ldd);                   \
    size_t tqt_get_d_size_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t m, size_t n);            \
    size_t tqt_get_a_packed_size_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t m, size_t k);     \
    size_t tqt_get_b_packed_size_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t n, size_t k);     \
    /* A [m,k] int8 row-major (lda) -> A_packed. */                                                                     \
    void tqt_run_a_pack_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                                  \
        size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A, void *A_packed);               \
    /* B [n,k] int4 stored [n,k/2] bytes, byte = (q_even+8) | (q_odd+8)<<4, ldb in int4 elements -> B_packed. */        \
    void tqt_run_bt_pack_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                                 \
        size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed);               \
    void tqt_run_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                                         \
        size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a, const void *B_packed,          \
        size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,                  \
        TDTYPE clamp_min, TDTYPE clamp_max, const struct tqt_qai8dx_qsi4cx_params *params);                            \
    struct tqt_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_ukernel {                                                 \
        size_t (*get_m_step)(void);                                                                                     \
        size_t (*get_n_step)(void);                                                                                     \
        size_t (*get_a_packed_offset)(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);                         \
        size_t (*get_b_packed_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);                         \
        size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);                                                 \
        size_t (*get_bias_offset)(size_t n_idx);                                                                        \
        size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);                                                 \
        size_t (*get_d_size)(size_t m, size_t n);                                                                       \
        size_t (*get_a_packed_size)(size_t m, size_t k);                                                                \
        size_t (*get_b_packed_size)(size_t n, size_t k);                                                                \
        void (*run_a_pack)(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A,              \
                           void *A_packed);                                                                             \
        void (*run_bt_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B,             \
                            void *B_packed);                                                                            \
        void (*run_gemm)(size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a,                \
                         const void *B_packed, size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D,          \
                         size_t ldd, const void *bias, TDTYPE clamp_min, TDTYPE clamp_max,                              \
                         const struct tqt_qai8dx_qsi4cx_params *params);                                                \
    };

TQT_B200_DECLARE_W4A8_PACKED(f32, float)
#if !defined(TQT_B200_NO_HALF_TYPES)
TQT_B200_DECLARE_W4A8_PACKED(f16, float16_t)
TQT_B200_DECLARE_W4A8_PACKED(bf16, bfloat16_t)
#endif

#ifdef __cplusplus
}
#endif

#endif /* TQT_B200_GEMM_I8_I4_H */
