/*
 * W4A16 GEMM micro-kernels for B200: f16 activations times block-quantised int4 weights (qsi4c2:
 * one f16 scale per bl consecutive k of each output channel).
 *
 *   D = clamp(C + A * dequant(B)^T + bias, clamp_min, clamp_max),
 *   dequant(B)[n,k] = (nib[n,k] - 8) * scale_b[n, k / bl]
 *
 * Kernel types and the reference variants they replace (paths under src/gemm/gemm_f16_i4/):
 *   gemm_1xnbias_clamp_f16_f16p_qsi4c2p   gemm_1xnbias_clamp_f16_f16p_qsi4c2p/
 *                                         tqt_gemm_1xnbias_clamp_f16_f16p_qsi4c2p_8x2vl_rvv.h:30-101
 *                                         (run_gemm: ..._8x2vl_rvv.cpp:224-283)
 *   gemm_1xnbias_clamp_f32_f16p_qsi4c2p   gemm_1xnbias_clamp_f32_f16p_qsi4c2p/..._8x2vl_rvv.h (run_gemm: .cpp:224)
 *
 * Arithmetic: each weight is dequantised to f16 ((nib-8)*scale rounded once to f16, as the RVV
 * kernel does, tqt_kernel_gemm_f16_i4_8x2vl_rvv.h:296-298) and the products are accumulated in
 * f32 in tensor memory (the RVV kernel accumulates in f16; the reference's tests check it against
 * an f32-accumulating function, test/common/reference_gemm.cpp:132-179).
 *
 * scale_b is [n, k/bl] f16 row-major with leading dimension ldsb, NOT packed (as in the
 * reference); bl is a run-time argument: even, >= 2, k % bl == 0.
 *
 * Packed layouts (opaque): A_packed is [ceil(m/128)][ceil(k/64)] blocks of 128 rows x 64 f16
 * (16 KiB, 128-byte-swizzled K-major); B_packed is [ceil(n/128)][ceil(k/128)] blocks of 128 rows x
 * 128 int4 (8 KiB), nibbles ordered for a shift-and-mask expansion to f16 pairs.
 */
#ifndef TQT_B200_GEMM_F16_I4_H
#define TQT_B200_GEMM_F16_I4_H

#include "tqt_b200_common.h"

#ifdef __cplusplus
extern "C" {
#endif

#define TQT_B200_DECLARE_W4A16_PACKED(TDNAME, TDTYPE)                                                                  \
    size_t tqt_get_m_step_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(void);                            \
    size_t tqt_get_n_step_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(void);                            \
    size_t tqt_get_a_packed_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                         \
        size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);                                                      \
    size_t tqt_get_b_packed_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                         \
        size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);                                                      \
    size_t tqt_get_scale_b_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t n_idx,             \
                                                                                            size_t b_idx,             \
                                                                                            size_t ldsb);             \
    size_t tqt_get_c_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t m_idx, size_t n_idx,     \
                                                                                      size_t ldc);                     \
    size_t tqt_get_bias_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t n_idx);               \
    size_t tqt_get_d_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t m_idx, size_t n_idx,     \
                                                                                      size_t ldd);                     \
    size_t tqt_get_d_size_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t m, size_t n);              \
    size_t tqt_get_a_packed_size_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t m, size_t k);       \
    size_t tqt_get_b_packed_size_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t n, size_t k);       \
    void tqt_run_a_pack_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                                    \
        size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A, void *A_packed);              \
    void tqt_run_bt_pack_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                                   \
        size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed);              \
    void tqt_run_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                                           \
        size_t m, size_t n, size_t k, size_t bl, const void *A_packed, size_t lda, size_t k_idx_a,                    \
        const void *B_packed, size_t ldb, size_t k_idx_b, const void *scale_b, size_t ldsb, const void *C,            \
        size_t ldc, void *D, size_t ldd, const void *bias, TDTYPE clamp_min, TDTYPE clamp_max);                       \
    struct tqt_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_ukernel {                                                   \
        size_t (*get_m_step)(void);                                                                                    \
        size_t (*get_n_step)(void);                                                                                    \
        size_t (*get_a_packed_offset)(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);                        \
        size_t (*get_b_packed_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);                        \
        size_t (*get_scale_b_offset)(size_t n_idx, size_t b_idx, size_t ldsb);                                         \
        size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);                                                \
        size_t (*get_bias_offset)(size_t n_idx);                                                                       \
        size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);                                                \
        size_t (*get_d_size)(size_t m, size_t n);                                                                      \
        size_t (*get_a_packed_size)(size_t m, size_t k);                                                               \
        size_t (*get_b_packed_size)(size_t n, size_t k);                                                               \
        void (*run_a_pack)(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A,             \
                           void *A_packed);                                                                            \
        void (*run_bt_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B,            \
                            void *B_packed);                                                                           \
        void (*run_gemm)(size_t m, size_t n, size_t k, size_t bl, const void *A_packed, size_t lda,                    \
                         size_t k_idx_a, const void *B_packed, size_t ldb, size_t k_idx_b, const void *scale_b,        \
                         size_t ldsb, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,                \
                         TDTYPE clamp_min, TDTYPE clamp_max);                                                          \
    };

#if !defined(TQT_B200_NO_HALF_TYPES)
/* f16 output: clamp arguments are float16_t by value, as in the reference (..._8x2vl_rvv.h:97-101). */
TQT_B200_DECLARE_W4A16_PACKED(f16, float16_t)
#endif
/* f32 output (reference: gemm_1xnbias_clamp_f32_f16p_qsi4c2p, float clamps). */
TQT_B200_DECLARE_W4A16_PACKED(f32, float)

#ifdef __cplusplus
}
#endif

#endif /* TQT_B200_GEMM_F16_I4_H */
