/*
 * Unquantised GEMM kernel types (f32, f16, bf16 operands): D = clamp(A * B + C + bias), accumulated in f32 and narrowed
 * once to the output type.  Same names and argument lists as the reference with the variant suffix "_128x128_sm100a".
 *
 * Reference variants replaced (paths under src/gemm/; each type directory holds <type>_interface.h and the RVV variants):
 *   gemm_f32_f32/   gemm_1xnbias_clamp_f32_f32_f32, ..._f32_f32p, ..._f32_f32t, ..._f32p_f32p,
 *                   gemm_mx1bias_clamp_f32_f32_f32, gemm_mx1bias_clamp_f32_f32p_f32p
 *   gemm_f16_f16/   the same six with f16
 *   gemm_bf16_bf16/ gemm_1xnbias_clamp_{bf16,f16,f32}_bf16_bf16, ..._bf16_bf16t, ..._bf16p_bf16p, and
 *                   gemm_1xnbias_clamp_bf16_bf16_bf16p
 * Type name = gemm_<bias>_clamp_<TD>_<TA>[p]_<TB>[p|t]: TD the type of C, D, bias and the clamps; A is [m, lda] or packed
 * (p); B is [k, ldb] (no suffix), [n, ldb] (t) or packed (p); 1xnbias adds bias[n], mx1bias bias[m].
 * Arithmetic: test/common/reference_gemm.cpp:11-61 (the reference's portable oracle for these kernels).
 *
 * The f16 / bf16 types run on the tcgen05 CTA-pair kernel (kind::f16, f32 accumulators in tensor memory) when their
 * operands are packed or are row-major [rows, k] with base address and row stride multiples of 16 bytes (tiled TMA
 * loads); every other call (f32 operands, B stored [k, n], unaligned operands) runs on a generic CUDA-core kernel
 * that reproduces the reference's k-order f32 arithmetic bit for bit.  Packed blocks: 128 rows x 128 bytes (64 or 32
 * elements of k), 128-byte swizzle, zero padded; m_step = n_step = 128; k_idx multiples of TQT_B200_K_STEP.
 * All data pointers are device pointers.
 */
#ifndef TQT_B200_GEMM_FLOAT_H
#define TQT_B200_GEMM_FLOAT_H

#include "tqt_b200_common.h"

#ifdef __cplusplus
extern "C" {
#endif

#define TQT_B200_FLOAT_RUN_ARGS(CLAMPT)                                                                               \
    size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B, size_t ldb,               \
        size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, CLAMPT clamp_min,           \
        CLAMPT clamp_max

#define TQT_B200_FLOAT_COMMON(TYPE)                                                                                   \
    size_t tqt_get_m_step_##TYPE##_128x128_sm100a(void);                                                               \
    size_t tqt_get_n_step_##TYPE##_128x128_sm100a(void);                                                               \
    size_t tqt_get_c_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldc);                           \
    size_t tqt_get_bias_offset_##TYPE##_128x128_sm100a(size_t idx);                                                    \
    size_t tqt_get_d_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldd);                           \
    size_t tqt_get_d_size_##TYPE##_128x128_sm100a(size_t m, size_t n);

/* both operands in the caller's layouts */
#define TQT_B200_DECLARE_FLOAT_UU(TYPE, CLAMPT)                                                                       \
    TQT_B200_FLOAT_COMMON(TYPE)                                                                                       \
    size_t tqt_get_a_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t k_idx, size_t lda);                           \
    size_t tqt_get_b_offset_##TYPE##_128x128_sm100a(size_t n_idx, size_t k_idx, size_t ldb);                           \
    void tqt_run_##TYPE##_128x128_sm100a(TQT_B200_FLOAT_RUN_ARGS(CLAMPT));                                             \
    struct tqt_##TYPE##_ukernel {                                                                                      \
        size_t (*get_m_step)(void);                                                                                    \
        size_t (*get_n_step)(void);                                                                                    \
        size_t (*get_a_offset)(size_t m_idx, size_t k_idx, size_t lda);                                                \
        size_t (*get_b_offset)(size_t n_idx, size_t k_idx, size_t ldb);                                                \
        size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);                                                \
        size_t (*get_bias_offset)(size_t idx);                                                                         \
        size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);                                                \
        size_t (*get_d_size)(size_t m, size_t n);                                                                      \
        void (*run_gemm)(TQT_B200_FLOAT_RUN_ARGS(CLAMPT));                                                             \
    };

/* A in the caller's layout, B packed */
#define TQT_B200_DECLARE_FLOAT_UP(TYPE, CLAMPT)                                                                       \
    TQT_B200_FLOAT_COMMON(TYPE)                                                                                       \
    size_t tqt_get_a_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t k_idx, size_t lda);                           \
    size_t tqt_get_b_packed_offset_##TYPE##_128x128_sm100a(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);   \
    size_t tqt_get_b_packed_size_##TYPE##_128x128_sm100a(size_t n, size_t k);                                          \
    void tqt_run_b_pack_##TYPE##_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx,       \
                                                const void *B, void *B_packed);                                        \
    void tqt_run_bt_pack_##TYPE##_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx,      \
                                                 const void *B, void *B_packed);                                       \
    void tqt_run_##TYPE##_128x128_sm100a(TQT_B200_FLOAT_RUN_ARGS(CLAMPT));                                             \
    struct tqt_##TYPE##_ukernel {                                                                                      \
        size_t (*get_m_step)(void);                                                                                    \
        size_t (*get_n_step)(void);                                                                                    \
        size_t (*get_a_offset)(size_t m_idx, size_t k_idx, size_t lda);                                                \
        size_t (*get_b_packed_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);                        \
        size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);                                                \
        size_t (*get_bias_offset)(size_t idx);                                                                         \
        size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);                                                \
        size_t (*get_d_size)(size_t m, size_t n);                                                                      \
        size_t (*get_b_packed_size)(size_t n, size_t k);                                                               \
        void (*run_b_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed); \
        void (*run_bt_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed); \
        void (*run_gemm)(TQT_B200_FLOAT_RUN_ARGS(CLAMPT));                                                             \
    };

/* both operands packed */
#define TQT_B200_DECLARE_FLOAT_PP(TYPE, CLAMPT)                                                                       \
    TQT_B200_FLOAT_COMMON(TYPE)                                                                                       \
    size_t tqt_get_a_packed_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);   \
    size_t tqt_get_b_packed_offset_##TYPE##_128x128_sm100a(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);   \
    size_t tqt_get_a_packed_size_##TYPE##_128x128_sm100a(size_t m, size_t k);                                          \
    size_t tqt_get_b_packed_size_##TYPE##_128x128_sm100a(size_t n, size_t k);                                          \
    void tqt_run_a_pack_##TYPE##_128x128_sm100a(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx,       \
                                                const void *A, void *A_packed);                                        \
    void tqt_run_b_pack_##TYPE##_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx,       \
                                                const void *B, void *B_packed);                                        \
    void tqt_run_bt_pack_##TYPE##_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx,      \
                                                 const void *B, void *B_packed);                                       \
    void tqt_run_##TYPE##_128x128_sm100a(TQT_B200_FLOAT_RUN_ARGS(CLAMPT));                                             \
    struct tqt_##TYPE##_ukernel {                                                                                      \
        size_t (*get_m_step)(void);                                                                                    \
        size_t (*get_n_step)(void);                                                                                    \
        size_t (*get_a_packed_offset)(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);                        \
        size_t (*get_b_packed_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);                        \
        size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);                                                \
        size_t (*get_bias_offset)(size_t idx);                                                                         \
        size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);                                                \
        size_t (*get_d_size)(size_t m, size_t n);                                                                      \
        size_t (*get_a_packed_size)(size_t m, size_t k);                                                               \
        size_t (*get_b_packed_size)(size_t n, size_t k);                                                               \
        void (*run_a_pack)(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A, void *A_packed); \
        void (*run_b_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed); \
        void (*run_bt_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed); \
        void (*run_gemm)(TQT_B200_FLOAT_RUN_ARGS(CLAMPT));                                                             \
    };

/* ---- f32 family (src/gemm/gemm_f32_f32/) ---- */
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_f32_f32_f32, float)
TQT_B200_DECLARE_FLOAT_UP(gemm_1xnbias_clamp_f32_f32_f32p, float)
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_f32_f32_f32t, float)
TQT_B200_DECLARE_FLOAT_PP(gemm_1xnbias_clamp_f32_f32p_f32p, float)
TQT_B200_DECLARE_FLOAT_UU(gemm_mx1bias_clamp_f32_f32_f32, float)
TQT_B200_DECLARE_FLOAT_PP(gemm_mx1bias_clamp_f32_f32p_f32p, float)
/* f32 output from bf16 operands (src/gemm/gemm_bf16_bf16/) */
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_f32_bf16_bf16, float)
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_f32_bf16_bf16t, float)
TQT_B200_DECLARE_FLOAT_PP(gemm_1xnbias_clamp_f32_bf16p_bf16p, float)

#if !defined(TQT_B200_NO_HALF_TYPES)
/* ---- f16 family (src/gemm/gemm_f16_f16/) ---- */
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_f16_f16_f16, float16_t)
TQT_B200_DECLARE_FLOAT_UP(gemm_1xnbias_clamp_f16_f16_f16p, float16_t)
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_f16_f16_f16t, float16_t)
TQT_B200_DECLARE_FLOAT_PP(gemm_1xnbias_clamp_f16_f16p_f16p, float16_t)
TQT_B200_DECLARE_FLOAT_UU(gemm_mx1bias_clamp_f16_f16_f16, float16_t)
TQT_B200_DECLARE_FLOAT_PP(gemm_mx1bias_clamp_f16_f16p_f16p, float16_t)
/* ---- bf16 family (src/gemm/gemm_bf16_bf16/) ---- */
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_bf16_bf16_bf16, bfloat16_t)
TQT_B200_DECLARE_FLOAT_UP(gemm_1xnbias_clamp_bf16_bf16_bf16p, bfloat16_t)
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_bf16_bf16_bf16t, bfloat16_t)
TQT_B200_DECLARE_FLOAT_PP(gemm_1xnbias_clamp_bf16_bf16p_bf16p, bfloat16_t)
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_f16_bf16_bf16, float16_t)
TQT_B200_DECLARE_FLOAT_UU(gemm_1xnbias_clamp_f16_bf16_bf16t, float16_t)
TQT_B200_DECLARE_FLOAT_PP(gemm_1xnbias_clamp_f16_bf16p_bf16p, float16_t)
#endif

#ifdef __cplusplus
}
#endif

#endif /* TQT_B200_GEMM_FLOAT_H */
