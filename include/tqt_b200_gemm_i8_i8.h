/*
 * W8A8 GEMM micro-kernels for B200 (int8 x int8 -> int32 accumulate).
 *
 * Kernel types and the reference variants they replace (paths under src/gemm/gemm_i8_i8/):
 *   gemm_clamp_i32_i8_i8                       gemm_clamp_i32_i8_i8/tqt_gemm_clamp_i32_i8_i8_4x1vl_rvv.h:24-108
 *                                              (run_gemm: ..._4x1vl_rvv.cpp:118-146)
 *       D = clamp(C + A*B);  A [m,k] int8 row-major, B [k,n] int8 row-major, C/D [m,n] int32.
 *   gemm_clamp_i32_i8p_i8p                     gemm_clamp_i32_i8p_i8p/tqt_gemm_clamp_i32_i8p_i8p_4x1vl_rvv.h:31-166
 *       same result from packed operands.
 *   gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp
 *                                              gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp/
 *                                              tqt_gemm_..._4x1vl_rvv.h:36-183 (run_gemm: ..._4x1vl_rvv.cpp:177-241)
 *       acc = C + A*B + bias[n] (int32, wrapping); per column
 *       real = (double)scale_a * (double)scale_b[n] / (double)scale_d  (column 0 for all when
 *       quant_channel_b == 1); (mult, s) = tqt_quantize_multiplier(real); sh = -s - 1;
 *       t = high32((int64)acc * mult); t >>= (sh & 31) (arithmetic, no rounding); t += zero_point_d;
 *       saturate to int16, then to int8; clamp to [clamp_min, clamp_max].
 *       zero_point_a is NOT applied by the kernel: callers fuse  bias - zero_point_a * sum_k b  into
 *       the bias, as the reference's callers do (test/common/test_common.h:280-290).
 *
 * Packed layouts (opaque): both operands are stored as [ceil(rows/128)][ceil(k/128)] blocks of
 * 128 rows x 128 int8 (16 KiB each) in the 128-byte-swizzled K-major order that tcgen05.mma reads
 * from shared memory; padding is zero.  run_b_pack takes B as [k,n] row-major, run_bt_pack as
 * [n,k] row-major; both produce the same packed buffer.
 *
 * params->scale_b is a DEVICE array indexed from the call's own first column.
 */
#ifndef TQT_B200_GEMM_I8_I8_H
#define TQT_B200_GEMM_I8_I8_H

#include "tqt_b200_common.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Same layout as the reference's struct (src/gemm/gemm_i8_i8/tqt_params_i8_i8.h:16-24). */
struct tqt_qai8_qai8_qsi8cx_params {
    float scale_a;
    int32_t zero_point_a;
    float *scale_b;
    int32_t quant_channel_b;
    float scale_d;
    int32_t zero_point_d;
};

/* ---- gemm_clamp_i32_i8_i8 (unpacked operands) ------------------------------------------------ */
size_t tqt_get_m_step_gemm_clamp_i32_i8_i8_128x128_sm100a(void);
size_t tqt_get_n_step_gemm_clamp_i32_i8_i8_128x128_sm100a(void);
size_t tqt_get_a_offset_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m_idx, size_t k_idx, size_t lda);
size_t tqt_get_b_offset_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t n_idx, size_t k_idx, size_t ldb);
size_t tqt_get_c_offset_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldc);
size_t tqt_get_d_offset_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldd);
size_t tqt_get_d_size_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m, size_t n);
void tqt_run_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m, size_t n, size_t k, const void *A, size_t lda,
                                                 size_t k_idx_a, const void *B, size_t ldb, size_t k_idx_b,
                                                 const void *C, size_t ldc, void *D, size_t ldd,
                                                 int32_t clamp_min, int32_t clamp_max);

/* Mirrors gemm_clamp_i32_i8_i8/tqt_gemm_clamp_i32_i8_i8_interface.h:20-50. */
struct tqt_gemm_clamp_i32_i8_i8_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_a_offset)(size_t m_idx, size_t k_idx, size_t lda);
    size_t (*get_b_offset)(size_t n_idx, size_t k_idx, size_t ldb);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    void (*run_gemm)(size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B,
                     size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd,
                     int32_t clamp_min, int32_t clamp_max);
};

/* ---- gemm_clamp_i32_i8p_i8p (packed operands) ------------------------------------------------ */
size_t tqt_get_m_step_gemm_clamp_i32_i8p_i8p_128x128_sm100a(void);
size_t tqt_get_n_step_gemm_clamp_i32_i8p_i8p_128x128_sm100a(void);
size_t tqt_get_a_packed_offset_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t m_idx, size_t k_idx, size_t lda,
                                                                     size_t actual_m);
size_t tqt_get_b_packed_offset_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t n_idx, size_t k_idx, size_t ldb,
                                                                     size_t actual_n);
size_t tqt_get_c_offset_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldc);
size_t tqt_get_d_offset_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldd);
size_t tqt_get_d_size_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t m, size_t n);
size_t tqt_get_a_packed_size_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t m, size_t k);
size_t tqt_get_b_packed_size_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t n, size_t k);
void tqt_run_a_pack_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t m, size_t k, size_t lda, size_t lda_packed,
                                                          size_t k_idx, const void *A, void *A_packed);
void tqt_run_b_pack_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed,
                                                          size_t k_idx, const void *B, void *B_packed);
void tqt_run_bt_pack_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed,
                                                           size_t k_idx, const void *B, void *B_packed);
void tqt_run_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t m, size_t n, size_t k, const void *A_packed,
                                                   size_t lda, size_t k_idx_a, const void *B_packed, size_t ldb,
                                                   size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd,
                                                   int32_t clamp_min, int32_t clamp_max);

/* Mirrors gemm_clamp_i32_i8p_i8p/tqt_gemm_clamp_i32_i8p_i8p_interface.h. */
struct tqt_gemm_clamp_i32_i8p_i8p_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_a_packed_offset)(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);
    size_t (*get_b_packed_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    size_t (*get_a_packed_size)(size_t m, size_t k);
    size_t (*get_b_packed_size)(size_t n, size_t k);
    void (*run_a_pack)(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A,
                       void *A_packed);
    void (*run_b_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B,
                       void *B_packed);
    void (*run_bt_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B,
                        void *B_packed);
    void (*run_gemm)(size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a,
                     const void *B_packed, size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D,
                     size_t ldd, int32_t clamp_min, int32_t clamp_max);
};

/* ---- gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp (static W8A8, int8 out) ------------------ */
size_t tqt_get_m_step_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(void);
size_t tqt_get_n_step_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(void);
size_t tqt_get_a_packed_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);
size_t tqt_get_b_packed_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);
size_t tqt_get_c_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(size_t m_idx,
                                                                                        size_t n_idx,
                                                                                        size_t ldc);
size_t tqt_get_bias_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(size_t n_idx);
size_t tqt_get_d_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(size_t m_idx,
                                                                                        size_t n_idx,
                                                                                        size_t ldd);
size_t tqt_get_d_size_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(size_t m, size_t n);
size_t tqt_get_a_packed_size_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(size_t m,
                                                                                             size_t k);
size_t tqt_get_b_packed_size_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(size_t n,
                                                                                             size_t k);
void tqt_run_a_pack_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A, void *A_packed);
void tqt_run_b_pack_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed);
void tqt_run_bt_pack_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed);
void tqt_run_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a, const void *B_packed,
    size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,
    int8_t clamp_min, int8_t clamp_max, const struct tqt_qai8_qai8_qsi8cx_params *params);

/* Mirrors gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp/tqt_gemm_..._interface.h. */
struct tqt_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_a_packed_offset)(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);
    size_t (*get_b_packed_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t n_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    size_t (*get_a_packed_size)(size_t m, size_t k);
    size_t (*get_b_packed_size)(size_t n, size_t k);
    void (*run_a_pack)(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A,
                       void *A_packed);
    void (*run_b_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B,
                       void *B_packed);
    void (*run_bt_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B,
                        void *B_packed);
    void (*run_gemm)(size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a,
                     const void *B_packed, size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D,
                     size_t ldd, const void *bias, int8_t clamp_min, int8_t clamp_max,
                     const struct tqt_qai8_qai8_qsi8cx_params *params);
};

#ifdef __cplusplus
}
#endif

#endif /* TQT_B200_GEMM_I8_I8_H */
