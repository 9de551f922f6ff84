/*
 * int8 convolution wrappers: im2col (plain, or fused with the pack into the tensor-core block layout) followed by
 * the requantising GEMM of the same kernel type; and, at the end of this header, the implicit-GEMM types.  Same names and argument lists as the reference's conv_i8_i8
 * family with the variant suffix "_128x128_sm100a".
 *
 * Reference variants replaced (paths under src/conv/conv_i8_i8/):
 *   convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp/tqt_convcl_..._4x1vl_rvv.{h,cpp}
 *       channel-last input [D, H, W, C]; run_a_im2colpack (..._4x1vl_rvv.cpp:161-182) writes the packed A of
 *       gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp (rows = output positions (od, oh, ow), K order
 *       (kd, kh, kw, ic)); run_conv (:185-195) is that type's run_gemm; interface: ..._interface.h:20-78.
 *   convcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt/...   run_im2col = tqt_im2col_cl<int8_t>
 *       (src/common/tqt_conv.h:124-196) into a plain [M, K] matrix, run_conv = run_gemm of
 *       gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt.
 *   convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8/...    channel-first input [C, D, H, W]; run_im2col =
 *       tqt_im2col_cf<int8_t> (src/common/tqt_conv.h:52-121) into a plain [K, N] matrix (K order (ic, kd, kh, kw),
 *       N = output positions); the weights are the A operand; run_conv = run_gemm of
 *       gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8.
 *   convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p/...  run_b_im2colpack writes the packed B of
 *       gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p, run_conv = that type's run_gemm.
 *
 * Padding positions hold 0, as in the reference.  The activation and every matrix are device pointers; the
 * tqt_conv_params struct is a host struct read at call time.  Every extent, the number of output positions and
 * K = kernel volume x input channels per group must be below 2^31.  The packed matrices are caller-owned buffers of
 * get_*_im2colpack_size bytes; padding rows / columns of the last blocks are written as zeros.
 */
#ifndef TQT_B200_CONV_I8_I8_H
#define TQT_B200_CONV_I8_I8_H

#include "tqt_b200_common.h"
#include "tqt_b200_gemm_i8_i8.h"
#include "tqt_b200_gemm_siblings.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Same members as the reference's struct (src/common/tqt_conv.h:23-34).  Define TQT_B200_HAVE_CONV_PARAMS before
 * including this header when the reference's own header is in the same translation unit. */
#if !defined(TQT_B200_HAVE_CONV_PARAMS)
#define TQT_B200_HAVE_CONV_PARAMS
struct tqt_conv_params {
    size_t input_shape[3];  /* {input_d, input_h, input_w} */
    size_t output_shape[3]; /* {output_d, output_h, output_w}, computed by the caller */
    size_t kernel_shape[3];
    size_t stride[3];
    size_t dilation[3];
    size_t pad[3];
    size_t input_channel;
    size_t output_channel;
    size_t groups;
};
#endif

#define TQT_B200_CONV_COMMON_HELPERS(TYPE)                                                                            \
    size_t tqt_get_m_step_##TYPE##_128x128_sm100a(void);                                                               \
    size_t tqt_get_n_step_##TYPE##_128x128_sm100a(void);                                                               \
    size_t tqt_get_c_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldc);                           \
    size_t tqt_get_bias_offset_##TYPE##_128x128_sm100a(size_t idx);                                                    \
    size_t tqt_get_d_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldd);                           \
    size_t tqt_get_d_size_##TYPE##_128x128_sm100a(size_t m, size_t n);

#define TQT_B200_CONV_RUN_ARGS(PARAMS)                                                                                \
    size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B, size_t ldb,               \
        size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, int8_t clamp_min,           \
        int8_t clamp_max, const struct PARAMS *params

/* ---- channel-last, both operands packed ---------------------------------------------------------------- */
TQT_B200_CONV_COMMON_HELPERS(convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp)
size_t tqt_get_a_im2colpack_offset_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);
size_t tqt_get_b_packed_offset_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);
size_t tqt_get_a_im2colpack_size_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(size_t m, size_t k);
size_t tqt_get_b_packed_size_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(size_t n, size_t k);
void tqt_run_bt_pack_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed);
/* lda_packed: the K extent the packed buffer was sized with (>= K of the convolution); k_idx: multiple of
 * TQT_B200_K_STEP, already applied to A_packed by the caller through get_a_im2colpack_offset. */
void tqt_run_a_im2colpack_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t group_idx, const void *activation, size_t lda_packed, size_t k_idx, void *A_packed,
    const struct tqt_conv_params *params);
void tqt_run_conv_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    TQT_B200_CONV_RUN_ARGS(tqt_qai8_qai8_qsi8cx_params));

struct tqt_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_a_im2colpack_offset)(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);
    size_t (*get_b_packed_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t n_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    size_t (*get_a_im2colpack_size)(size_t m, size_t k);
    size_t (*get_b_packed_size)(size_t n, size_t k);
    void (*run_bt_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed);
    void (*run_a_im2colpack)(size_t group_idx, const void *activation, size_t lda_packed, size_t k_idx, void *A_packed,
                             const struct tqt_conv_params *params);
    void (*run_conv)(TQT_B200_CONV_RUN_ARGS(tqt_qai8_qai8_qsi8cx_params));
};

/* ---- channel-last, plain im2col matrix and transposed weights -------------------------------------------- */
TQT_B200_CONV_COMMON_HELPERS(convcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt)
size_t tqt_get_b_offset_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_128x128_sm100a(size_t n_idx, size_t k_idx,
                                                                                         size_t ldb);
size_t tqt_get_a_im2col_size_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_128x128_sm100a(size_t m, size_t k);
size_t tqt_get_a_im2col_offset_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_128x128_sm100a(size_t m_idx,
                                                                                                size_t k_idx,
                                                                                                size_t lda_im2col);
void tqt_run_im2col_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_128x128_sm100a(
    size_t group_idx, const void *activation, void *im2col_buf, const struct tqt_conv_params *params);
void tqt_run_conv_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_128x128_sm100a(
    TQT_B200_CONV_RUN_ARGS(tqt_qai8_qai8_qsi8cx_params));

struct tqt_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_b_offset)(size_t n_idx, size_t k_idx, size_t ldb);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t n_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    size_t (*get_a_im2col_size)(size_t m, size_t k);
    size_t (*get_a_im2col_offset)(size_t m_idx, size_t k_idx, size_t lda_im2col);
    void (*run_im2col)(size_t group_idx, const void *activation, void *im2col_buf, const struct tqt_conv_params *params);
    void (*run_conv)(TQT_B200_CONV_RUN_ARGS(tqt_qai8_qai8_qsi8cx_params));
};

/* ---- channel-first, plain matrices (weights = A [M, K], im2col = B [K, N]) --------------------------------- */
TQT_B200_CONV_COMMON_HELPERS(convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8)
size_t tqt_get_a_offset_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_128x128_sm100a(size_t m_idx, size_t k_idx,
                                                                                        size_t lda);
size_t tqt_get_b_im2col_size_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_128x128_sm100a(size_t k, size_t n);
size_t tqt_get_b_im2col_offset_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_128x128_sm100a(size_t n_idx,
                                                                                               size_t k_idx,
                                                                                               size_t ldb_im2col);
void tqt_run_im2col_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_128x128_sm100a(
    size_t group_idx, const void *activation, void *im2col_buf, const struct tqt_conv_params *params);
void tqt_run_conv_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_128x128_sm100a(
    TQT_B200_CONV_RUN_ARGS(tqt_qai8_qsi8dx_qai8_params));

struct tqt_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_a_offset)(size_t m_idx, size_t k_idx, size_t lda);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t m_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    size_t (*get_b_im2col_size)(size_t k, size_t n);
    size_t (*get_b_im2col_offset)(size_t n_idx, size_t k_idx, size_t ldb_im2col);
    void (*run_im2col)(size_t group_idx, const void *activation, void *im2col_buf, const struct tqt_conv_params *params);
    void (*run_conv)(TQT_B200_CONV_RUN_ARGS(tqt_qai8_qsi8dx_qai8_params));
};

/* ---- channel-first, both operands packed ----------------------------------------------------------------- */
TQT_B200_CONV_COMMON_HELPERS(convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p)
size_t tqt_get_a_packed_offset_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a(
    size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);
size_t tqt_get_b_im2colpack_offset_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a(
    size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);
size_t tqt_get_a_packed_size_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a(size_t m, size_t k);
size_t tqt_get_b_im2colpack_size_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a(size_t n, size_t k);
void tqt_run_a_pack_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a(
    size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A, void *A_packed);
void tqt_run_b_im2colpack_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a(
    size_t group_idx, const void *activation, size_t ldb_packed, size_t k_idx, void *B_packed,
    const struct tqt_conv_params *params);
void tqt_run_conv_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a(
    TQT_B200_CONV_RUN_ARGS(tqt_qai8_qsi8dx_qai8_params));

struct tqt_convcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_a_packed_offset)(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);
    size_t (*get_b_im2colpack_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t m_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    size_t (*get_a_packed_size)(size_t m, size_t k);
    size_t (*get_b_im2colpack_size)(size_t n, size_t k);
    void (*run_a_pack)(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A, void *A_packed);
    void (*run_b_im2colpack)(size_t group_idx, const void *activation, size_t ldb_packed, size_t k_idx, void *B_packed,
                             const struct tqt_conv_params *params);
    void (*run_conv)(TQT_B200_CONV_RUN_ARGS(tqt_qai8_qsi8dx_qai8_params));
};

/* ==== implicit-GEMM convolutions (reference: src/conv/igemm_i8_i8/) ========================================
 * No im2col matrix: run_igemm gathers the activation operand from `input` on the fly.  As in the reference
 * (igemmcl_..._qsi8cxp/tqt_igemmcl_..._4x1vl_rvv.cpp:178-298, igemmcf_..._qsi8dxp_qai8/tqt_igemmcf_..._1vlx4_rvv.cpp:185-303):
 *   - channel-last: rows of the GEMM are output positions m_idx .. m_idx + m, columns the n output channels the weight
 *     / bias / scale_b pointers start at; D is the base of the output matrix [positions, ldd]: row m_idx + i is written
 *     at D + (m_idx + i) * ldd (the row offset is NOT applied by the caller, the column offset is);
 *   - channel-first: rows are the m output channels the weight / bias / scale_a pointers start at, columns the output
 *     positions n_idx .. n_idx + n; D is the base of [channels, ldd] and column n_idx + j is written at D + i * ldd + n_idx + j;
 *   - k, C, ldc and the k indices are ignored (K follows from conv_params; no K slabs); a NULL conv_params or
 *     quant_params returns silently.
 * These four types run on the generic CUDA-core kernel with an im2col operand accessor. */
#define TQT_B200_IGEMM_CL_ARGS(PARAMS)                                                                                \
    size_t m, size_t n, size_t k, const void *input, size_t group_idx, size_t m_idx, size_t k_idx_a, const void *B,   \
        size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,                 \
        int8_t clamp_min, int8_t clamp_max, const struct tqt_conv_params *conv_params, const struct PARAMS *quant_params
#define TQT_B200_IGEMM_CF_ARGS(PARAMS)                                                                                \
    size_t m, size_t n, size_t k, const void *input, size_t group_idx, size_t n_idx, size_t k_idx_b, const void *A,   \
        size_t lda, size_t k_idx_a, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,                 \
        int8_t clamp_min, int8_t clamp_max, const struct tqt_conv_params *conv_params, const struct PARAMS *quant_params

/* ---- channel-last, packed weights ---- */
TQT_B200_CONV_COMMON_HELPERS(igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp)
size_t tqt_get_b_packed_offset_igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t n_idx, size_t k_idx,
                                                                                                 size_t ldb, size_t actual_n);
size_t tqt_get_b_packed_size_igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t n, size_t k);
void tqt_run_bt_pack_igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(
    size_t n, size_t k, size_t ldw, size_t ldw_packed, size_t k_idx, const void *weight, void *weight_packed);
void tqt_run_igemm_igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(
    TQT_B200_IGEMM_CL_ARGS(tqt_qai8_qai8_qsi8cx_params));

struct tqt_igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_b_packed_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t n_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    size_t (*get_b_packed_size)(size_t n, size_t k);
    void (*run_bt_pack)(size_t n, size_t k, size_t ldw, size_t ldw_packed, size_t k_idx, const void *weight,
                        void *weight_packed);
    void (*run_igemm)(TQT_B200_IGEMM_CL_ARGS(tqt_qai8_qai8_qsi8cx_params));
};

/* ---- channel-last, transposed weights [n, ldb] ---- */
TQT_B200_CONV_COMMON_HELPERS(igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt)
size_t tqt_get_b_offset_igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_128x128_sm100a(size_t n_idx, size_t k_idx,
                                                                                          size_t ldb);
void tqt_run_igemm_igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_128x128_sm100a(
    TQT_B200_IGEMM_CL_ARGS(tqt_qai8_qai8_qsi8cx_params));

struct tqt_igemmcl_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_b_offset)(size_t n_idx, size_t k_idx, size_t ldb);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t n_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    void (*run_igemm)(TQT_B200_IGEMM_CL_ARGS(tqt_qai8_qai8_qsi8cx_params));
};

/* ---- channel-first, plain weights [m, lda] ---- */
TQT_B200_CONV_COMMON_HELPERS(igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8)
size_t tqt_get_a_offset_igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_128x128_sm100a(size_t m_idx, size_t k_idx,
                                                                                         size_t lda);
void tqt_run_igemm_igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_128x128_sm100a(
    TQT_B200_IGEMM_CF_ARGS(tqt_qai8_qsi8dx_qai8_params));

struct tqt_igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_a_offset)(size_t m_idx, size_t k_idx, size_t lda);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t m_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    void (*run_igemm)(TQT_B200_IGEMM_CF_ARGS(tqt_qai8_qsi8dx_qai8_params));
};

/* ---- channel-first, packed weights ---- */
TQT_B200_CONV_COMMON_HELPERS(igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8)
size_t tqt_get_a_packed_offset_igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8_128x128_sm100a(size_t m_idx, size_t k_idx,
                                                                                                 size_t lda, size_t actual_m);
size_t tqt_get_a_packed_size_igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8_128x128_sm100a(size_t m, size_t k);
void tqt_run_a_pack_igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8_128x128_sm100a(
    size_t m, size_t k, size_t ldw, size_t ldw_packed, size_t k_idx, const void *weight, void *weight_packed);
void tqt_run_igemm_igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8_128x128_sm100a(
    TQT_B200_IGEMM_CF_ARGS(tqt_qai8_qsi8dx_qai8_params));

struct tqt_igemmcf_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_a_packed_offset)(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t m_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    size_t (*get_a_packed_size)(size_t m, size_t k);
    void (*run_a_pack)(size_t m, size_t k, size_t ldw, size_t ldw_packed, size_t k_idx, const void *weight,
                       void *weight_packed);
    void (*run_igemm)(TQT_B200_IGEMM_CF_ARGS(tqt_qai8_qsi8dx_qai8_params));
};

#ifdef __cplusplus
}
#endif

#endif /* TQT_B200_CONV_I8_I8_H */
