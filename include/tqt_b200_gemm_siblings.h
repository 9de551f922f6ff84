/*
 * The remaining kernel types of the three quantised GEMM families: the unpacked ("t" layouts) and
 * otherwise-packed siblings of the types in tqt_b200_gemm_i8_i8.h, tqt_b200_gemm_i8_i4.h and
 * tqt_b200_gemm_f16_i4.h.  Same contraction, different operand layout or epilogue.  The fully packed types (mx1bias
 * ..._qsi8dxp_qai8p, ..._qai8dxp_qsi8cxp) run on the tcgen05 CTA-pair kernel.  Types with a row-major ("unpacked")
 * operand run on the same tensor-core kernels, each stage fetched from the caller's matrix by tiled TMA loads, when
 * that operand's base address and row stride (in bytes) are multiples of 16; any other call runs on a generic
 * CUDA-core kernel (any alignment, any layout, much slower).  The packed B of the qai8dxp_qsi8cxp types is opaque
 * like every packed buffer: 16 KiB blocks followed by 128 int16 partial row sums each (get_b_packed_size /
 * get_b_packed_offset account for it).
 *
 * Reference variants replaced (paths under src/gemm/):
 *   gemm_i8_i4/gemm_1xnbias_clamp_{f32,f16,bf16}_qai8dx_qsi4cxt/tqt_gemm_..._4x1vl_rvv.h
 *       (run_gemm f32: ..._4x1vl_rvv.cpp:158-197)  A int8 [m,lda], B nibbles [n, ldb/2 bytes]
 *       (byte = (q_hi+8)<<4 | (q_lo+8), low nibble = even k), epilogue as the packed W4A8 types.
 *   gemm_i8_i8/gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt/...  A [m,lda], B [n,ldb] int8
 *   gemm_i8_i8/gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp/...  A [m,lda], B packed
 *       requantisation as gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp.
 *   gemm_i8_i8/gemm_1xnbias_clamp_{f32,f16}_qai8dx_qsi8cxt/...      A [m,lda], B [n,ldb] int8
 *   gemm_i8_i8/gemm_1xnbias_clamp_{f32,f16}_qai8dxp_qsi8cxp/...     both packed
 *       acc = sum_k (a - zero_point_a[m]) * b;  r = (float)acc * (scale_b[n] * scale_a[m]);  C is ignored
 *       (..._f32_qai8dxp_qsi8cxp_4x1vl_rvv.cpp:174);  f32: + bias, clamp;  f16: narrow to f16 first, then
 *       add the bias and clamp in f16 (tqt_kernel_gemm_qai8dx_qsi8cx_4x1vl_rvv.h:95-139, 167-176, 262-278).
 *   gemm_i8_i8/gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8/...   A [m,lda] int8, B [k,ldb] int8
 *   gemm_i8_i8/gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p/... both packed
 *       acc = C + A*B + bias[m];  per row  real = (double)scale_a[m] * (double)scale_b / (double)scale_d
 *       (row 0 for all rows when quant_channel_a == 1), then the same integer tail as the 1xnbias
 *       requantisation (..._qsi8dx_qai8_4x1vl_rvv.cpp:84-118, 141-163; tqt_kernel_gemm_i8_i8_4x1vl_rvv.h:264-330).
 *       zero_point_b is not applied by the kernel: callers fuse  bias - zero_point_b * sum_k a  into the bias.
 *   gemm_f16_i4/gemm_1xnbias_clamp_{f16,f32}_f16_qsi4c2t/tqt_gemm_..._8x2vl_rvv.h
 *       A f16 [m,lda], B nibbles [n, ldb/2 bytes], scale_b f16 [n, ldsb]; arithmetic as the packed W4A16 types.
 *
 * All data pointers are device pointers; the arrays inside the params structs are device arrays indexed
 * from the call's own first row / column; params == NULL returns silently, as in the reference.
 */
#ifndef TQT_B200_GEMM_SIBLINGS_H
#define TQT_B200_GEMM_SIBLINGS_H

#include "tqt_b200_common.h"
#include "tqt_b200_gemm_i8_i4.h"
#include "tqt_b200_gemm_i8_i8.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Same layouts as the reference's structs (src/gemm/gemm_i8_i8/tqt_params_i8_i8.h:26-41). */
struct tqt_qai8_qsi8dx_qai8_params {
    float *scale_a;
    int32_t quant_channel_a;
    float scale_b;
    int32_t zero_point_b;
    float scale_d;
    int32_t zero_point_d;
};

struct tqt_qai8dxp_qsi8cxp_params {
    float *scale_a;
    int32_t *zero_point_a;
    float *scale_b;
};

/* Offsets and sizes of a kernel type whose A and B are both unpacked. */
#define TQT_B200_DECLARE_UNPACKED_HELPERS(TYPE)                                                          \
    size_t tqt_get_m_step_##TYPE##_128x128_sm100a(void);                                                 \
    size_t tqt_get_n_step_##TYPE##_128x128_sm100a(void);                                                 \
    size_t tqt_get_a_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t k_idx, size_t lda);             \
    size_t tqt_get_b_offset_##TYPE##_128x128_sm100a(size_t n_idx, size_t k_idx, size_t ldb);             \
    size_t tqt_get_c_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldc);             \
    size_t tqt_get_bias_offset_##TYPE##_128x128_sm100a(size_t idx);                                      \
    size_t tqt_get_d_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldd);             \
    size_t tqt_get_d_size_##TYPE##_128x128_sm100a(size_t m, size_t n);

/* Offsets, sizes and pack entry points of a kernel type whose A and B are both packed int8. */
#define TQT_B200_DECLARE_PACKED_I8_HELPERS(TYPE)                                                                      \
    size_t tqt_get_m_step_##TYPE##_128x128_sm100a(void);                                                              \
    size_t tqt_get_n_step_##TYPE##_128x128_sm100a(void);                                                              \
    size_t tqt_get_a_packed_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m);  \
    size_t tqt_get_b_packed_offset_##TYPE##_128x128_sm100a(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);  \
    size_t tqt_get_c_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldc);                          \
    size_t tqt_get_bias_offset_##TYPE##_128x128_sm100a(size_t idx);                                                   \
    size_t tqt_get_d_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldd);                          \
    size_t tqt_get_d_size_##TYPE##_128x128_sm100a(size_t m, size_t n);                                                \
    size_t tqt_get_a_packed_size_##TYPE##_128x128_sm100a(size_t m, size_t k);                                         \
    size_t tqt_get_b_packed_size_##TYPE##_128x128_sm100a(size_t n, size_t k);                                         \
    void tqt_run_a_pack_##TYPE##_128x128_sm100a(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx,      \
                                                const void *A, void *A_packed);                                       \
    void tqt_run_b_pack_##TYPE##_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx,      \
                                                const void *B, void *B_packed);                                       \
    void tqt_run_bt_pack_##TYPE##_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx,     \
                                                 const void *B, void *B_packed);

/* The function-pointer table of a kernel type, member for member as the reference's <type>_interface.h
 * (src/gemm/<family>/<type>/tqt_<type>_interface.h): a caller fills it with this variant's symbols exactly as it
 * does with the RVV variant's (examples/gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp_rvv/..._rvv.cpp:28-41). */
#define TQT_B200_DECLARE_UNPACKED_UKERNEL(TYPE, CLAMPT, PARAMS)                                                        \
    struct tqt_##TYPE##_ukernel {                                                                                      \
        size_t (*get_m_step)(void);                                                                                    \
        size_t (*get_n_step)(void);                                                                                    \
        size_t (*get_a_offset)(size_t m_idx, size_t k_idx, size_t lda);                                                \
        size_t (*get_b_offset)(size_t n_idx, size_t k_idx, size_t ldb);                                                \
        size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);                                                \
        size_t (*get_bias_offset)(size_t idx);                                                                         \
        size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);                                                \
        size_t (*get_d_size)(size_t m, size_t n);                                                                      \
        void (*run_gemm)(size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B,       \
                         size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, \
                         CLAMPT clamp_min, CLAMPT clamp_max, const struct PARAMS *params);                             \
    };

#define TQT_B200_DECLARE_PACKED_I8_UKERNEL(TYPE, CLAMPT, PARAMS)                                                       \
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
        void (*run_a_pack)(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A,             \
                           void *A_packed);                                                                            \
        void (*run_b_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B,             \
                           void *B_packed);                                                                            \
        void (*run_bt_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B,            \
                            void *B_packed);                                                                           \
        void (*run_gemm)(size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a,       \
                         const void *B_packed, size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, \
                         CLAMPT clamp_min, CLAMPT clamp_max, const struct PARAMS *params);                             \
    };

/* ---- W4A8 on unpacked operands ----------------------------------------------------------------------- */
#define TQT_B200_DECLARE_W4A8_UNPACKED(TDNAME, TDTYPE)                                                                \
    TQT_B200_DECLARE_UNPACKED_HELPERS(gemm_1xnbias_clamp_##TDNAME##_qai8dx_qsi4cxt)                                   \
    void tqt_run_gemm_1xnbias_clamp_##TDNAME##_qai8dx_qsi4cxt_128x128_sm100a(                                         \
        size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B, size_t ldb,           \
        size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, TDTYPE clamp_min,           \
        TDTYPE clamp_max, const struct tqt_qai8dx_qsi4cx_params *params);                                             \
    TQT_B200_DECLARE_UNPACKED_UKERNEL(gemm_1xnbias_clamp_##TDNAME##_qai8dx_qsi4cxt, TDTYPE, tqt_qai8dx_qsi4cx_params)

TQT_B200_DECLARE_W4A8_UNPACKED(f32, float)
#if !defined(TQT_B200_NO_HALF_TYPES)
TQT_B200_DECLARE_W4A8_UNPACKED(f16, float16_t)
TQT_B200_DECLARE_W4A8_UNPACKED(bf16, bfloat16_t)
#endif

/* ---- static W8A8 requantisation, 1xN bias: A unpacked, B transposed-unpacked or packed ----------------- */
TQT_B200_DECLARE_UNPACKED_HELPERS(gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt)
void tqt_run_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B, size_t ldb,
    size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, int8_t clamp_min,
    int8_t clamp_max, const struct tqt_qai8_qai8_qsi8cx_params *params);
TQT_B200_DECLARE_UNPACKED_UKERNEL(gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxt, int8_t, tqt_qai8_qai8_qsi8cx_params)

size_t tqt_get_m_step_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(void);
size_t tqt_get_n_step_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(void);
size_t tqt_get_a_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t m_idx, size_t k_idx,
                                                                                       size_t lda);
size_t tqt_get_b_packed_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t n_idx,
                                                                                              size_t k_idx,
                                                                                              size_t ldb,
                                                                                              size_t actual_n);
size_t tqt_get_c_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t m_idx, size_t n_idx,
                                                                                       size_t ldc);
size_t tqt_get_bias_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t n_idx);
size_t tqt_get_d_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t m_idx, size_t n_idx,
                                                                                       size_t ldd);
size_t tqt_get_d_size_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t m, size_t n);
size_t tqt_get_b_packed_size_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t n, size_t k);
void tqt_run_b_pack_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t n, size_t k, size_t ldb,
                                                                                   size_t ldb_packed, size_t k_idx,
                                                                                   const void *B, void *B_packed);
void tqt_run_bt_pack_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(size_t n, size_t k, size_t ldb,
                                                                                    size_t ldb_packed, size_t k_idx,
                                                                                    const void *B, void *B_packed);
void tqt_run_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B_packed, size_t ldb,
    size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, int8_t clamp_min,
    int8_t clamp_max, const struct tqt_qai8_qai8_qsi8cx_params *params);
/* A in its original layout, B packed (src/gemm/gemm_i8_i8/gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp/
 * tqt_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_interface.h:52-67). */
struct tqt_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8_qsi8cxp_ukernel {
    size_t (*get_m_step)(void);
    size_t (*get_n_step)(void);
    size_t (*get_a_offset)(size_t m_idx, size_t k_idx, size_t lda);
    size_t (*get_b_packed_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n);
    size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);
    size_t (*get_bias_offset)(size_t n_idx);
    size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);
    size_t (*get_d_size)(size_t m, size_t n);
    size_t (*get_b_packed_size)(size_t n, size_t k);
    void (*run_b_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed);
    void (*run_bt_pack)(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed);
    void (*run_gemm)(size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B_packed,
                     size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,
                     int8_t clamp_min, int8_t clamp_max, const struct tqt_qai8_qai8_qsi8cx_params *params);
};

/* ---- static W8A8 requantisation, Mx1 bias, per-row scale of A ------------------------------------------ */
TQT_B200_DECLARE_UNPACKED_HELPERS(gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8)
void tqt_run_gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B, size_t ldb,
    size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, int8_t clamp_min,
    int8_t clamp_max, const struct tqt_qai8_qsi8dx_qai8_params *params);
TQT_B200_DECLARE_UNPACKED_UKERNEL(gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8, int8_t, tqt_qai8_qsi8dx_qai8_params)

TQT_B200_DECLARE_PACKED_I8_HELPERS(gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p)
void tqt_run_gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a, const void *B_packed,
    size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,
    int8_t clamp_min, int8_t clamp_max, const struct tqt_qai8_qsi8dx_qai8_params *params);
TQT_B200_DECLARE_PACKED_I8_UKERNEL(gemm_mx1bias_reqi32toi8_clamp_qai8_qsi8dxp_qai8p, int8_t, tqt_qai8_qsi8dx_qai8_params)

/* ---- dynamic-activation W8A8 with float output (qai8dx x qsi8cx) --------------------------------------- */
#define TQT_B200_DECLARE_DXCX(TDNAME, TDTYPE)                                                                         \
    TQT_B200_DECLARE_UNPACKED_HELPERS(gemm_1xnbias_clamp_##TDNAME##_qai8dx_qsi8cxt)                                   \
    void tqt_run_gemm_1xnbias_clamp_##TDNAME##_qai8dx_qsi8cxt_128x128_sm100a(                                         \
        size_t m, size_t n, size_t k, const void *A, size_t lda, size_t k_idx_a, const void *B, size_t ldb,           \
        size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, TDTYPE clamp_min,           \
        TDTYPE clamp_max, const struct tqt_qai8dxp_qsi8cxp_params *params);                                           \
    TQT_B200_DECLARE_UNPACKED_UKERNEL(gemm_1xnbias_clamp_##TDNAME##_qai8dx_qsi8cxt, TDTYPE, tqt_qai8dxp_qsi8cxp_params) \
    TQT_B200_DECLARE_PACKED_I8_HELPERS(gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi8cxp)                                 \
    void tqt_run_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi8cxp_128x128_sm100a(                                        \
        size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a, const void *B_packed,         \
        size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,                 \
        TDTYPE clamp_min, TDTYPE clamp_max, const struct tqt_qai8dxp_qsi8cxp_params *params);                         \
    TQT_B200_DECLARE_PACKED_I8_UKERNEL(gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi8cxp, TDTYPE, tqt_qai8dxp_qsi8cxp_params)

TQT_B200_DECLARE_DXCX(f32, float)
#if !defined(TQT_B200_NO_HALF_TYPES)
TQT_B200_DECLARE_DXCX(f16, float16_t)
#endif

/* ---- W4A16 on unpacked operands ---------------------------------------------------------------------- */
#define TQT_B200_DECLARE_W4A16_UNPACKED(TDNAME, TDTYPE)                                                               \
    size_t tqt_get_m_step_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(void);                             \
    size_t tqt_get_n_step_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(void);                             \
    size_t tqt_get_a_offset_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(size_t m_idx, size_t k_idx,      \
                                                                                     size_t lda, size_t bl);          \
    size_t tqt_get_b_offset_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(size_t n_idx, size_t k_idx,      \
                                                                                     size_t ldb, size_t bl);          \
    size_t tqt_get_scale_b_offset_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(size_t n_idx,              \
                                                                                           size_t b_idx,              \
                                                                                           size_t ldsb);              \
    size_t tqt_get_c_offset_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(size_t m_idx, size_t n_idx,      \
                                                                                     size_t ldc);                     \
    size_t tqt_get_bias_offset_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(size_t n_idx);                \
    size_t tqt_get_d_offset_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(size_t m_idx, size_t n_idx,      \
                                                                                     size_t ldd);                     \
    size_t tqt_get_d_size_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(size_t m, size_t n);               \
    void tqt_run_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_128x128_sm100a(                                            \
        size_t m, size_t n, size_t k, size_t bl, const void *A, size_t lda, size_t k_idx_a, const void *B,            \
        size_t ldb, size_t k_idx_b, const void *scale_b, size_t ldsb, const void *C, size_t ldc, void *D,             \
        size_t ldd, const void *bias, TDTYPE clamp_min, TDTYPE clamp_max);                                            \
    struct tqt_gemm_1xnbias_clamp_##TDNAME##_f16_qsi4c2t_ukernel {                                                    \
        size_t (*get_m_step)(void);                                                                                   \
        size_t (*get_n_step)(void);                                                                                   \
        size_t (*get_a_offset)(size_t m_idx, size_t k_idx, size_t lda, size_t bl);                                    \
        size_t (*get_b_offset)(size_t n_idx, size_t k_idx, size_t ldb, size_t bl);                                    \
        size_t (*get_scale_b_offset)(size_t n_idx, size_t b_idx, size_t ldsb);                                        \
        size_t (*get_c_offset)(size_t m_idx, size_t n_idx, size_t ldc);                                               \
        size_t (*get_bias_offset)(size_t n_idx);                                                                      \
        size_t (*get_d_offset)(size_t m_idx, size_t n_idx, size_t ldd);                                               \
        size_t (*get_d_size)(size_t m, size_t n);                                                                     \
        void (*run_gemm)(size_t m, size_t n, size_t k, size_t bl, const void *A, size_t lda, size_t k_idx_a,          \
                         const void *B, size_t ldb, size_t k_idx_b, const void *scale_b, size_t ldsb, const void *C,  \
                         size_t ldc, void *D, size_t ldd, const void *bias, TDTYPE clamp_min, TDTYPE clamp_max);      \
    };

TQT_B200_DECLARE_W4A16_UNPACKED(f32, float)
#if !defined(TQT_B200_NO_HALF_TYPES)
TQT_B200_DECLARE_W4A16_UNPACKED(f16, float16_t)
#endif

#ifdef __cplusplus
}
#endif

#endif /* TQT_B200_GEMM_SIBLINGS_H */
