// The C ABI: every exported entry point of the library.  Compiled by g++ (the f16 / bf16 kernel
// types take _Float16 / __bf16 clamp arguments by value, as the reference's prototypes do).
// Argument checks mirror the reference's TQT_ASSUME preconditions but never abort: a failed check
// records TQT_CUDA_INVALID_ARGUMENT for tqt_cuda_get_last_status() and returns without launching.
#include "../../include/tqt_b200_conv_i8_i8.h"
#include "../../include/tqt_b200_ext.h"
#include "../../include/tqt_b200_gemm_f16_i4.h"
#include "../../include/tqt_b200_gemm_float.h"
#include "../../include/tqt_b200_gemm_i8_i4.h"
#include "../../include/tqt_b200_gemm_i8_i8.h"
#include "../../include/tqt_b200_gemm_siblings.h"
#include "tqt_internal.h"

using namespace tqt;

namespace {

thread_local void *t_stream = nullptr;
thread_local int t_status = TQT_CUDA_OK;
thread_local int t_cuda_error = 0;
thread_local size_t t_n_replicas = 0;
thread_local const char *t_replica_local = nullptr;
thread_local size_t t_replica_bytes = 0;
thread_local long long t_replica_delta[7] = {0, 0, 0, 0, 0, 0, 0};

inline void set_result(Result r)
{
    t_status = r.status;
    t_cuda_error = r.cuda_error;
}
inline void set_invalid() { set_result(Result{kInvalid, 0}); }
inline void set_ok() { set_result(Result{kOk, 0}); }

constexpr size_t M_STEP = TQT_B200_M_STEP, N_STEP = TQT_B200_N_STEP, K_STEP = TQT_B200_K_STEP;

// ---- offsets and sizes of the packed layouts ------------------------------------------------------
inline size_t packed_offset(size_t idx, size_t k_idx, size_t ld, size_t kblk, size_t block_bytes)
{
    return ((idx / kTileRows) * ceil_div(ld, kblk) + k_idx / kblk) * block_bytes;
}
inline size_t packed_size(size_t rows, size_t k, size_t kblk, size_t block_bytes)
{
    return ceil_div(rows, kTileRows) * ceil_div(k, kblk) * block_bytes;
}

inline GemmCommon common(size_t m, size_t n, size_t k, const void *A, size_t lda, const void *B, size_t ldb,
                         const void *C, size_t ldc, void *D, size_t ldd, const void *bias)
{
    GemmCommon g;
    g.m = m; g.n = n; g.k = k;
    g.A = A; g.lda = lda;
    g.B = B; g.ldb = ldb;
    g.C = C; g.ldc = ldc;
    g.D = D; g.ldd = ldd;
    g.bias = bias;
    g.stream = t_stream;
    g.n_replicas = t_n_replicas;
    for (size_t i = 0; i < t_n_replicas; ++i) g.replica_delta[i] = t_replica_delta[i];
    return g;
}

inline bool ptrs_ok(size_t m, size_t n, const void *A, const void *B, const void *D)
{
    return m == 0 || n == 0 || (A && B && D);
}

// While output replicas are set, every element the call stores, [D, D + ((m-1)*ldd + n) * elem), must lie inside
// the registered local buffer: the replica stores go to the same offsets of buffers on other GPUs, so an output
// outside the registered range would be written at arbitrary peer addresses.
inline bool replicas_cover(size_t m, size_t n, const void *D, size_t ldd, size_t elem)
{
    if (t_n_replicas == 0 || m == 0 || n == 0) return true;
    const char *d0 = static_cast<const char *>(D);
    const size_t span = ((m - 1) * ldd + n) * elem;
    return d0 >= t_replica_local && span <= t_replica_bytes &&
           (size_t)(d0 - t_replica_local) <= t_replica_bytes - span;
}

void run_pack_a_i8(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A, void *A_packed)
{
    if ((m && k && (!A || !A_packed)) || k_idx % K_STEP) return set_invalid();
    set_result(launch_pack_rows(t_stream, m, k, lda, lda_packed, A, A_packed, 1, false));
}
void run_pack_bt_i8(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed)
{
    if ((n && k && (!B || !B_packed)) || k_idx % K_STEP) return set_invalid();
    set_result(launch_pack_rows(t_stream, n, k, ldb, ldb_packed, B, B_packed, 1, false));
}
void run_pack_b_i8(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed)
{
    if ((n && k && (!B || !B_packed)) || k_idx % K_STEP) return set_invalid();
    set_result(launch_pack_rows(t_stream, n, k, ldb, ldb_packed, B, B_packed, 1, true));
}
void run_pack_bt_i4(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed,
                    bool c2)
{
    if ((n && k && (!B || !B_packed)) || k_idx % K_STEP || (k & 1) || (ldb & 1)) return set_invalid();
    set_result(launch_pack_i4(t_stream, n, k, ldb / 2, ldb_packed, B, B_packed, c2));
}

void run_w4a8(size_t m, size_t n, size_t k, const void *A_packed, size_t lda, const void *B_packed, size_t ldb,
              const void *C, size_t ldc, void *D, size_t ldd, const void *bias, float cmin, float cmax,
              const struct tqt_qai8dx_qsi4cx_params *params, Dtype td)
{
    if (!params) return set_ok();  // the reference returns silently
    if (!ptrs_ok(m, n, A_packed, B_packed, D) || (k & 1)) return set_invalid();
    if (m && n && (!params->scale_a || !params->zero_point_a || !params->scale_b)) return set_invalid();
    // The reference strides the packed operands by the call's k and ignores lda / ldb, which is the same
    // thing whenever lda == ldb == k, the only way its callers use this kernel type.  Here a larger lda / ldb
    // names the K extent the packed buffers were built for, so that a K-slab call (k < lda, operands offset
    // with get_*_packed_offset(idx, k_idx, ld, ...)) finds its blocks; smaller values fall back to k.
    if (lda < k) lda = k;
    if (ldb < k) ldb = k;
    if (!replicas_cover(m, n, D, ldd, td == Dtype::F32 ? 4 : 2)) return set_invalid();
    GemmCommon g = common(m, n, k, A_packed, lda, B_packed, ldb, C, ldc, D, ldd, bias);
    W4A8Params p{params->scale_a, params->zero_point_a, params->scale_b};
    set_result(launch_gemm_w4a8(g, p, td, cmin, cmax, env_path()));
}

void run_w4a16(size_t m, size_t n, size_t k, size_t bl, const void *A_packed, size_t lda, const void *B_packed,
               size_t ldb, const void *scale_b, size_t ldsb, const void *C, size_t ldc, void *D, size_t ldd,
               const void *bias, float cmin, float cmax, Dtype td)
{
    if (!ptrs_ok(m, n, A_packed, B_packed, D)) return set_invalid();
    if (bl < 2 || (bl & 1) || (k % bl) || (m && n && k && !scale_b)) return set_invalid();
    if (!replicas_cover(m, n, D, ldd, td == Dtype::F32 ? 4 : 2)) return set_invalid();
    GemmCommon g = common(m, n, k, A_packed, lda, B_packed, ldb, C, ldc, D, ldd, bias);
    set_result(launch_gemm_w4a16(g, bl, scale_b, ldsb, td, cmin, cmax, env_path()));
}

void run_quant(size_t m, size_t k, const void *A, size_t lda, void *out, size_t ldq, bool packed, float *scale_a,
               int32_t *zp_a, Dtype ta)
{
    if (m && k && (!A || !out || !scale_a || !zp_a)) return set_invalid();
    set_result(launch_quant_qai8dx(t_stream, m, k, A, lda, ta, out, ldq, packed, scale_a, zp_a));
}

// Quantise the activations and run the W4A8 GEMM: one cooperative launch where the shape allows (the GEMM kernel
// quantises its own activations before its mainloop), else the quantiser and the GEMM as two launches.
void run_quant_w4a8(size_t m, size_t n, size_t k, const void *A, size_t lda, int a_type, void *A_packed, float *scale_a,
                    int32_t *zp_a, const void *B_packed, size_t ldb, const void *C, size_t ldc, void *D, size_t ldd,
                    const void *bias, float cmin, float cmax, const float *scale_b, Dtype td)
{
    if (a_type < 0 || a_type > 2 || (k & 1)) return set_invalid();
    if (m && n && (!A || !A_packed || !scale_a || !zp_a || !B_packed || !D || !scale_b)) return set_invalid();
    if (m == 0 || n == 0) return set_ok();
    if (ldb < k) ldb = k;
    if (!replicas_cover(m, n, D, ldd, td == Dtype::F32 ? 4 : 2)) return set_invalid();
    const Dtype ta = (Dtype)a_type;
    note_kernel(kKernelNone);
    GemmCommon g = common(m, n, k, A_packed, k, B_packed, ldb, C, ldc, D, ldd, bias);
    W4A8Params p{scale_a, zp_a, scale_b};
    if (ta != Dtype::F32 && env_path() == Path::Auto && m > 16) {
        Result r = umma_gemm_w4a8_fusedq(g, p, td, cmin, cmax, A, lda, ta == Dtype::BF16);
        if (r.status != kUnsupported) return set_result(r);
    }
    Result q = launch_quant_qai8dx(t_stream, m, k, A, lda, ta, A_packed, 0, true, scale_a, zp_a);
    if (q.status != kOk) return set_result(q);
    set_result(launch_gemm_w4a8(g, p, td, cmin, cmax, env_path()));
}

}  // namespace

extern "C" {

// ---- status / stream ---------------------------------------------------------------------------------
void tqt_cuda_set_stream(void *stream) { t_stream = stream; }
void *tqt_cuda_get_stream(void) { return t_stream; }
int tqt_cuda_get_last_status(void) { return t_status; }
int tqt_cuda_get_last_cuda_error(void) { return t_cuda_error; }
int tqt_cuda_read_device_fault(void) { return read_device_fault(t_stream); }
const char *tqt_cuda_version(void) { return "torq-tile-b200 0.1 (sm_100a)"; }

// ---- gemm_clamp_i32_i8_i8 ---------------------------------------------------------------------------
size_t tqt_get_m_step_gemm_clamp_i32_i8_i8_128x128_sm100a(void) { return M_STEP; }
size_t tqt_get_n_step_gemm_clamp_i32_i8_i8_128x128_sm100a(void) { return N_STEP; }
size_t tqt_get_a_offset_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m_idx, size_t k_idx, size_t lda)
{
    return (m_idx * lda + k_idx) * sizeof(int8_t);
}
size_t tqt_get_b_offset_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t n_idx, size_t k_idx, size_t ldb)
{
    return (k_idx * ldb + n_idx) * sizeof(int8_t);
}
size_t tqt_get_c_offset_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldc)
{
    return (m_idx * ldc + n_idx) * sizeof(int32_t);
}
size_t tqt_get_d_offset_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldd)
{
    return (m_idx * ldd + n_idx) * sizeof(int32_t);
}
size_t tqt_get_d_size_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m, size_t n) { return m * n * sizeof(int32_t); }
void tqt_run_gemm_clamp_i32_i8_i8_128x128_sm100a(size_t m, size_t n, size_t k, const void *A, size_t lda,
                                                 size_t k_idx_a, const void *B, size_t ldb, size_t k_idx_b,
                                                 const void *C, size_t ldc, void *D, size_t ldd, int32_t clamp_min,
                                                 int32_t clamp_max)
{
    (void)k_idx_a;
    (void)k_idx_b;
    if (m && n && (!D || (k && (!A || !B)))) return set_invalid();
    GemmCommon g = common(m, n, k, A, lda, B, ldb, C, ldc, D, ldd, nullptr);
    set_result(launch_gemm_i32(g, false, clamp_min, clamp_max, env_path()));
}

// ---- packed int8 kernel types: helpers shared by i8p_i8p and the requant kernel ----------------------
#define TQT_DEFINE_I8_PACKED_HELPERS(TYPE, DSIZE, WITH_BIAS)                                                           \
    size_t tqt_get_m_step_##TYPE##_128x128_sm100a(void) { return M_STEP; }                                             \
    size_t tqt_get_n_step_##TYPE##_128x128_sm100a(void) { return N_STEP; }                                             \
    size_t tqt_get_a_packed_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t k_idx, size_t lda, size_t actual_m)    \
    {                                                                                                                  \
        (void)actual_m;                                                                                                \
        return packed_offset(m_idx, k_idx, lda, kI8BlockK, kI8BlockBytes);                                             \
    }                                                                                                                  \
    size_t tqt_get_b_packed_offset_##TYPE##_128x128_sm100a(size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n)    \
    {                                                                                                                  \
        (void)actual_n;                                                                                                \
        return packed_offset(n_idx, k_idx, ldb, kI8BlockK, kI8BlockBytes);                                             \
    }                                                                                                                  \
    size_t tqt_get_c_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldc)                            \
    {                                                                                                                  \
        return (m_idx * ldc + n_idx) * sizeof(int32_t);                                                                \
    }                                                                                                                  \
    size_t tqt_get_d_offset_##TYPE##_128x128_sm100a(size_t m_idx, size_t n_idx, size_t ldd)                            \
    {                                                                                                                  \
        return (m_idx * ldd + n_idx) * (DSIZE);                                                                        \
    }                                                                                                                  \
    size_t tqt_get_d_size_##TYPE##_128x128_sm100a(size_t m, size_t n) { return m * n * (DSIZE); }                      \
    size_t tqt_get_a_packed_size_##TYPE##_128x128_sm100a(size_t m, size_t k)                                           \
    {                                                                                                                  \
        return packed_size(m, k, kI8BlockK, kI8BlockBytes);                                                            \
    }                                                                                                                  \
    size_t tqt_get_b_packed_size_##TYPE##_128x128_sm100a(size_t n, size_t k)                                           \
    {                                                                                                                  \
        return packed_size(n, k, kI8BlockK, kI8BlockBytes);                                                            \
    }                                                                                                                  \
    void tqt_run_a_pack_##TYPE##_128x128_sm100a(size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx,       \
                                                const void *A, void *A_packed)                                         \
    {                                                                                                                  \
        run_pack_a_i8(m, k, lda, lda_packed, k_idx, A, A_packed);                                                      \
    }                                                                                                                  \
    void tqt_run_b_pack_##TYPE##_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx,       \
                                                const void *B, void *B_packed)                                         \
    {                                                                                                                  \
        run_pack_b_i8(n, k, ldb, ldb_packed, k_idx, B, B_packed);                                                      \
    }                                                                                                                  \
    void tqt_run_bt_pack_##TYPE##_128x128_sm100a(size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx,      \
                                                 const void *B, void *B_packed)                                        \
    {                                                                                                                  \
        run_pack_bt_i8(n, k, ldb, ldb_packed, k_idx, B, B_packed);                                                     \
    }

TQT_DEFINE_I8_PACKED_HELPERS(gemm_clamp_i32_i8p_i8p, sizeof(int32_t), 0)
TQT_DEFINE_I8_PACKED_HELPERS(gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp, sizeof(int8_t), 1)

size_t tqt_get_bias_offset_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(size_t n_idx)
{
    return n_idx * sizeof(int32_t);
}

void tqt_run_gemm_clamp_i32_i8p_i8p_128x128_sm100a(size_t m, size_t n, size_t k, const void *A_packed, size_t lda,
                                                   size_t k_idx_a, const void *B_packed, size_t ldb, size_t k_idx_b,
                                                   const void *C, size_t ldc, void *D, size_t ldd, int32_t clamp_min,
                                                   int32_t clamp_max)
{
    (void)k_idx_a;
    (void)k_idx_b;
    if (!ptrs_ok(m, n, A_packed, B_packed, D)) return set_invalid();
    GemmCommon g = common(m, n, k, A_packed, lda, B_packed, ldb, C, ldc, D, ldd, nullptr);
    set_result(launch_gemm_i32(g, true, clamp_min, clamp_max, env_path()));
}

void tqt_run_gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a, const void *B_packed,
    size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,
    int8_t clamp_min, int8_t clamp_max, const struct tqt_qai8_qai8_qsi8cx_params *params)
{
    (void)k_idx_a;
    (void)k_idx_b;
    if (!params) return set_ok();  // the reference returns silently
    if (!ptrs_ok(m, n, A_packed, B_packed, D) || (m && n && !params->scale_b)) return set_invalid();
    GemmCommon g = common(m, n, k, A_packed, lda, B_packed, ldb, C, ldc, D, ldd, bias);
    RequantParams p{params->scale_a, params->scale_b, params->quant_channel_b, params->scale_d, params->zero_point_d};
    set_result(launch_gemm_requant_i8(g, p, clamp_min, clamp_max, env_path()));
}

// ---- W4A8 ------------------------------------------------------------------------------------------
#define TQT_DEFINE_W4A8_PACKED(TDNAME, TDTYPE, TDENUM, TDSIZE)                                                         \
    size_t tqt_get_m_step_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(void) { return M_STEP; }       \
    size_t tqt_get_n_step_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(void) { return N_STEP; }       \
    size_t tqt_get_a_packed_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                      \
        size_t m_idx, size_t k_idx, size_t lda, size_t actual_m)                                                       \
    {                                                                                                                  \
        (void)actual_m;                                                                                                \
        return packed_offset(m_idx, k_idx, lda, kI8BlockK, kI8BlockBytes);                                             \
    }                                                                                                                  \
    size_t tqt_get_b_packed_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                      \
        size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n)                                                       \
    {                                                                                                                  \
        (void)actual_n;                                                                                                \
        return packed_offset(n_idx, k_idx, ldb, kI4BlockK, kI4CxBlockBytes);                                           \
    }                                                                                                                  \
    size_t tqt_get_c_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t m_idx, size_t n_idx,  \
                                                                                         size_t ldc)                   \
    {                                                                                                                  \
        return (m_idx * ldc + n_idx) * (TDSIZE);                                                                       \
    }                                                                                                                  \
    size_t tqt_get_bias_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t n_idx)             \
    {                                                                                                                  \
        return n_idx * (TDSIZE);                                                                                       \
    }                                                                                                                  \
    size_t tqt_get_d_offset_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t m_idx, size_t n_idx,  \
                                                                                         size_t ldd)                   \
    {                                                                                                                  \
        return (m_idx * ldd + n_idx) * (TDSIZE);                                                                       \
    }                                                                                                                  \
    size_t tqt_get_d_size_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t m, size_t n)            \
    {                                                                                                                  \
        return m * n * (TDSIZE);                                                                                       \
    }                                                                                                                  \
    size_t tqt_get_a_packed_size_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t m, size_t k)     \
    {                                                                                                                  \
        return packed_size(m, k, kI8BlockK, kI8BlockBytes);                                                            \
    }                                                                                                                  \
    size_t tqt_get_b_packed_size_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(size_t n, size_t k)     \
    {                                                                                                                  \
        return packed_size(n, k, kI4BlockK, kI4CxBlockBytes);                                                          \
    }                                                                                                                  \
    void tqt_run_a_pack_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                                 \
        size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A, void *A_packed)                \
    {                                                                                                                  \
        run_pack_a_i8(m, k, lda, lda_packed, k_idx, A, A_packed);                                                      \
    }                                                                                                                  \
    void tqt_run_bt_pack_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                                \
        size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed)                \
    {                                                                                                                  \
        run_pack_bt_i4(n, k, ldb, ldb_packed, k_idx, B, B_packed, false);                                              \
    }                                                                                                                  \
    void tqt_run_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                                        \
        size_t m, size_t n, size_t k, const void *A_packed, size_t lda, size_t k_idx_a, const void *B_packed,          \
        size_t ldb, size_t k_idx_b, const void *C, size_t ldc, void *D, size_t ldd, const void *bias,                  \
        TDTYPE clamp_min, TDTYPE clamp_max, const struct tqt_qai8dx_qsi4cx_params *params)                             \
    {                                                                                                                  \
        (void)k_idx_a; (void)k_idx_b;                                                                                  \
        run_w4a8(m, n, k, A_packed, lda, B_packed, ldb, C, ldc, D, ldd, bias, (float)clamp_min, (float)clamp_max,      \
                 params, TDENUM);                                                                                      \
    }

TQT_DEFINE_W4A8_PACKED(f32, float, Dtype::F32, sizeof(float))
TQT_DEFINE_W4A8_PACKED(f16, float16_t, Dtype::F16, 2)
TQT_DEFINE_W4A8_PACKED(bf16, bfloat16_t, Dtype::BF16, 2)

// ---- W4A16 -----------------------------------------------------------------------------------------
#define TQT_DEFINE_W4A16_PACKED(TDNAME, TDTYPE, TDENUM, TDSIZE)                                                        \
    size_t tqt_get_m_step_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(void) { return M_STEP; }          \
    size_t tqt_get_n_step_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(void) { return N_STEP; }          \
    size_t tqt_get_a_packed_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                         \
        size_t m_idx, size_t k_idx, size_t lda, size_t actual_m)                                                       \
    {                                                                                                                  \
        (void)actual_m;                                                                                                \
        return packed_offset(m_idx, k_idx, lda, kF16BlockK, kF16BlockBytes);                                           \
    }                                                                                                                  \
    size_t tqt_get_b_packed_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                         \
        size_t n_idx, size_t k_idx, size_t ldb, size_t actual_n)                                                       \
    {                                                                                                                  \
        (void)actual_n;                                                                                                \
        return packed_offset(n_idx, k_idx, ldb, kI4BlockK, kI4C2BlockBytes);                                           \
    }                                                                                                                  \
    size_t tqt_get_scale_b_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t n_idx,             \
                                                                                            size_t b_idx,             \
                                                                                            size_t ldsb)              \
    {                                                                                                                  \
        return (n_idx * ldsb + b_idx) * 2;                                                                             \
    }                                                                                                                  \
    size_t tqt_get_c_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t m_idx, size_t n_idx,     \
                                                                                      size_t ldc)                      \
    {                                                                                                                  \
        return (m_idx * ldc + n_idx) * (TDSIZE);                                                                       \
    }                                                                                                                  \
    size_t tqt_get_bias_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t n_idx)                \
    {                                                                                                                  \
        return n_idx * (TDSIZE);                                                                                       \
    }                                                                                                                  \
    size_t tqt_get_d_offset_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t m_idx, size_t n_idx,     \
                                                                                      size_t ldd)                      \
    {                                                                                                                  \
        return (m_idx * ldd + n_idx) * (TDSIZE);                                                                       \
    }                                                                                                                  \
    size_t tqt_get_d_size_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t m, size_t n)               \
    {                                                                                                                  \
        return m * n * (TDSIZE);                                                                                       \
    }                                                                                                                  \
    size_t tqt_get_a_packed_size_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t m, size_t k)        \
    {                                                                                                                  \
        return packed_size(m, k, kF16BlockK, kF16BlockBytes);                                                          \
    }                                                                                                                  \
    size_t tqt_get_b_packed_size_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(size_t n, size_t k)        \
    {                                                                                                                  \
        return packed_size(n, k, kI4BlockK, kI4C2BlockBytes);                                                          \
    }                                                                                                                  \
    void tqt_run_a_pack_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                                    \
        size_t m, size_t k, size_t lda, size_t lda_packed, size_t k_idx, const void *A, void *A_packed)                \
    {                                                                                                                  \
        if ((m && k && (!A || !A_packed)) || k_idx % kF16BlockK) return set_invalid();                                 \
        set_result(launch_pack_rows(t_stream, m, k, lda, lda_packed, A, A_packed, 2, false));                          \
    }                                                                                                                  \
    void tqt_run_bt_pack_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                                   \
        size_t n, size_t k, size_t ldb, size_t ldb_packed, size_t k_idx, const void *B, void *B_packed)                \
    {                                                                                                                  \
        run_pack_bt_i4(n, k, ldb, ldb_packed, k_idx, B, B_packed, true);                                               \
    }                                                                                                                  \
    void tqt_run_gemm_1xnbias_clamp_##TDNAME##_f16p_qsi4c2p_128x128_sm100a(                                           \
        size_t m, size_t n, size_t k, size_t bl, const void *A_packed, size_t lda, size_t k_idx_a,                    \
        const void *B_packed, size_t ldb, size_t k_idx_b, const void *scale_b, size_t ldsb, const void *C,            \
        size_t ldc, void *D, size_t ldd, const void *bias, TDTYPE clamp_min, TDTYPE clamp_max)                        \
    {                                                                                                                  \
        (void)k_idx_a; (void)k_idx_b;                                                                                  \
        run_w4a16(m, n, k, bl, A_packed, lda, B_packed, ldb, scale_b, ldsb, C, ldc, D, ldd, bias, (float)clamp_min,    \
                  (float)clamp_max, TDENUM);                                                                           \
    }

TQT_DEFINE_W4A16_PACKED(f16, float16_t, Dtype::F16, 2)
TQT_DEFINE_W4A16_PACKED(f32, float, Dtype::F32, 4)

// ---- extensions --------------------------------------------------------------------------------------
void tqt_run_quant_pack_qai8dxp_f32_128x128_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_packed,
                                                   float *scale_a, int32_t *zero_point_a)
{
    run_quant(m, k, A, lda, A_packed, 0, true, scale_a, zero_point_a, Dtype::F32);
}
void tqt_run_quant_pack_qai8dxp_f16_128x128_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_packed,
                                                   float *scale_a, int32_t *zero_point_a)
{
    run_quant(m, k, A, lda, A_packed, 0, true, scale_a, zero_point_a, Dtype::F16);
}
void tqt_run_quant_pack_qai8dxp_bf16_128x128_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_packed,
                                                    float *scale_a, int32_t *zero_point_a)
{
    run_quant(m, k, A, lda, A_packed, 0, true, scale_a, zero_point_a, Dtype::BF16);
}
#define TQT_DEFINE_QUANT_GEMM(TDNAME, TDTYPE, TDENUM)                                                                  \
    void tqt_run_quant_gemm_1xnbias_clamp_##TDNAME##_qai8dxp_qsi4cxp_128x128_sm100a(                                   \
        size_t m, size_t n, size_t k, const void *A, size_t lda, int a_type, void *A_packed, float *scale_a,           \
        int32_t *zero_point_a, const void *B_packed, size_t ldb, const void *C, size_t ldc, void *D, size_t ldd,       \
        const void *bias, TDTYPE clamp_min, TDTYPE clamp_max, const float *scale_b)                                    \
    {                                                                                                                  \
        run_quant_w4a8(m, n, k, A, lda, a_type, A_packed, scale_a, zero_point_a, B_packed, ldb, C, ldc, D, ldd, bias,  \
                       (float)clamp_min, (float)clamp_max, scale_b, TDENUM);                                           \
    }
TQT_DEFINE_QUANT_GEMM(f32, float, Dtype::F32)
TQT_DEFINE_QUANT_GEMM(f16, float16_t, Dtype::F16)
TQT_DEFINE_QUANT_GEMM(bf16, bfloat16_t, Dtype::BF16)

// The variant that allocates nothing and takes no workspace: static_scratch.cu.
void tqt_run_quant_gemm_static_1xnbias_clamp_f32_qai8dxp_qsi4cxp_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A, size_t lda, int a_type, const void *B_packed, size_t ldb, const void *C,
    size_t ldc, void *D, size_t ldd, const void *bias, float clamp_min, float clamp_max, const float *scale_b)
{
    if (a_type < 0 || a_type > 2 || (k & 1)) return set_invalid();
    if (m && n && (!A || !B_packed || !D || !scale_b)) return set_invalid();
    if (m == 0 || n == 0) return set_ok();
    if (ldb < k) ldb = k;
    if (!replicas_cover(m, n, D, ldd, 4)) return set_invalid();
    GemmCommon g = common(m, n, k, nullptr, k, B_packed, ldb, C, ldc, D, ldd, bias);
    set_result(quant_gemm_w4a8_static(g, A, lda, (Dtype)a_type, scale_b, Dtype::F32, clamp_min, clamp_max));
}

void tqt_run_quant_qai8dx_f32_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_q, size_t ldq,
                                     float *scale_a, int32_t *zero_point_a)
{
    run_quant(m, k, A, lda, A_q, ldq, false, scale_a, zero_point_a, Dtype::F32);
}
void tqt_run_quant_qai8dx_f16_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_q, size_t ldq,
                                     float *scale_a, int32_t *zero_point_a)
{
    run_quant(m, k, A, lda, A_q, ldq, false, scale_a, zero_point_a, Dtype::F16);
}
void tqt_run_quant_qai8dx_bf16_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_q, size_t ldq,
                                      float *scale_a, int32_t *zero_point_a)
{
    run_quant(m, k, A, lda, A_q, ldq, false, scale_a, zero_point_a, Dtype::BF16);
}

void tqt_run_a_unpack_i8_128x128_sm100a(size_t m, size_t k, const void *A_packed, size_t lda_packed, void *A,
                                        size_t lda)
{
    set_result(launch_unpack_rows(t_stream, m, k, lda_packed, A_packed, A, lda, 1));
}
void tqt_run_a_unpack_f16_128x128_sm100a(size_t m, size_t k, const void *A_packed, size_t lda_packed, void *A,
                                         size_t lda)
{
    set_result(launch_unpack_rows(t_stream, m, k, lda_packed, A_packed, A, lda, 2));
}
void tqt_run_bt_unpack_qsi4cxp_128x128_sm100a(size_t n, size_t k, const void *B_packed, size_t ldb_packed, void *B,
                                              size_t ldb)
{
    set_result(launch_unpack_i4(t_stream, n, k, ldb_packed, B_packed, B, ldb / 2, false));
}
void tqt_run_bt_unpack_qsi4c2p_128x128_sm100a(size_t n, size_t k, const void *B_packed, size_t ldb_packed, void *B,
                                              size_t ldb)
{
    set_result(launch_unpack_i4(t_stream, n, k, ldb_packed, B_packed, B, ldb / 2, true));
}

void tqt_shard_plan_n(size_t n, size_t world, size_t rank, size_t *n_begin, size_t *n_count)
{
    if (world == 0) world = 1;
    const size_t blocks = ceil_div(n, N_STEP);
    const size_t base = blocks / world, extra = blocks % world;
    const size_t b0 = rank * base + (rank < extra ? rank : extra);
    const size_t nb = base + (rank < extra ? 1 : 0);
    size_t begin = b0 * N_STEP, end = (b0 + nb) * N_STEP;
    if (begin > n) begin = n;
    if (end > n) end = n;
    if (n_begin) *n_begin = begin;
    if (n_count) *n_count = end - begin;
}

uint16_t tqt_cuda_debug_f16_bits(float16_t v)
{
    uint16_t u;
    __builtin_memcpy(&u, &v, 2);
    return u;
}
uint16_t tqt_cuda_debug_bf16_bits(bfloat16_t v)
{
    uint16_t u;
    __builtin_memcpy(&u, &v, 2);
    return u;
}

void tqt_cuda_debug_set_timing_buffer(void *dev_ptr) { set_timing_buffer(dev_ptr); }

void tqt_cuda_debug_set_path(const char *path, const char *umma) { set_path_switches(path, umma); }

void tqt_cuda_debug_inject_wait_failure(unsigned wait_shift, unsigned flags) { set_failure_injection(wait_shift, flags); }

void tqt_cuda_debug_stream_read(const void *src, size_t bytes, void *sink) { set_result(stream_read(src, bytes, sink, t_stream)); }

void tqt_cuda_set_output_replicas(const void *local_base, size_t local_bytes, void *const *replica_bases, size_t count)
{
    if (count > 7 || (count && (!local_base || !replica_bases || local_bytes == 0))) return set_invalid();
    for (size_t i = 0; i < count; ++i)
        if (!replica_bases[i]) return set_invalid();
    t_n_replicas = count;
    t_replica_local = static_cast<const char *>(local_base);
    t_replica_bytes = count ? local_bytes : 0;
    for (size_t i = 0; i < count; ++i)
        t_replica_delta[i] = (long long)(static_cast<const char *>(replica_bases[i]) - t_replica_local);
    set_ok();
}

#include "abi_siblings.inc"
#include "abi_conv.inc"
#include "abi_float.inc"

int tqt_cuda_debug_last_kernel(void) { return last_kernel(); }

int tqt_cuda_kernel_choice_w4a8(size_t m, size_t n, size_t k)
{
    (void)n;
    if (k == 0) return 2;
    return m <= 16 ? 1 : 0;
}

}  // extern "C"
