// Kernel choice for each run_gemm call.  Host-only logic (no CUDA headers).
//
//   packed kernel types : tcgen05 tensor-core GEMM (kernels_umma.cu); W4A8 with m <= 16 goes to the
//                         HBM-streaming GEMV (kernels_gemv.cu)
//   unpacked kernel types and k == 0 : generic CUDA-core kernel (kernels_simt.cu)
// TQT_B200_PATH=simt|umma|gemv forces a path and TQT_B200_UMMA=single|pair|ts a tensor-core kernel (used by
// the tests to cross-check the kernels against each other); a forced path that cannot take the call reports
// TQT_CUDA_UNSUPPORTED.  The environment is read once, at the first call; tqt_cuda_debug_set_path changes the
// two switches at run time (process-wide atomics, so concurrent run_gemm calls see one value or the other).
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "tqt_internal.h"

namespace tqt {

Result simt_gemm_i32(const GemmCommon &g, bool packed, int32_t cmin, int32_t cmax);
Result simt_gemm_requant_i8(const GemmCommon &g, const RequantParams &p, int cmin, int cmax);
Result simt_gemm_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax);
Result simt_gemm_w4a16(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td, float cmin,
                       float cmax);
Result umma_gemm_i32(const GemmCommon &g, int32_t cmin, int32_t cmax);
Result umma_gemm_i32_layouts(const GemmCommon &g, int32_t cmin, int32_t cmax, Layout la, Layout lb);
Result umma_gemm_requant_i8(const GemmCommon &g, const RequantParams &p, int cmin, int cmax);
Result umma_gemm_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax);
Result umma_gemm_w4a16(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td, float cmin,
                       float cmax);
Result gemv_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax);

static std::atomic<int> g_path{0}, g_umma{0};
static std::once_flag g_switch_once;

static int parse_path(const char *e)
{
    if (!e) return (int)Path::Auto;
    if (!std::strcmp(e, "simt")) return (int)Path::Simt;
    if (!std::strcmp(e, "umma")) return (int)Path::Umma;
    if (!std::strcmp(e, "gemv")) return (int)Path::Gemv;
    return (int)Path::Auto;
}

static int parse_umma(const char *e)
{
    if (!e) return 0;
    if (!std::strcmp(e, "single")) return 1;
    if (!std::strcmp(e, "pair")) return 2;
    if (!std::strcmp(e, "ts")) return 3;
    return 0;
}

static void init_switches()
{
    std::call_once(g_switch_once, [] {
        g_path.store(parse_path(std::getenv("TQT_B200_PATH")));
        g_umma.store(parse_umma(std::getenv("TQT_B200_UMMA")));
    });
}

Path env_path()
{
    init_switches();
    return (Path)g_path.load(std::memory_order_relaxed);
}

int umma_variant()
{
    init_switches();
    return g_umma.load(std::memory_order_relaxed);
}

void set_path_switches(const char *path, const char *umma)
{
    init_switches();   // a later first call must not overwrite what is set here
    g_path.store(parse_path(path));
    g_umma.store(parse_umma(umma));
}

static std::atomic<int> g_last_kernel{0};
void note_kernel(int family) { g_last_kernel.store(family, std::memory_order_relaxed); }
int last_kernel() { return g_last_kernel.load(std::memory_order_relaxed); }

static inline bool empty_problem(const GemmCommon &g) { return g.m == 0 || g.n == 0; }

Result launch_gemm_i32(const GemmCommon &g, bool packed, int32_t cmin, int32_t cmax, Path path)
{
    if (empty_problem(g)) return Result{kOk, 0};
    if (path == Path::Gemv) return Result{kUnsupported, 0};
    if (!packed && g.k != 0 && path != Path::Simt) {
        // unpacked operands (A [m, lda], B [k, ldb]): tensor cores through tiled TMA loads when base addresses and row
        // strides are multiples of 16 bytes, else the generic kernel
        Result r = umma_gemm_i32_layouts(g, cmin, cmax, Layout::RowMajor, Layout::KMajor);
        if (r.status != kUnsupported || path == Path::Umma) return r;
    }
    if (!packed || g.k == 0 || path == Path::Simt) {
        if (path == Path::Umma || g.n_replicas) return Result{kUnsupported, 0};
        return simt_gemm_i32(g, packed, cmin, cmax);
    }
    return umma_gemm_i32(g, cmin, cmax);
}

Result launch_gemm_requant_i8(const GemmCommon &g, const RequantParams &p, int cmin, int cmax, Path path)
{
    if (empty_problem(g)) return Result{kOk, 0};
    if (path == Path::Gemv) return Result{kUnsupported, 0};
    if (g.k == 0 || path == Path::Simt) {
        if (path == Path::Umma || g.n_replicas) return Result{kUnsupported, 0};
        return simt_gemm_requant_i8(g, p, cmin, cmax);
    }
    return umma_gemm_requant_i8(g, p, cmin, cmax);
}

Result launch_gemm_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax, Path path)
{
    if (empty_problem(g)) return Result{kOk, 0};
    if (g.k == 0 || path == Path::Simt) {
        if (path == Path::Umma || path == Path::Gemv || g.n_replicas) return Result{kUnsupported, 0};
        return simt_gemm_w4a8(g, p, td, cmin, cmax);
    }
    if (path == Path::Gemv) return g.n_replicas ? Result{kUnsupported, 0} : gemv_w4a8(g, p, td, cmin, cmax);
    if (path == Path::Auto && g.m <= 16 && !g.n_replicas) {
        Result r = gemv_w4a8(g, p, td, cmin, cmax);
        if (r.status != kUnsupported) return r;  // shapes the GEMV cannot hold fall through to the GEMM
    }
    return umma_gemm_w4a8(g, p, td, cmin, cmax);
}

Result launch_gemm_w4a16(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td, float cmin,
                         float cmax, Path path)
{
    if (empty_problem(g)) return Result{kOk, 0};
    if (path == Path::Gemv) return Result{kUnsupported, 0};
    if (g.k == 0 || path == Path::Simt) {
        if (path == Path::Umma || g.n_replicas) return Result{kUnsupported, 0};
        return simt_gemm_w4a16(g, bl, scale_b, ldsb, td, cmin, cmax);
    }
    return umma_gemm_w4a16(g, bl, scale_b, ldsb, td, cmin, cmax);
}

}  // namespace tqt
