// Quantise + W4A8 GEMM for callers that cannot allocate device memory: the intermediates of the call (the packed int8
// activations, the per-row scales and zero points) live in a file-scope device array of this library instead of in
// buffers the caller provides.  No counterpart in the reference, whose callers own every buffer.
//
// Who needs this: a plug-in that runs inside a serving process whose memory pool has already claimed the whole GPU (a
// further cudaMalloc fails there), or inside a latency-critical loop where cudaMalloc's device-wide synchronisation is
// not acceptable, and that has no way to ask its host for a workspace.
#include "dev_common.cuh"
#include "tqt_internal.h"

namespace tqt {

namespace {

// Limits of the static variant: the packed activations of one call may take up to 8 MiB (for instance 2048 rows of
// k = 4096, or 8192 rows of k = 1024) and the call may have up to 8192 rows.  Every GPU that loads the library holds
// these 8 MiB + 64 KiB until the process exits.
constexpr size_t kStaticPackedBytes = size_t(8) << 20;
constexpr size_t kStaticMaxRows = 8192;
constexpr size_t kStaticScaleOff = kStaticPackedBytes;                         // float [kStaticMaxRows]
constexpr size_t kStaticZpOff = kStaticScaleOff + kStaticMaxRows * 4;          // int32 [kStaticMaxRows]
constexpr size_t kStaticBytes = kStaticZpOff + kStaticMaxRows * 4;

static __device__ __align__(256) uint8_t g_static_quant[kStaticBytes];

// The array's name is only a handle in host code: its device address is looked up once per device, with that device
// current, and cached.
Result static_quant_base(uint8_t **base)
{
    static uint8_t *cache[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    if (dev < 0 || dev >= 64) return Result{kUnsupported, 0};
    uint8_t *p = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        void *addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_static_quant);
        if (e != cudaSuccess || !addr) return Result{kLaunchFailed, (int)e};
        p = static_cast<uint8_t *>(addr);
        __atomic_store_n(&cache[dev], p, __ATOMIC_RELEASE);
    }
    *base = p;
    return Result{kOk, 0};
}

}  // namespace

// g: the GEMM's arguments with A / lda still unset.  kUnsupported (nothing launched) when the call does not fit the array.
Result quant_gemm_w4a8_static(GemmCommon g, const void *A, size_t lda, Dtype ta, const float *scale_b, Dtype td,
                              float clamp_min, float clamp_max)
{
    const size_t packed = ceil_div(g.m, 128) * ceil_div(g.k, 128) * kI8BlockBytes;
    if (g.m > kStaticMaxRows || packed > kStaticPackedBytes) return Result{kUnsupported, 0};
    uint8_t *base = nullptr;
    Result r = static_quant_base(&base);
    if (r.status != kOk) return r;
    float *scale_a = reinterpret_cast<float *>(base + kStaticScaleOff);
    int32_t *zp_a = reinterpret_cast<int32_t *>(base + kStaticZpOff);
    // Nothing in the array has to start at zero: the quantiser writes every byte of the rows [0, m) of the blocks the
    // GEMM reads (padding columns up to the block width included) and every scale / zero point of those rows; rows
    // beyond m inside the last 128-row block keep an earlier call's bytes, which only reach accumulator rows that
    // are never stored.
    r = launch_quant_qai8dx(g.stream, g.m, g.k, A, lda, ta, base, 0, true, scale_a, zp_a);
    if (r.status != kOk) return r;
    g.A = base;
    g.lda = g.k;
    W4A8Params p{scale_a, zp_a, scale_b};
    return launch_gemm_w4a8(g, p, td, clamp_min, clamp_max, env_path());
}

}  // namespace tqt
