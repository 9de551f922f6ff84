// Unquantised GEMM families (f32 / f16 / bf16 operands): D = clamp(A * B + C + bias), narrowed once to the output type.
// Reference semantics: test/common/reference_gemm.cpp:11-61 (f32 accumulation, C then bias, clamp in f32); kernel types
// under src/gemm/gemm_{f32_f32,f16_f16,bf16_bf16}/.
//
// This file holds the generic CUDA-core kernel: any operand layout (row-major [rows, k], [k, rows], or the packed
// 128-row blocks of 128 bytes per row with the 128-byte swizzle), any alignment.  One output per thread; the K loop
// multiplies and adds in k order with separately rounded operations, which is the reference's arithmetic bit for bit.
// The f16 / bf16 kernel types run on tensor cores instead where their operands allow it (kernels_pair.cu).
#include "dev_common.cuh"

namespace tqt {

namespace {

template <Dtype TA>
struct FloatOperand {
    const uint8_t *p;
    size_t ld;        // row stride in elements (row-major / k-major), or blocks per row tile (packed)
    int layout;       // Layout
    __device__ __forceinline__ float get(size_t r, size_t k) const
    {
        constexpr size_t ES = TA == Dtype::F32 ? 4 : 2;
        constexpr size_t KPB = 128 / ES;   // k elements per packed block row
        size_t idx;
        if (layout == (int)Layout::RowMajor) {
            idx = r * ld + k;
        } else if (layout == (int)Layout::KMajor) {
            idx = k * ld + r;
        } else {
            const size_t byte = ((r >> 7) * ld + k / KPB) * kI8BlockBytes + sw128_byte((uint32_t)(r & 127), (uint32_t)(k % KPB) * (uint32_t)ES);
            idx = byte / ES;
        }
        return TdTraits<TA>::load(p, idx);
    }
};

template <Dtype TA, Dtype TD>
__global__ void __launch_bounds__(256) gemm_simt_float_kernel(size_t m, size_t n, size_t k, FloatOperand<TA> a, FloatOperand<TA> b, const void *C,
                                                              size_t ldc, void *D, size_t ldd, const void *bias, int bias_per_row,
                                                              float cmin, float cmax)
{
    const size_t total = m * n;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t i = idx / n, j = idx - i * n;
        float acc = 0.0f;
        for (size_t p = 0; p < k; ++p) acc = __fadd_rn(acc, __fmul_rn(a.get(i, p), b.get(j, p)));
        if (C) acc = __fadd_rn(acc, TdTraits<TD>::load(C, i * ldc + j));
        if (bias) acc = __fadd_rn(acc, TdTraits<TD>::load(bias, bias_per_row ? i : j));
        acc = fmaxf(acc, cmin);
        acc = fminf(acc, cmax);
        TdTraits<TD>::store(D, i * ldd + j, acc);
    }
}

template <Dtype TA, Dtype TD>
Result run_float_simt(const GemmCommon &g, Layout la, Layout lb, bool bias_per_row, float cmin, float cmax)
{
    constexpr size_t ES = TA == Dtype::F32 ? 4 : 2, KPB = 128 / ES;
    FloatOperand<TA> a{(const uint8_t *)g.A, la == Layout::Packed ? ceil_div(g.lda, KPB) : g.lda, (int)la};
    FloatOperand<TA> b{(const uint8_t *)g.B, lb == Layout::Packed ? ceil_div(g.ldb, KPB) : g.ldb, (int)lb};
    const size_t total = g.m * g.n;
    const size_t blocks = (total + 255) / 256;
    const unsigned grid = (unsigned)(blocks > 148 * 32 ? 148 * 32 : blocks);
    gemm_simt_float_kernel<TA, TD><<<grid, 256, 0, (cudaStream_t)g.stream>>>(g.m, g.n, g.k, a, b, g.C, g.ldc, g.D, g.ldd, g.bias,
                                                                           bias_per_row ? 1 : 0, cmin, cmax);
    note_kernel(kKernelSimt);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

}  // namespace

Result umma_gemm_float(const GemmCommon &g, Dtype ta, Dtype td, float cmin, float cmax, Layout la, Layout lb, bool bias_per_row);

Result launch_gemm_float(const GemmCommon &g, Dtype ta, Dtype td, float cmin, float cmax, Layout la, Layout lb, bool bias_per_row)
{
    if (g.m == 0 || g.n == 0) return Result{kOk, 0};
    if (g.n_replicas || la == Layout::KMajor) return Result{kUnsupported, 0};
    // 16-bit operands: tensor cores where the layouts and alignments allow (TQT_B200_PATH=simt keeps this kernel)
    if (ta != Dtype::F32 && g.k && env_path() != Path::Simt) {
        Result r = umma_gemm_float(g, ta, td, cmin, cmax, la, lb, bias_per_row);
        if (r.status != kUnsupported) return r;
    }
#define TQT_FLOAT_CASE(TA_, TD_) \
    if (ta == TA_ && td == TD_) return run_float_simt<TA_, TD_>(g, la, lb, bias_per_row, cmin, cmax)
    TQT_FLOAT_CASE(Dtype::F32, Dtype::F32);
    TQT_FLOAT_CASE(Dtype::F16, Dtype::F16);
    TQT_FLOAT_CASE(Dtype::BF16, Dtype::BF16);
    TQT_FLOAT_CASE(Dtype::BF16, Dtype::F32);
    TQT_FLOAT_CASE(Dtype::BF16, Dtype::F16);
#undef TQT_FLOAT_CASE
    return Result{kUnsupported, 0};
}

}  // namespace tqt
