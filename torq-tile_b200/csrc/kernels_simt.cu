// Generic CUDA-core GEMM kernels.  They serve the unpacked kernel types (operands in the caller's
// row-major layouts, any alignment) and, through TQT_B200_PATH=simt, re-compute any packed call
// without tensor cores so that layout and epilogue code can be checked in isolation.  Operands
// are fetched through small accessor structs, staged in shared memory as packed int8 words and
// multiplied with dp4a.
#include "conv_geom.cuh"
#include "epilogues.cuh"

namespace tqt {

// ---- operand accessors (element (row, k) -> int8) ---------------------------------------------------
struct RowMajorI8 {  // [rows, k], ld in elements
    const int8_t *p;
    size_t ld;
    __device__ int8_t get(size_t r, size_t k) const { return p[r * ld + k]; }
};
struct ColMajorI8 {  // stored [k, rows]: element (row, k) at p[k * ld + row]
    const int8_t *p;
    size_t ld;
    __device__ int8_t get(size_t r, size_t k) const { return p[k * ld + r]; }
};
struct PackedI8 {  // swizzled 128 x 128 blocks, block_bytes apart (16 KiB, or 16 KiB + row sums)
    const int8_t *p;
    size_t kblocks_total;
    size_t block_bytes = kI8BlockBytes;
    __device__ int8_t get(size_t r, size_t k) const
    {
        return p[((r >> 7) * kblocks_total + (k >> 7)) * block_bytes + sw128_byte((uint32_t)(r & 127), (uint32_t)(k & 127))];
    }
};
struct PackedI4Cx {  // qsi4cx blocks, returns the signed value q
    const uint8_t *p;
    size_t kblocks_total;
    __device__ int8_t get(size_t r, size_t k) const
    {
        uint32_t hi;
        const uint32_t b = i4cx_byte((uint32_t)(r & 127), (uint32_t)(k & 127), &hi);
        const uint32_t v = (p[((r >> 7) * kblocks_total + (k >> 7)) * kI4CxBlockBytes + b] >> (hi * 4)) & 0xFu;
        return (int8_t)((int)(v ^ 8u) - 8);
    }
};

struct RowMajorNib {  // [rows, k / 2] bytes, row stride in bytes; byte = (q_hi + 8) << 4 | (q_lo + 8), low nibble = even k
    const uint8_t *p;
    size_t ld_bytes;
    __device__ int8_t get(size_t r, size_t k) const
    {
        const uint32_t v = (p[r * ld_bytes + (k >> 1)] >> ((k & 1) * 4)) & 0xFu;
        return (int8_t)((int)v - 8);
    }
};

// The im2col view of a convolution input as an operand: element (row = output position - pos0, k) is gathered from the
// activation tensor on the fly (implicit GEMM: no im2col matrix exists anywhere).
template <bool CF>
struct Im2colI8 {
    const int8_t *p;
    ConvGeom g;
    uint32_t pos0;   // output position of row 0 of this call
    __device__ int8_t get(size_t r, size_t k) const
    {
        uint32_t od, oh, ow;
        split_position(g, pos0 + (uint32_t)r, od, oh, ow);
        KCursor<CF> cur;
        cur.seek(g, (uint32_t)k);
        size_t off;
        return cur.source(g, od, oh, ow, off) ? p[off] : (int8_t)0;
    }
};

template <class LA, class LB, class Epi, bool RSUM>
__global__ void __launch_bounds__(256) gemm_simt_i8_kernel(size_t m, size_t n, size_t k, LA la, LB lb, Epi epi)
{
    __shared__ uint32_t As[64][9];  // 64 rows x 32 k (8 words) + 1 pad
    __shared__ uint32_t Bs[64][9];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const size_t m0 = (size_t)blockIdx.y * 64, n0 = (size_t)blockIdx.x * 64;
    int32_t acc[4][4];
    int32_t rs[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0;

    const int lrow = threadIdx.x >> 2, lseg = threadIdx.x & 3;  // this thread stages 8 k of one row
    for (size_t k0 = 0; k0 < k; k0 += 32) {
        uint32_t wa[2] = {0, 0}, wb[2] = {0, 0};
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const size_t kk = k0 + lseg * 8 + e;
            int8_t a = 0, b = 0;
            if (kk < k) {
                if (m0 + lrow < m) a = la.get(m0 + lrow, kk);
                if (n0 + lrow < n) b = lb.get(n0 + lrow, kk);
            }
            wa[e >> 2] |= (uint32_t)(uint8_t)a << ((e & 3) * 8);
            wb[e >> 2] |= (uint32_t)(uint8_t)b << ((e & 3) * 8);
        }
        As[lrow][lseg * 2] = wa[0];
        As[lrow][lseg * 2 + 1] = wa[1];
        Bs[lrow][lseg * 2] = wb[0];
        Bs[lrow][lseg * 2 + 1] = wb[1];
        __syncthreads();
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            uint32_t av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                av[i] = As[ty * 4 + i][w];
                bv[i] = Bs[tx * 4 + i][w];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a((int)av[i], (int)bv[j], acc[i][j]);
            if (RSUM) {
#pragma unroll
                for (int j = 0; j < 4; ++j) rs[j] = __dp4a((int)bv[j], 0x01010101, rs[j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const size_t mm = m0 + ty * 4 + i;
        if (mm >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const size_t nn = n0 + tx * 4 + j;
            if (nn < n) epi(mm, nn, acc[i][j], rs[j]);
        }
    }
}

static inline Result check_launch()
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

template <class LA, class LB, class Epi, bool RSUM>
static Result run_simt(const GemmCommon &g, LA la, LB lb, Epi epi)
{
    if (g.m == 0 || g.n == 0) return Result{kOk, 0};
    if (g.n_replicas) return Result{kUnsupported, 0};   // output replicas are a feature of the tensor-core kernels
    const size_t gx = ceil_div(g.n, 64), gy = ceil_div(g.m, 64);
    if (gy > 65535 || gx > 0x7fffffffull) return Result{kUnsupported, 0};
    dim3 grid((unsigned)gx, (unsigned)gy);
    gemm_simt_i8_kernel<LA, LB, Epi, RSUM><<<grid, 256, 0, (cudaStream_t)g.stream>>>(g.m, g.n, g.k, la, lb, epi);
    note_kernel(kKernelSimt);
    return check_launch();
}

Result simt_gemm_i32(const GemmCommon &g, bool packed, int32_t cmin, int32_t cmax)
{
    EpiI32 epi{(const int32_t *)g.C, g.ldc, (int32_t *)g.D, g.ldd, cmin, cmax};
    if (packed) {
        PackedI8 la{(const int8_t *)g.A, ceil_div(g.lda, 128)};
        PackedI8 lb{(const int8_t *)g.B, ceil_div(g.ldb, 128)};
        return run_simt<PackedI8, PackedI8, EpiI32, false>(g, la, lb, epi);
    }
    RowMajorI8 la{(const int8_t *)g.A, g.lda};
    ColMajorI8 lb{(const int8_t *)g.B, g.ldb};
    return run_simt<RowMajorI8, ColMajorI8, EpiI32, false>(g, la, lb, epi);
}

Result simt_gemm_requant_i8(const GemmCommon &g, const RequantParams &p, int cmin, int cmax)
{
    EpiRequant epi{(const int32_t *)g.C, g.ldc, (const int32_t *)g.bias, (int8_t *)g.D, g.ldd, p.scale_a, p.scale_b,
                   p.quant_channel_b, p.scale_d, p.zero_point_d, cmin, cmax};
    PackedI8 la{(const int8_t *)g.A, ceil_div(g.lda, 128)};
    PackedI8 lb{(const int8_t *)g.B, ceil_div(g.ldb, 128)};
    return run_simt<PackedI8, PackedI8, EpiRequant, false>(g, la, lb, epi);
}

template <Dtype TD>
static Result simt_w4a8_t(const GemmCommon &g, const W4A8Params &p, float cmin, float cmax)
{
    EpiW4A8<TD> epi{g.C, g.ldc, g.bias, g.D, g.ldd, p.scale_a, p.zp_a, p.scale_b, cmin, cmax};
    PackedI8 la{(const int8_t *)g.A, ceil_div(g.lda, 128)};
    PackedI4Cx lb{(const uint8_t *)g.B, ceil_div(g.ldb, 128)};
    return run_simt<PackedI8, PackedI4Cx, EpiW4A8<TD>, true>(g, la, lb, epi);
}

Result simt_gemm_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax)
{
    switch (td) {
        case Dtype::F32: return simt_w4a8_t<Dtype::F32>(g, p, cmin, cmax);
        case Dtype::F16: return simt_w4a8_t<Dtype::F16>(g, p, cmin, cmax);
        default: return simt_w4a8_t<Dtype::BF16>(g, p, cmin, cmax);
    }
}

// ---- sibling kernel types: any operand layout -------------------------------------------------------------
// Calls f(accessor) with the int8 accessor that matches the layout.
template <class F>
static Result with_i8_layout(Layout l, const void *p, size_t ld, F f, size_t block_bytes = kI8BlockBytes)
{
    switch (l) {
        case Layout::Packed: return f(PackedI8{(const int8_t *)p, ceil_div(ld, 128), block_bytes});
        case Layout::RowMajor: return f(RowMajorI8{(const int8_t *)p, ld});
        default: return f(ColMajorI8{(const int8_t *)p, ld});
    }
}

template <class Epi, bool RSUM>
static Result run_simt_layouts(const GemmCommon &g, Layout la, Layout lb, Epi epi, size_t b_block_bytes = kI8BlockBytes)
{
    return with_i8_layout(la, g.A, g.lda, [&](auto a) {
        return with_i8_layout(lb, g.B, g.ldb,
                              [&](auto b) { return run_simt<decltype(a), decltype(b), Epi, RSUM>(g, a, b, epi); }, b_block_bytes);
    });
}

// Implicit-GEMM convolutions (the igemm kernel types): the activation operand is the im2col view of `input`, the other
// operand the weights in `wl` layout (Packed or RowMajor [rows, ld]).  Channel-last: A = im2col (rows = output positions
// pos0 .. pos0 + m), B = weights [n, k], 1xN-bias requantisation.  Channel-first: A = weights [m, k], B = im2col
// (columns = output positions pos0 .. pos0 + n), Mx1-bias requantisation.  g.D is the output cell of (row 0, column 0)
// of this call.  Generic CUDA-core kernel.
Result launch_igemm_cl_requant_i8(const GemmCommon &g, const ConvGeom &geom, uint32_t pos0, const void *input,
                                  const RequantParams &p, int cmin, int cmax, Layout wl)
{
    if (g.m == 0 || g.n == 0) return Result{kOk, 0};
    if (wl == Layout::KMajor) return Result{kUnsupported, 0};
    EpiRequant epi{nullptr, 0, (const int32_t *)g.bias, (int8_t *)g.D, g.ldd, p.scale_a, p.scale_b,
                   p.quant_channel_b, p.scale_d, p.zero_point_d, cmin, cmax};
    Im2colI8<false> la{(const int8_t *)input, geom, pos0};
    return with_i8_layout(wl, g.B, g.ldb, [&](auto b) { return run_simt<Im2colI8<false>, decltype(b), EpiRequant, false>(g, la, b, epi); });
}

Result launch_igemm_cf_requant_rows_i8(const GemmCommon &g, const ConvGeom &geom, uint32_t pos0, const void *input,
                                       const RowRequantParams &p, int cmin, int cmax, Layout wl)
{
    if (g.m == 0 || g.n == 0) return Result{kOk, 0};
    if (wl == Layout::KMajor) return Result{kUnsupported, 0};
    EpiRequantRow epi{nullptr, 0, (const int32_t *)g.bias, (int8_t *)g.D, g.ldd, p.scale_a,
                      p.quant_channel_a, p.scale_b, p.scale_d, p.zero_point_d, cmin, cmax};
    Im2colI8<true> lb{(const int8_t *)input, geom, pos0};
    return with_i8_layout(wl, g.A, g.lda, [&](auto a) { return run_simt<decltype(a), Im2colI8<true>, EpiRequantRow, false>(g, a, lb, epi); });
}

Result umma_gemm_requant_i8_layouts(const GemmCommon &g, const RequantParams &p, int cmin, int cmax, Layout la, Layout lb);
Result umma_gemm_requant_rows_i8_layouts(const GemmCommon &g, const RowRequantParams &p, int cmin, int cmax, Layout la,
                                         Layout lb);

Result launch_gemm_requant_i8_layouts(const GemmCommon &g, const RequantParams &p, int cmin, int cmax, Layout la,
                                      Layout lb)
{
    // a row-major operand whose base and row stride are multiples of 16 bytes: tensor cores through tiled TMA loads
    // (TQT_B200_PATH=simt keeps the generic kernel, for cross-checks; it also takes what a tensor map cannot describe)
    if (g.m && g.n && g.k && env_path() != Path::Simt) {
        Result r = umma_gemm_requant_i8_layouts(g, p, cmin, cmax, la, lb);
        if (r.status != kUnsupported) return r;
    }
    EpiRequant epi{(const int32_t *)g.C, g.ldc, (const int32_t *)g.bias, (int8_t *)g.D, g.ldd, p.scale_a, p.scale_b,
                   p.quant_channel_b, p.scale_d, p.zero_point_d, cmin, cmax};
    return run_simt_layouts<EpiRequant, false>(g, la, lb, epi);
}

Result umma_gemm_requant_rows_i8(const GemmCommon &g, const RowRequantParams &p, int cmin, int cmax);

Result launch_gemm_requant_rows_i8(const GemmCommon &g, const RowRequantParams &p, int cmin, int cmax, Layout la,
                                   Layout lb)
{
    // both operands packed: tensor cores (TQT_B200_PATH=simt keeps the generic kernel, for cross-checks)
    if (la == Layout::Packed && lb == Layout::Packed && g.m && g.n && g.k && env_path() != Path::Simt) {
        Result r = umma_gemm_requant_rows_i8(g, p, cmin, cmax);
        if (r.status != kUnsupported) return r;
    }
    if (g.m && g.n && g.k && env_path() != Path::Simt) {   // a row-major operand: tiled TMA loads, where a tensor map can describe it
        Result r = umma_gemm_requant_rows_i8_layouts(g, p, cmin, cmax, la, lb);
        if (r.status != kUnsupported) return r;
    }
    EpiRequantRow epi{(const int32_t *)g.C, g.ldc, (const int32_t *)g.bias, (int8_t *)g.D, g.ldd, p.scale_a,
                      p.quant_channel_a, p.scale_b, p.scale_d, p.zero_point_d, cmin, cmax};
    return run_simt_layouts<EpiRequantRow, false>(g, la, lb, epi);
}

Result umma_gemm_dxcx(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax);
Result umma_gemm_dxcx_layouts(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax, Layout la, Layout lb);

Result launch_gemm_dxcx(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax, Layout la,
                        Layout lb)
{
    if (td != Dtype::F32 && td != Dtype::F16) return Result{kUnsupported, 0};
    // both operands packed: tensor cores (TQT_B200_PATH=simt keeps the generic kernel, for cross-checks)
    if (la == Layout::Packed && lb == Layout::Packed && g.m && g.n && g.k && env_path() != Path::Simt) {
        Result r = umma_gemm_dxcx(g, p, td, cmin, cmax);
        if (r.status != kUnsupported) return r;
    }
    if (la == Layout::RowMajor && lb == Layout::RowMajor && g.m && g.n && g.k && env_path() != Path::Simt) {
        Result r = umma_gemm_dxcx_layouts(g, p, td, cmin, cmax, la, lb);   // tiled TMA loads, where tensor maps can describe the operands
        if (r.status != kUnsupported) return r;
    }
    const size_t bb = lb == Layout::Packed ? kI8SumBlockBytes : kI8BlockBytes;   // packed B of these types carries row sums
    if (td == Dtype::F32) {
        EpiDxCx<Dtype::F32> epi{g.bias, g.D, g.ldd, p.scale_a, p.zp_a, p.scale_b, cmin, cmax};
        return run_simt_layouts<EpiDxCx<Dtype::F32>, true>(g, la, lb, epi, bb);
    }
    EpiDxCx<Dtype::F16> epi{g.bias, g.D, g.ldd, p.scale_a, p.zp_a, p.scale_b, cmin, cmax};
    return run_simt_layouts<EpiDxCx<Dtype::F16>, true>(g, la, lb, epi, bb);
}

template <Dtype TD>
static Result simt_w4a8_unpacked_t(const GemmCommon &g, const W4A8Params &p, float cmin, float cmax)
{
    EpiW4A8<TD> epi{g.C, g.ldc, g.bias, g.D, g.ldd, p.scale_a, p.zp_a, p.scale_b, cmin, cmax};
    RowMajorI8 la{(const int8_t *)g.A, g.lda};
    RowMajorNib lb{(const uint8_t *)g.B, g.ldb / 2};
    return run_simt<RowMajorI8, RowMajorNib, EpiW4A8<TD>, true>(g, la, lb, epi);
}

Result umma_gemm_w4a8_unpacked(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax);
Result umma_gemm_w4a16_unpacked(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td, float cmin,
                                float cmax);

Result launch_gemm_w4a8_unpacked(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax)
{
    // operands whose base addresses and row strides are multiples of 16 bytes: tiled TMA loads into the tensor-core
    // kernel (TQT_B200_PATH=simt keeps the generic kernel, which also takes everything else)
    if (g.m && g.n && g.k && env_path() != Path::Simt) {
        Result r = umma_gemm_w4a8_unpacked(g, p, td, cmin, cmax);
        if (r.status != kUnsupported) return r;
    }
    switch (td) {
        case Dtype::F32: return simt_w4a8_unpacked_t<Dtype::F32>(g, p, cmin, cmax);
        case Dtype::F16: return simt_w4a8_unpacked_t<Dtype::F16>(g, p, cmin, cmax);
        default: return simt_w4a8_unpacked_t<Dtype::BF16>(g, p, cmin, cmax);
    }
}

// ---- W4A16 (float) ------------------------------------------------------------------------------------
// One output per thread, k-order f32 accumulation of a * f16((nib-8)*scale).  Test-size only.
// PACKED: A / B in the block layouts (a_ld / b_ld = blocks per row tile); else A f16 [m, a_ld elements],
// B nibbles [n, b_ld bytes] with byte = (q_hi + 8) << 4 | (q_lo + 8), low nibble = even k.
template <Dtype TD, bool PACKED>
__global__ void gemm_simt_w4a16_kernel(size_t m, size_t n, size_t k, size_t bl, const uint8_t *__restrict__ A,
                                       size_t a_kblocks, const uint8_t *__restrict__ B, size_t b_kblocks,
                                       const __half *__restrict__ scale_b, size_t ldsb, const void *C, size_t ldc,
                                       void *D, size_t ldd, const void *bias, float cmin, float cmax)
{
    const size_t nn = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    const size_t mm = blockIdx.y;
    if (nn >= n || mm >= m) return;
    float acc = 0.0f;
    for (size_t kk = 0; kk < k; ++kk) {
        float a;
        int q;
        if (PACKED) {
            const uint8_t *ab = A + ((mm >> 7) * a_kblocks + (kk >> 6)) * kF16BlockBytes + sw128_byte((uint32_t)(mm & 127), (uint32_t)(kk & 63) * 2);
            a = __half2float(*reinterpret_cast<const __half *>(ab));
            uint32_t hi;
            const uint32_t bb = i4c2_byte((uint32_t)(nn & 127), (uint32_t)(kk & 127), &hi);
            q = (int)((B[((nn >> 7) * b_kblocks + (kk >> 7)) * kI4C2BlockBytes + bb] >> (hi * 4)) & 0xFu) - 8;
        } else {
            a = __half2float(reinterpret_cast<const __half *>(A)[mm * a_kblocks + kk]);
            q = (int)((B[nn * b_kblocks + (kk >> 1)] >> ((kk & 1) * 4)) & 0xFu) - 8;
        }
        const __half w = __hmul(__int2half_rn(q), scale_b[nn * ldsb + kk / bl]);
        acc = __fmaf_rn(a, __half2float(w), acc);
    }
    if (C) acc = __fadd_rn(acc, TdTraits<TD>::load(C, mm * ldc + nn));
    if (bias) acc = __fadd_rn(acc, TdTraits<TD>::load(bias, nn));
    acc = acc < cmin ? cmin : acc;
    acc = acc > cmax ? cmax : acc;
    TdTraits<TD>::store(D, mm * ldd + nn, acc);
}

Result simt_gemm_w4a16(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td, float cmin,
                       float cmax)
{
    if (g.m == 0 || g.n == 0) return Result{kOk, 0};
    if (g.k && env_path() != Path::Simt) {   // tensor cores through tiled TMA loads, where tensor maps can describe the operands
        Result r = umma_gemm_w4a16_unpacked(g, bl, scale_b, ldsb, td, cmin, cmax);
        if (r.status != kUnsupported) return r;
    }
    if (g.m > 65535 || g.n_replicas) return Result{kUnsupported, 0};
    note_kernel(kKernelSimt);
    dim3 grid((unsigned)ceil_div(g.n, 128), (unsigned)g.m);
    cudaStream_t st = (cudaStream_t)g.stream;
    if (td == Dtype::F16)
        gemm_simt_w4a16_kernel<Dtype::F16, true><<<grid, 128, 0, st>>>(g.m, g.n, g.k, bl, (const uint8_t *)g.A, ceil_div(g.lda, 64),
                                                               (const uint8_t *)g.B, ceil_div(g.ldb, 128), (const __half *)scale_b,
                                                               ldsb, g.C, g.ldc, g.D, g.ldd, g.bias, cmin, cmax);
    else
        gemm_simt_w4a16_kernel<Dtype::F32, true><<<grid, 128, 0, st>>>(g.m, g.n, g.k, bl, (const uint8_t *)g.A, ceil_div(g.lda, 64),
                                                               (const uint8_t *)g.B, ceil_div(g.ldb, 128), (const __half *)scale_b,
                                                               ldsb, g.C, g.ldc, g.D, g.ldd, g.bias, cmin, cmax);
    return check_launch();
}

Result launch_gemm_w4a16_unpacked(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td,
                                  float cmin, float cmax)
{
    if (g.m == 0 || g.n == 0) return Result{kOk, 0};
    if (g.m > 65535 || g.n_replicas) return Result{kUnsupported, 0};
    dim3 grid((unsigned)ceil_div(g.n, 128), (unsigned)g.m);
    cudaStream_t st = (cudaStream_t)g.stream;
    if (td == Dtype::F16)
        gemm_simt_w4a16_kernel<Dtype::F16, false><<<grid, 128, 0, st>>>(g.m, g.n, g.k, bl, (const uint8_t *)g.A, g.lda,
                                                                      (const uint8_t *)g.B, g.ldb / 2, (const __half *)scale_b,
                                                                      ldsb, g.C, g.ldc, g.D, g.ldd, g.bias, cmin, cmax);
    else if (td == Dtype::F32)
        gemm_simt_w4a16_kernel<Dtype::F32, false><<<grid, 128, 0, st>>>(g.m, g.n, g.k, bl, (const uint8_t *)g.A, g.lda,
                                                                      (const uint8_t *)g.B, g.ldb / 2, (const __half *)scale_b,
                                                                      ldsb, g.C, g.ldc, g.D, g.ldd, g.bias, cmin, cmax);
    else
        return Result{kUnsupported, 0};
    return check_launch();
}

}  // namespace tqt
