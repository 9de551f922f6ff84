// im2col for the int8 convolution wrappers: the activation tensor is gathered either into a plain matrix or straight
// into the 16 KiB swizzled int8 blocks the tensor-core GEMMs copy into shared memory, so a convolution is one
// gather launch followed by the requantising GEMM of the same kernel type.
//
// Reference counterparts: src/common/tqt_conv.h:52-121 (channel-first im2col: K order (ic, kd, kh, kw), matrix [K, N]),
// :124-196 (channel-last im2col: K order (kd, kh, kw, ic), matrix [M, K]) and the fused im2col + pack of
// src/conv/conv_i8_i8/convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp/
// tqt_convcl_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp_4x1vl_rvv.cpp:96-182.  Padding positions hold 0 there and
// here.  Streaming kernels, bounded by HBM bandwidth on the written matrix.
#include "conv_geom.cuh"

namespace tqt {

namespace {

inline Result conv_check_launch()
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

// One thread per 16-byte chunk of the packed matrix: row = output position, 16 consecutive columns.  Channel-last
// inputs whose channel counts are multiples of 16 move each chunk with one 128-bit load (the 16 columns are 16
// consecutive channels of one input pixel); everything else gathers bytes.  Channel-first: consecutive threads take
// consecutive rows, which are consecutive input pixels along w for stride 1.
template <bool CF>
__global__ void __launch_bounds__(256) im2col_pack_i8_kernel(ConvGeom g, const int8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                                             size_t kblocks, size_t kblocks_total, size_t total_chunks, int vec_ok)
{
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total_chunks;
         idx += (size_t)gridDim.x * blockDim.x) {
        uint32_t c, r;
        if (CF) {
            r = (uint32_t)(idx & 127);
            c = (uint32_t)((idx >> 7) & 7);
        } else {
            c = (uint32_t)(idx & 7);
            r = (uint32_t)((idx >> 3) & 127);
        }
        const size_t blk = idx >> 10, kb = blk % kblocks, tile = blk / kblocks;
        const size_t row = tile * 128 + r;
        const uint32_t k0 = (uint32_t)(kb * 128 + c * 16);
        alignas(16) int8_t v[16];
        *reinterpret_cast<uint4 *>(v) = make_uint4(0u, 0u, 0u, 0u);
        if (row < g.rows && k0 < g.k) {
            uint32_t od, oh, ow;
            split_position(g, (uint32_t)row, od, oh, ow);
            KCursor<CF> cur;
            cur.seek(g, k0);
            size_t off;
            if (!CF && vec_ok) {
                if (cur.source(g, od, oh, ow, off)) *reinterpret_cast<uint4 *>(v) = *reinterpret_cast<const uint4 *>(src + off);
            } else {
#pragma unroll 4
                for (uint32_t e = 0; e < 16; ++e) {
                    if (k0 + e < g.k && cur.source(g, od, oh, ow, off)) v[e] = src[off];
                    cur.next(g);
                }
            }
        }
        uint8_t *blk_base = dst + (tile * kblocks_total + kb) * kI8BlockBytes;
        *reinterpret_cast<uint4 *>(blk_base + sw128_byte(r, c * 16)) = *reinterpret_cast<const uint4 *>(v);
    }
}

// Channel-last inputs whose channel counts are multiples of 16: thread (row, chunk c) walks the K blocks of its row,
// carrying the kernel-window cursor forward by 128 columns per step instead of dividing the column index down again, so a
// 16-byte chunk costs a bounds test, a 128-bit load and a 128-bit store.  A warp still writes four rows x 128 contiguous bytes.
__global__ void __launch_bounds__(256) im2col_pack_cl16_kernel(ConvGeom g, const int8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                                               size_t kblocks, size_t kblocks_total, size_t total_threads)
{
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total_threads; idx += (size_t)gridDim.x * blockDim.x) {
        const uint32_t c = (uint32_t)(idx & 7);
        const size_t row = idx >> 3;               // rows of all tiles, padding rows of the last tile included
        const uint32_t r = (uint32_t)(row & 127);
        uint8_t *out = dst + (row >> 7) * kblocks_total * kI8BlockBytes + sw128_byte(r, c * 16);
        const bool row_ok = row < g.rows;
        uint32_t od = 0, oh = 0, ow = 0;
        KCursor<false> cur;
        cur.kd = cur.kh = cur.kw = cur.ic = 0;
        if (row_ok) {
            split_position(g, (uint32_t)row, od, oh, ow);
            cur.seek(g, c * 16u);
        }
        uint32_t k0 = c * 16u;
        for (size_t kb = 0; kb < kblocks; ++kb, k0 += 128u, out += kI8BlockBytes) {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            size_t off;
            if (row_ok && k0 < g.k && cur.source(g, od, oh, ow, off)) v = *reinterpret_cast<const uint4 *>(src + off);
            *reinterpret_cast<uint4 *>(out) = v;
            // 128 columns on: whole kernel taps are skipped a channel run at a time
            cur.ic += 128u;
            while (cur.ic >= g.ic_pg) {
                cur.ic -= g.ic_pg;
                if (++cur.kw == g.ker[2]) { cur.kw = 0; if (++cur.kh == g.ker[1]) { cur.kh = 0; ++cur.kd; } }
            }
        }
    }
}

// Plain im2col matrix: channel-last [rows, k] (consecutive threads along k = along the input's channels), channel-first
// [k, rows] (consecutive threads along the output positions).
template <bool CF>
__global__ void __launch_bounds__(256) im2col_i8_kernel(ConvGeom g, const int8_t *__restrict__ src, int8_t *__restrict__ dst, size_t total)
{
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        uint32_t pos, k;
        if (CF) {
            k = (uint32_t)(idx / g.rows);
            pos = (uint32_t)(idx - (size_t)k * g.rows);
        } else {
            pos = (uint32_t)(idx / g.k);
            k = (uint32_t)(idx - (size_t)pos * g.k);
        }
        uint32_t od, oh, ow;
        split_position(g, pos, od, oh, ow);
        KCursor<CF> cur;
        cur.seek(g, k);
        size_t off;
        dst[idx] = cur.source(g, od, oh, ow, off) ? src[off] : (int8_t)0;
    }
}

inline unsigned grid_for(size_t items)
{
    const size_t blocks = (items + 255) / 256;
    return (unsigned)(blocks > 148 * 64 ? 148 * 64 : blocks);
}

}  // namespace

Result launch_im2col_pack_i8(void *stream, const ConvGeom &g, bool channel_first, const void *activation, size_t ld_packed,
                             void *packed)
{
    if (g.rows == 0 || g.k == 0) return Result{kOk, 0};
    const size_t kblocks = ceil_div(g.k, 128), kblocks_total = ceil_div(ld_packed, 128);
    if (kblocks_total < kblocks) return Result{kInvalid, 0};
    const size_t chunks = ceil_div(g.rows, 128) * kblocks * 1024;
    cudaStream_t st = (cudaStream_t)stream;
    if (channel_first) {
        im2col_pack_i8_kernel<true><<<grid_for(chunks), 256, 0, st>>>(g, (const int8_t *)activation, (uint8_t *)packed, kblocks,
                                                                     kblocks_total, chunks, 0);
    } else {
        const int vec_ok = g.ic_pg % 16 == 0 && g.c_total % 16 == 0 && (reinterpret_cast<uintptr_t>(activation) & 15) == 0;
        if (vec_ok) {
            const size_t threads = ceil_div(g.rows, 128) * 128 * 8;
            im2col_pack_cl16_kernel<<<grid_for(threads), 256, 0, st>>>(g, (const int8_t *)activation, (uint8_t *)packed, kblocks,
                                                                      kblocks_total, threads);
        } else {
            im2col_pack_i8_kernel<false><<<grid_for(chunks), 256, 0, st>>>(g, (const int8_t *)activation, (uint8_t *)packed, kblocks,
                                                                          kblocks_total, chunks, 0);
        }
    }
    return conv_check_launch();
}

Result launch_im2col_i8(void *stream, const ConvGeom &g, bool channel_first, const void *activation, void *matrix)
{
    if (g.rows == 0 || g.k == 0) return Result{kOk, 0};
    const size_t total = (size_t)g.rows * g.k;
    cudaStream_t st = (cudaStream_t)stream;
    if (channel_first)
        im2col_i8_kernel<true><<<grid_for(total), 256, 0, st>>>(g, (const int8_t *)activation, (int8_t *)matrix, total);
    else
        im2col_i8_kernel<false><<<grid_for(total), 256, 0, st>>>(g, (const int8_t *)activation, (int8_t *)matrix, total);
    return conv_check_launch();
}

}  // namespace tqt
