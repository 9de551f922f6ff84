// One-time layout kernels: LHS / RHS packers (and their inverses) and the qai8dx activation
// quantiser.  All are streaming kernels bounded by HBM bandwidth.
//
// Reference counterparts: src/common/tqt_gemm_pack_rvv.h:740-772 (A row interleave),
// :777-798 (B^T int8 / int4-as-bytes), :542-567 (B [k,n]), :852-856 (qsi4c2); the quantiser follows
// test/gemm/test_gemm_i8_i4_rvv.cpp:40-77.  The packed layouts here are different by design: blocks
// of 128 rows in the order the tensor-core kernels copy straight into shared memory.
#include "dev_common.cuh"
#include "quant_row.cuh"

namespace tqt {

int sm_count_cached();   // kernels_umma.cu

bool pdl_enabled();   // kernels_gemv.cu: programmatic dependent launch on (TQT_B200_PDL=0 switches it off)

__device__ unsigned int g_device_fault = 0;

unsigned int *fault_word_device_ptr()
{
    static unsigned int *cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    unsigned int *p = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        void *addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_device_fault) != cudaSuccess) return nullptr;
        p = static_cast<unsigned int *>(addr);
        __atomic_store_n(&cache[dev], p, __ATOMIC_RELEASE);
    }
    return p;
}

static inline Result check_launch()
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

// ---- swizzled 128 x 128 B blocks (int8 / f16) ---------------------------------------------------
// One thread per 16-byte chunk of the destination.  grid.x covers chunks, ES = element size.
template <int ES, bool TRANSPOSED>
__global__ void pack_rows_kernel(size_t rows, size_t k, size_t ld_src, size_t kblocks_total, const uint8_t *__restrict__ src,
                                 uint8_t *__restrict__ dst, size_t kblocks, size_t total_chunks, size_t block_bytes)
{
    constexpr uint32_t EPC = 16 / ES;          // elements per 16-byte chunk
    constexpr uint32_t KPB = 128 / ES;         // k elements per block row
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total_chunks;
         idx += (size_t)gridDim.x * blockDim.x) {
        uint32_t c, r;
        size_t blk;
        if (TRANSPOSED) {  // consecutive threads -> consecutive rows (coalesced reads of [k, rows])
            r = (uint32_t)(idx & 127);
            c = (uint32_t)((idx >> 7) & 7);
            blk = idx >> 10;
        } else {  // consecutive threads -> consecutive chunks of a row
            c = (uint32_t)(idx & 7);
            r = (uint32_t)((idx >> 3) & 127);
            blk = idx >> 10;
        }
        const size_t kb = blk % kblocks, tile = blk / kblocks;
        const size_t row = tile * 128 + r;
        const size_t k0 = kb * KPB + (size_t)c * EPC;
        alignas(16) uint8_t v[16];
        if (!TRANSPOSED && row < rows && k0 + EPC <= k &&
            ((reinterpret_cast<uintptr_t>(src + (row * ld_src + k0) * ES) & 15) == 0)) {
            *reinterpret_cast<uint4 *>(v) = *reinterpret_cast<const uint4 *>(src + (row * ld_src + k0) * ES);
        } else {
#pragma unroll
            for (uint32_t e = 0; e < EPC; ++e) {
                const size_t kk = k0 + e;
                const bool ok = row < rows && kk < k;
                const size_t off = TRANSPOSED ? (kk * ld_src + row) : (row * ld_src + kk);
#pragma unroll
                for (int b = 0; b < ES; ++b) v[e * ES + b] = ok ? src[off * ES + b] : (uint8_t)0;
            }
        }
        uint8_t *blk_base = dst + (tile * kblocks_total + kb) * block_bytes;
        *reinterpret_cast<uint4 *>(blk_base + sw128_byte(r, c * 16)) = *reinterpret_cast<const uint4 *>(v);
    }
}

template <int ES>
__global__ void unpack_rows_kernel(size_t rows, size_t k, size_t kblocks_total, const uint8_t *__restrict__ src,
                                   uint8_t *__restrict__ dst, size_t ld_dst)
{
    constexpr uint32_t KPB = 128 / ES;
    const size_t total = rows * k;
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t row = idx / k, kk = idx % k;
        const size_t tile = row >> 7, kb = kk / KPB;
        const uint32_t r = (uint32_t)(row & 127), e = (uint32_t)(kk % KPB);
        const uint8_t *p = src + (tile * kblocks_total + kb) * kI8BlockBytes + sw128_byte(r, e * ES);
#pragma unroll
        for (int b = 0; b < ES; ++b) dst[(row * ld_dst + kk) * ES + b] = p[b];
    }
}

// One thread per (block, row): the int16 sum of the row's 128 int8 values (the swizzle permutes inside a row only).
__global__ void block_row_sums_kernel(uint8_t *__restrict__ packed, size_t tiles, size_t kblocks, size_t kblocks_total)
{
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= tiles * kblocks * 128) return;
    const uint32_t r = (uint32_t)(idx & 127);
    const size_t blk = idx >> 7, kb = blk % kblocks, tile = blk / kblocks;
    uint8_t *base = packed + (tile * kblocks_total + kb) * kI8SumBlockBytes;
    int32_t sum = 0;
#pragma unroll
    for (uint32_t c = 0; c < 8; ++c) {
        const uint4 v = *reinterpret_cast<const uint4 *>(base + r * 128u + c * 16u);
        sum = __dp4a((int)v.x, 0x01010101, sum);
        sum = __dp4a((int)v.y, 0x01010101, sum);
        sum = __dp4a((int)v.z, 0x01010101, sum);
        sum = __dp4a((int)v.w, 0x01010101, sum);
    }
    reinterpret_cast<int16_t *>(base + kI8BlockBytes)[r] = (int16_t)sum;
}

static Result pack_rows_impl(void *stream, size_t rows, size_t k, size_t ld_src, size_t ld_packed, const void *src,
                             void *dst, int elem_size, bool transposed_src, size_t block_bytes);

Result launch_pack_rows(void *stream, size_t rows, size_t k, size_t ld_src, size_t ld_packed, const void *src,
                        void *dst, int elem_size, bool transposed_src)
{
    return pack_rows_impl(stream, rows, k, ld_src, ld_packed, src, dst, elem_size, transposed_src, kI8BlockBytes);
}

Result launch_pack_rows_sums(void *stream, size_t rows, size_t k, size_t ld_src, size_t ld_packed, const void *src,
                             void *dst, bool transposed_src)
{
    if (rows == 0 || k == 0) return Result{kOk, 0};
    Result r = pack_rows_impl(stream, rows, k, ld_src, ld_packed, src, dst, 1, transposed_src, kI8SumBlockBytes);
    if (r.status != kOk) return r;
    const size_t tiles = ceil_div(rows, 128), kblocks = ceil_div(k, 128), total = tiles * kblocks * 128;
    block_row_sums_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, (cudaStream_t)stream>>>((uint8_t *)dst, tiles, kblocks,
                                                                                          ceil_div(ld_packed, 128));
    return check_launch();
}

static Result pack_rows_impl(void *stream, size_t rows, size_t k, size_t ld_src, size_t ld_packed, const void *src,
                             void *dst, int elem_size, bool transposed_src, size_t block_bytes)
{
    if (rows == 0 || k == 0) return Result{kOk, 0};
    const size_t kpb = 128 / elem_size;
    const size_t kblocks = ceil_div(k, kpb), kblocks_total = ceil_div(ld_packed, kpb);
    const size_t tiles = ceil_div(rows, 128);
    const size_t chunks = tiles * kblocks * 1024;
    const int threads = 256;
    const unsigned grid = (unsigned)((chunks + threads - 1) / threads > 148 * 64 ? 148 * 64 : (chunks + threads - 1) / threads);
    cudaStream_t st = (cudaStream_t)stream;
    const uint8_t *s = (const uint8_t *)src;
    uint8_t *d = (uint8_t *)dst;
    if (elem_size == 1) {
        if (transposed_src)
            pack_rows_kernel<1, true><<<grid, threads, 0, st>>>(rows, k, ld_src, kblocks_total, s, d, kblocks, chunks, block_bytes);
        else
            pack_rows_kernel<1, false><<<grid, threads, 0, st>>>(rows, k, ld_src, kblocks_total, s, d, kblocks, chunks, block_bytes);
    } else if (elem_size == 2) {
        if (transposed_src)
            pack_rows_kernel<2, true><<<grid, threads, 0, st>>>(rows, k, ld_src, kblocks_total, s, d, kblocks, chunks, block_bytes);
        else
            pack_rows_kernel<2, false><<<grid, threads, 0, st>>>(rows, k, ld_src, kblocks_total, s, d, kblocks, chunks, block_bytes);
    } else {
        if (transposed_src)
            pack_rows_kernel<4, true><<<grid, threads, 0, st>>>(rows, k, ld_src, kblocks_total, s, d, kblocks, chunks, block_bytes);
        else
            pack_rows_kernel<4, false><<<grid, threads, 0, st>>>(rows, k, ld_src, kblocks_total, s, d, kblocks, chunks, block_bytes);
    }
    return check_launch();
}

Result launch_unpack_rows(void *stream, size_t rows, size_t k, size_t ld_packed, const void *src, void *dst,
                          size_t ld_dst, int elem_size)
{
    if (rows == 0 || k == 0) return Result{kOk, 0};
    const size_t kpb = 128 / elem_size;
    const size_t total = rows * k;
    const int threads = 256;
    const unsigned grid = (unsigned)((total + threads - 1) / threads > 148 * 64 ? 148 * 64 : (total + threads - 1) / threads);
    cudaStream_t st = (cudaStream_t)stream;
    if (elem_size == 1)
        unpack_rows_kernel<1><<<grid, threads, 0, st>>>(rows, k, ceil_div(ld_packed, kpb), (const uint8_t *)src,
                                                       (uint8_t *)dst, ld_dst);
    else
        unpack_rows_kernel<2><<<grid, threads, 0, st>>>(rows, k, ceil_div(ld_packed, kpb), (const uint8_t *)src,
                                                       (uint8_t *)dst, ld_dst);
    return check_launch();
}

// ---- int4 blocks -----------------------------------------------------------------------------------
// One CTA of 128 threads per (row-tile, k-block).  The 128 x 64-byte source tile is read with row-contiguous
// 128-bit loads (four threads per row: every 32-byte sector is fetched whole, once) into shared memory, at a
// swizzled position so that the per-row reads that follow are conflict-free; thread r then owns row r of the
// block: it re-orders the nibbles of its 64 bytes, (qsi4cx) adds up the row's partial sum, and writes its four
// 16-byte segments, which makes the CTA's output one contiguous 8 KiB (+ 256 B of sums) stream.  Sources whose
// rows are not 16-byte aligned, and the ragged right / bottom edges, take byte loads.
template <bool C2>
__global__ void __launch_bounds__(128) pack_i4_kernel(size_t n, size_t k, size_t ld_src_bytes, size_t kblocks_total,
                                                      const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, size_t kblocks,
                                                      int aligned)
{
    constexpr size_t BLOCK_BYTES = C2 ? kI4C2BlockBytes : kI4CxBlockBytes;
    __shared__ uint4 sTile[128 * 4];
    const size_t blk = blockIdx.x;
    const size_t kb = blk % kblocks, tile = blk / kblocks;
    const uint32_t r = threadIdx.x;
    uint8_t *base = dst + (tile * kblocks_total + kb) * BLOCK_BYTES;
    const size_t kbyte0 = kb * 64;
    const size_t kbytes = k / 2;

    // stage: chunk c = (row c / 4, 16-byte segment c % 4); consecutive threads take consecutive chunks
#pragma unroll
    for (uint32_t u = 0; u < 4; ++u) {
        const uint32_t c = r + u * 128u, lr = c >> 2, seg = c & 3u;
        const size_t row = tile * 128 + lr, kbyte = kbyte0 + seg * 16u;
        uint4 v = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);   // nibble 8 == value 0 (padding)
        if (row < n && kbyte < kbytes) {
            const uint8_t *p = src + row * ld_src_bytes + kbyte;
            if (aligned && kbyte + 16 <= kbytes) {
                v = __ldg(reinterpret_cast<const uint4 *>(p));
            } else {
                uint32_t w[4] = {0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u};
                for (uint32_t b = 0; b < 16 && kbyte + b < kbytes; ++b)
                    w[b >> 2] = (w[b >> 2] & ~(0xFFu << ((b & 3u) * 8u))) | ((uint32_t)p[b] << ((b & 3u) * 8u));
                v = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        sTile[lr * 4u + (seg ^ ((lr >> 1) & 3u))] = v;
    }
    __syncthreads();

    // this thread's row: 64 source bytes = 128 stored nibbles (value q + 8), k ascending
    uint32_t raw[16];
#pragma unroll
    for (uint32_t sg = 0; sg < 4; ++sg) {
        const uint4 v = sTile[r * 4u + (sg ^ ((r >> 1) & 3u))];
        raw[sg * 4 + 0] = v.x;
        raw[sg * 4 + 1] = v.y;
        raw[sg * 4 + 2] = v.z;
        raw[sg * 4 + 3] = v.w;
    }
    // Re-order whole words.  Source word w of a 32-k segment holds the stored nibbles (value q + 8) of k = 8 w ..
    // 8 w + 7, nibble i at bits 4 i.
    //   qsi4cx: output word j, byte b = q[4 j + b] | q[16 + 4 j + b] << 4 in two's complement: the four nibbles of
    //           a 16-bit half of a source word are spread over the low nibbles of four bytes.
    //   qsi4c2: output word j holds k = 8 j .. 8 j + 7 as (k0, k2, k4, k6, k1, k3, k5, k7), unsigned as stored: the
    //           even nibbles of source word j compressed into the low half, the odd ones into the high half.
    uint32_t out[16];
    int psum = -8 * 128;
    auto spread = [](uint32_t h) {   // nibbles n0..n3 of a 16-bit value -> bytes 0x0n3 0x0n2 0x0n1 0x0n0
        const uint32_t t = (h | (h << 8)) & 0x00FF00FFu;
        return (t | (t << 4)) & 0x0F0F0F0Fu;
    };
    auto even_nibbles = [](uint32_t w) {   // nibbles 0, 2, 4, 6 -> the low 16 bits
        uint32_t x = w & 0x0F0F0F0Fu;
        x = (x | (x >> 4)) & 0x00FF00FFu;
        return (x | (x >> 8)) & 0x0000FFFFu;
    };
#pragma unroll
    for (uint32_t sg = 0; sg < 4; ++sg) {
        const uint32_t *w = raw + sg * 4;
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            psum += __dp4a((int)((w[j] & 0x0F0F0F0Fu) + ((w[j] >> 4) & 0x0F0F0F0Fu)), 0x01010101, 0);
            if (C2) {
                out[sg * 4 + j] = even_nibbles(w[j]) | (even_nibbles(w[j] >> 4) << 16);
            } else {
                const uint32_t lo = (w[j >> 1] >> (16u * (j & 1u))) & 0xFFFFu;        // k = 4 j .. 4 j + 3
                const uint32_t hi = (w[2 + (j >> 1)] >> (16u * (j & 1u))) & 0xFFFFu;  // k = 16 + 4 j .. + 3
                out[sg * 4 + j] = (spread(lo) | (spread(hi) << 4)) ^ 0x88888888u;
            }
        }
    }
    // write the four 16-byte segments at their swizzled positions
#pragma unroll
    for (uint32_t sg = 0; sg < 4; ++sg) {
        const uint32_t pos = sg ^ ((r >> 1) & 3u);
        *reinterpret_cast<uint4 *>(base + r * 64u + pos * 16u) =
            make_uint4(out[sg * 4 + 0], out[sg * 4 + 1], out[sg * 4 + 2], out[sg * 4 + 3]);
    }
    if (!C2) reinterpret_cast<int16_t *>(base + kI4NibBytes)[r] = (int16_t)psum;
}

template <bool C2>
__global__ void unpack_i4_kernel(size_t n, size_t k, size_t kblocks_total, const uint8_t *__restrict__ src,
                                 uint8_t *__restrict__ dst, size_t ld_dst_bytes)
{
    constexpr size_t BLOCK_BYTES = C2 ? kI4C2BlockBytes : kI4CxBlockBytes;
    const size_t total = n * (k / 2);
    for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t row = idx / (k / 2), kbyte = idx % (k / 2);
        uint32_t outb = 0;
        for (uint32_t h = 0; h < 2; ++h) {
            const size_t kk = kbyte * 2 + h;
            const size_t tile = row >> 7, kb = kk >> 7;
            const uint32_t r = (uint32_t)(row & 127);
            uint32_t hi;
            const uint32_t byte = C2 ? i4c2_byte(r, (uint32_t)(kk & 127), &hi) : i4cx_byte(r, (uint32_t)(kk & 127), &hi);
            uint32_t v = (src[(tile * kblocks_total + kb) * BLOCK_BYTES + byte] >> (hi * 4)) & 0xFu;
            if (!C2) v ^= 8u;
            outb |= v << (h * 4);
        }
        dst[row * ld_dst_bytes + kbyte] = (uint8_t)outb;
    }
}

Result launch_pack_i4(void *stream, size_t n, size_t k, size_t ld_src_bytes, size_t ld_packed, const void *src,
                      void *dst, bool c2)
{
    if (n == 0 || k == 0) return Result{kOk, 0};
    const size_t kblocks = ceil_div(k, 128), kblocks_total = ceil_div(ld_packed, 128);
    const size_t blocks = ceil_div(n, 128) * kblocks;
    if (blocks > 0x7fffffffull) return Result{kUnsupported, 0};
    cudaStream_t st = (cudaStream_t)stream;
    // 128-bit source loads need 16-byte aligned rows (k blocks start at multiples of 64 bytes)
    const int aligned = ((reinterpret_cast<uintptr_t>(src) & 15) == 0 && (ld_src_bytes & 15) == 0) ? 1 : 0;
    if (c2)
        pack_i4_kernel<true><<<(unsigned)blocks, 128, 0, st>>>(n, k, ld_src_bytes, kblocks_total, (const uint8_t *)src,
                                                             (uint8_t *)dst, kblocks, aligned);
    else
        pack_i4_kernel<false><<<(unsigned)blocks, 128, 0, st>>>(n, k, ld_src_bytes, kblocks_total, (const uint8_t *)src,
                                                              (uint8_t *)dst, kblocks, aligned);
    return check_launch();
}

Result launch_unpack_i4(void *stream, size_t n, size_t k, size_t ld_packed, const void *src, void *dst,
                        size_t ld_dst_bytes, bool c2)
{
    if (n == 0 || k == 0) return Result{kOk, 0};
    const size_t total = n * (k / 2);
    const int threads = 256;
    const unsigned grid = (unsigned)((total + threads - 1) / threads > 148 * 64 ? 148 * 64 : (total + threads - 1) / threads);
    cudaStream_t st = (cudaStream_t)stream;
    if (c2)
        unpack_i4_kernel<true><<<grid, threads, 0, st>>>(n, k, ceil_div(ld_packed, 128), (const uint8_t *)src, (uint8_t *)dst, ld_dst_bytes);
    else
        unpack_i4_kernel<false><<<grid, threads, 0, st>>>(n, k, ceil_div(ld_packed, 128), (const uint8_t *)src, (uint8_t *)dst, ld_dst_bytes);
    return check_launch();
}

// ---- qai8dx: per-row asymmetric int8 quantiser -----------------------------------------------------
// One CTA per row.  Pass 1: min/max with 128-bit loads and a warp-shuffle + shared-memory reduction.
// Pass 2: re-read the row (it is in L2), quantise 16 elements per thread, store one 16-byte chunk.
template <Dtype TA>
__device__ inline void load16(const void *A, size_t base, size_t k_left, bool aligned, float (&x)[16])
{
    if (aligned && k_left >= 16) {
        if (TA == Dtype::F32) {
            const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(A) + base);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 v = __ldg(p + i);
                x[4 * i + 0] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
            }
        } else {
            const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(A) + base);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint4 v = __ldg(p + i);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (TA == Dtype::F16) {
                        const __half2 h = *reinterpret_cast<const __half2 *>(&w[j]);
                        x[8 * i + 2 * j] = __low2float(h);
                        x[8 * i + 2 * j + 1] = __high2float(h);
                    } else {
                        x[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
                        x[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                    }
                }
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = (size_t)i < k_left ? TdTraits<TA>::load(A, base + i) : 0.0f;
    }
}

template <Dtype TA, bool PACKED>
__global__ void __launch_bounds__(256) quant_qai8dx_kernel(size_t m, size_t k, const void *__restrict__ A, size_t lda,
                                                           uint8_t *__restrict__ out, size_t ldq, size_t kblocks_total,
                                                           float *__restrict__ scale_a, int32_t *__restrict__ zp_a)
{
    __shared__ float s_min[8], s_max[8];
    __shared__ float s_scale;
    __shared__ int s_zp;
    const size_t row = blockIdx.x;
    const size_t row_base = row * lda;
    constexpr int ES = (TA == Dtype::F32) ? 4 : 2;
    const bool aligned = ((reinterpret_cast<uintptr_t>(A) + row_base * ES) & 15) == 0;
    const size_t nchunks = (k + 15) / 16;

    // Rows of up to 16 * blockDim elements (K <= 4096 with 256 threads) are held in registers between
    // the min/max pass and the quantise pass; longer rows are read again (from L2).
    const size_t out_chunks_all = PACKED ? ((k + 127) / 128) * 8 : nchunks;
    const bool in_regs = out_chunks_all <= blockDim.x;
    float xr[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) xr[i] = 0.0f;
    float vmin = 3.402823466e+38f, vmax = -3.402823466e+38f;
    for (size_t c = threadIdx.x; c < nchunks; c += blockDim.x) {
        float x[16];
        const size_t k0 = c * 16;
        load16<TA>(A, row_base + k0, k - k0, aligned, x);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if ((size_t)i < k - k0) {
                vmin = x[i] < vmin ? x[i] : vmin;
                vmax = x[i] > vmax ? x[i] : vmax;
            }
            if (in_regs) xr[i] = x[i];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    }
    if ((threadIdx.x & 31) == 0) {
        s_min[threadIdx.x >> 5] = vmin;
        s_max[threadIdx.x >> 5] = vmax;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float fmin_ = s_min[0], fmax_ = s_max[0];
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
            fmin_ = fminf(fmin_, s_min[w]);
            fmax_ = fmaxf(fmax_, s_max[w]);
        }
        fmax_ = fmax_ > 0.0f ? fmax_ : 0.0f;
        fmin_ = fmin_ < 0.0f ? fmin_ : 0.0f;
        const float s = __fdiv_rn(__fsub_rn(fmax_, fmin_), 255.0f);
        int zp = 0;
        float sc = 1.0f;
        if (s != 0.0f) {
            const float zp_tmp = __fsub_rn(-128.0f, __fdiv_rn(fmin_, s));
            zp = (int)rintf(zp_tmp);
            zp = zp < -128 ? -128 : (zp > 127 ? 127 : zp);
            sc = s;
        }
        s_scale = (s != 0.0f) ? s : 0.0f;  // 0 marks the all-zero row
        s_zp = zp;
        scale_a[row] = sc;
        zp_a[row] = zp;
    }
    __syncthreads();
    const float s = s_scale;
    const float zpf = (float)s_zp;

    const size_t tile = row >> 7;
    const uint32_t r = (uint32_t)(row & 127);
    // packed rows are padded with zeros up to the block width
    const size_t out_chunks = out_chunks_all;
    for (size_t c = threadIdx.x; c < out_chunks; c += blockDim.x) {
        const size_t k0 = c * 16;
        alignas(16) int8_t q[16];
        if (k0 < k && s != 0.0f) {
            float x[16];
            if (in_regs) {
#pragma unroll
                for (int i = 0; i < 16; ++i) x[i] = xr[i];
            } else {
                load16<TA>(A, row_base + k0, k - k0, aligned, x);
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float v = __fadd_rn(rintf(__fdiv_rn(x[i], s)), zpf);
                v = v > 127.0f ? 127.0f : v;
                v = v < -128.0f ? -128.0f : v;
                q[i] = ((size_t)i < k - k0) ? (int8_t)v : (int8_t)0;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) q[i] = 0;
        }
        if (PACKED) {
            const size_t kb = c >> 3;
            uint8_t *base = out + (tile * kblocks_total + kb) * kI8BlockBytes;
            *reinterpret_cast<uint4 *>(base + sw128_byte(r, (uint32_t)(c & 7) * 16)) = *reinterpret_cast<const uint4 *>(q);
        } else {
            int8_t *dst = reinterpret_cast<int8_t *>(out) + row * ldq + k0;
            if (k - k0 >= 16 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
                *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(q);
            } else {
                for (int i = 0; i < 16 && (size_t)i < k - k0; ++i) dst[i] = q[i];
            }
        }
    }
}

// Warp-per-row variant for 16-bit inputs whose rows fit in registers: see quant_row.cuh.  SPLIT warps share a row.
template <Dtype TA, bool PACKED, uint32_t SPLIT>
__global__ void __launch_bounds__(256) quant_qai8dx_warp_kernel(size_t m, size_t k, const void *__restrict__ A, size_t lda,
                                                                uint8_t *__restrict__ out, size_t ldq, size_t kblocks_total,
                                                                float *__restrict__ scale_a, int32_t *__restrict__ zp_a)
{
    // programmatic dependent launch: the GEMM that follows may run its prologue now; this kernel itself waits
    // for its predecessor (which may still read the packed buffer it is about to overwrite) before touching memory
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ float s_red[16];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t slot = warp / SPLIT, sub = warp % SPLIT;
    const size_t row = (size_t)blockIdx.x * (8 / SPLIT) + slot;
    if (row >= m) return;   // a whole row's warps leave together: the named barrier below is per row
    quant_row_warp<TA, PACKED, SPLIT>(row, k, A, lda, out, ldq, kblocks_total, scale_a, zp_a, lane, sub, s_red + slot * SPLIT * 2,
                                      1u + slot);
}

Result launch_quant_qai8dx(void *stream, size_t m, size_t k, const void *A, size_t lda, Dtype ta, void *out,
                           size_t ldq, bool packed, float *scale_a, int32_t *zp_a)
{
    if (m == 0 || k == 0) return Result{kOk, 0};
    if (m > 0x7fffffffull) return Result{kUnsupported, 0};
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)m;
    const size_t kbt = ceil_div(k, 128);
    uint8_t *o = (uint8_t *)out;
    // many 16-bit rows that fit in registers: one warp per row
    const bool warp_rows = ta != Dtype::F32 && m >= 32 && k <= 4096 && k % 16 == 0 && lda % 8 == 0 &&
                           (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
                           (packed || (ldq % 16 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0));
    if (warp_rows) {
        // warps per row: a row's loads, its reduction and its stores run one after the other in a warp, so more and
        // lighter warps overlap them better.  Measured on k = 4096 bf16 rows (us for 1 / 2 / 4 warps per row): 1024 rows
        // 6.4 / 6.0 / 4.5, 2048 rows 7.8 / 7.1 / 7.3, 8192 rows 20.5 / 18.0 / 20.5.
        unsigned split = 1;
        if (m * 4 <= (size_t)sm_count_cached() * 32 && k >= 2048) split = 4;
        else if (k >= 1024) split = 2;
        const unsigned rows_per_cta = 8 / split;
        const unsigned wgrid = (unsigned)((m + rows_per_cta - 1) / rows_per_cta);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(wgrid, 1, 1);
        cfg.blockDim = dim3(256, 1, 1);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = pdl_enabled() ? 1 : 0;   // without the attribute the two griddepcontrol instructions are no-ops
        cudaError_t e = cudaSuccess;
#define TQT_LAUNCH_QW2(TA_, PK_)                                                                                                     \
    do {                                                                                                                             \
        if (split == 4)                                                                                                              \
            e = cudaLaunchKernelEx(&cfg, quant_qai8dx_warp_kernel<TA_, PK_, 4>, m, k, A, lda, o, ldq, kbt, scale_a, zp_a);           \
        else if (split == 2)                                                                                                         \
            e = cudaLaunchKernelEx(&cfg, quant_qai8dx_warp_kernel<TA_, PK_, 2>, m, k, A, lda, o, ldq, kbt, scale_a, zp_a);           \
        else                                                                                                                         \
            e = cudaLaunchKernelEx(&cfg, quant_qai8dx_warp_kernel<TA_, PK_, 1>, m, k, A, lda, o, ldq, kbt, scale_a, zp_a);           \
    } while (0)
#define TQT_LAUNCH_QW(TA_)                                                                                             \
    do {                                                                                                               \
        if (packed)                                                                                                    \
            TQT_LAUNCH_QW2(TA_, true);                                                                                 \
        else                                                                                                           \
            TQT_LAUNCH_QW2(TA_, false);                                                                                \
    } while (0)
        if (ta == Dtype::F16)
            TQT_LAUNCH_QW(Dtype::F16);
        else
            TQT_LAUNCH_QW(Dtype::BF16);
#undef TQT_LAUNCH_QW2
#undef TQT_LAUNCH_QW
        if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
        return check_launch();
    }
#define TQT_LAUNCH_Q(TA_)                                                                                              \
    do {                                                                                                               \
        if (packed)                                                                                                    \
            quant_qai8dx_kernel<TA_, true><<<grid, 256, 0, st>>>(m, k, A, lda, o, ldq, kbt, scale_a, zp_a);            \
        else                                                                                                           \
            quant_qai8dx_kernel<TA_, false><<<grid, 256, 0, st>>>(m, k, A, lda, o, ldq, kbt, scale_a, zp_a);           \
    } while (0)
    switch (ta) {
        case Dtype::F32: TQT_LAUNCH_Q(Dtype::F32); break;
        case Dtype::F16: TQT_LAUNCH_Q(Dtype::F16); break;
        case Dtype::BF16: TQT_LAUNCH_Q(Dtype::BF16); break;
    }
#undef TQT_LAUNCH_Q
    return check_launch();
}

int read_device_fault(void *stream)
{
    unsigned int v = 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (cudaStreamSynchronize(st) != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, g_device_fault, sizeof(v)) != cudaSuccess) return -1;
    if (v != 0) {
        unsigned int z = 0;
        cudaMemcpyToSymbol(g_device_fault, &z, sizeof(z));
    }
    return (int)v;
}

}  // namespace tqt
