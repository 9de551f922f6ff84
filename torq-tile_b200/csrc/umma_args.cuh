// Argument block and small helpers shared by the tensor-core GEMM kernels (single-CTA and CTA-pair).
#pragma once

#include "dev_common.cuh"

namespace tqt {

enum class BMode : int { I8 = 0, I4Cx = 1, I4C2 = 2 };
enum class EpiKind : int { S32 = 0, Req8 = 1, W4A8 = 2, W4A16 = 3, Req8Row = 4, DxCx = 5, Float = 6 };

// How the int8 CTA-pair kernel fetches an operand: packed 16 KiB blocks by untiled bulk copies, or boxes of the caller's
// row-major matrix by tiled TMA loads (K-major: k contiguous; MN-major, B only: n contiguous).
enum : uint32_t { kSrcBlocks = 0, kSrcTmaK = 1, kSrcTmaMn = 2 };

// A tensor map (the driver's opaque 128-byte descriptor, 64-byte aligned) per operand, passed as a __grid_constant__
// kernel parameter.
struct alignas(64) TmaDesc {
    uint64_t opaque[16];
};
struct TmaOperands {
    TmaDesc a, b;
};

struct UmmaArgs {
    uint32_t m, n, k;
    uint32_t a_src, b_src;     // kSrc*: int8 CTA-pair kernel with tensor maps only
    size_t b_ld;               // row stride (bytes) of a row-major B fetched through a tensor map
    // fused activation quantiser (W4A8, CTA pairs): the kernel first quantises q_rows rows of q_in (16-bit, row stride
    // q_lda elements) into its own packed A operand, scale_a and zp_a, one row per warp, and crosses a grid-wide
    // barrier on grid_sync ([arrivals, generation], a per-device static) before its mainloop roles start
    const void *q_in;
    size_t q_lda;
    int q_bf16;
    unsigned int *grid_sync;
    int in_bf16;               // unquantised 16-bit GEMM: operands are bf16 (else f16)
    int bias_per_row;          // unquantised GEMM: bias indexed by output row (mx1bias types)
    const uint8_t *A;
    const uint8_t *B;
    uint32_t a_kblocks_total;  // blocks per row-tile in the A buffer
    uint32_t b_kblocks_total;  // blocks per row-tile in the B buffer
    uint32_t b_block_bytes;    // int8 CTA-pair kernel: distance between B blocks (16 KiB, or 16 KiB + row sums)
    const void *C;
    size_t ldc;
    void *D;
    size_t ldd;
    const void *bias;
    int vec_store;  // D rows are 16-byte aligned
    // s32 / requant
    int32_t cmin_i, cmax_i;
    float rq_scale_a;
    const float *scale_b;  // requant: per channel; W4A8: per channel
    int rq_per_tensor;
    const float *rq_scale_rows;  // per-row requant (Mx1 bias types): scale_a[m]; rq_scale_a then holds scale_b
    float rq_scale_d;
    int32_t rq_zp_d;
    // W4A8
    const float *scale_a;
    const int32_t *zp_a;
    float cmin_f, cmax_f;
    // W4A16
    const __half *scale_blk;
    size_t ldsb;
    uint32_t bl;
    uint32_t n_replicas;          // output replicas (see GemmCommon)
    long long replica_delta[7];
    int pdl;          // launched with programmatic stream serialisation: wait for the preceding kernel after the prologue
    uint32_t mt;      // tensor-memory kernels: activation rows per tile (0 = default)
    uint32_t band_m;  // tile order: activation-row tiles are walked in bands of this many (0 = one band)
    unsigned int *fault;
    long long *dbg;  // optional per-CTA role timing (diagnostic), 16 slots per CTA
    uint32_t wait_shift;  // test knob: every wait limit is shifted right by this (0 = about a second)
    uint32_t inject;      // test knob, bit 0: the first producer warp withholds the copies and the arrive of its
                          // very first stage, so that the waits downstream of it run out (host-made failure:
                          // nothing traps, faults or spins without a limit)
};

// Tile t of a cm x cn tile grid, walked band by band: inside a band of `band` row tiles the row index
// runs fastest, so the tiles in flight at any time share `band` row tiles and a few column tiles and the
// row-tile operand of a band stays in L2 while the column-tile operand streams through once per band.
__device__ __forceinline__ void tile_coords(uint32_t t, uint32_t cm, uint32_t cn, uint32_t band, uint32_t &im, uint32_t &in)
{
    if (band == 0 || band >= cm) {
        im = t % cm;
        in = t / cm;
        return;
    }
    const uint32_t per_band = band * cn;
    const uint32_t b = t / per_band, r = t - b * per_band;
    const uint32_t m0 = b * band;
    const uint32_t h = min(band, cm - m0);
    im = m0 + r % h;
    in = r / h;
}

// output element type of each epilogue
template <EpiKind EK, Dtype TD>
struct OutType;
template <Dtype TD>
struct OutType<EpiKind::S32, TD> { using type = int32_t; };
template <Dtype TD>
struct OutType<EpiKind::Req8, TD> { using type = int8_t; };
template <Dtype TD>
struct OutType<EpiKind::Req8Row, TD> { using type = int8_t; };
template <Dtype TD>
struct OutType<EpiKind::DxCx, TD> { using type = typename TdTraits<TD>::type; };
template <Dtype TD>
struct OutType<EpiKind::Float, TD> { using type = typename TdTraits<TD>::type; };
template <Dtype TD>
struct OutType<EpiKind::W4A8, TD> { using type = typename TdTraits<TD>::type; };
template <Dtype TD>
struct OutType<EpiKind::W4A16, TD> { using type = typename TdTraits<TD>::type; };

template <typename T>
__device__ __forceinline__ T cvt_out(float v);
template <>
__device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cvt_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cvt_out<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

long long *timing_buffer();
bool pdl_enabled();   // programmatic dependent launch on (TQT_B200_PDL=0 switches it off)
int sm_count_cached();

}  // namespace tqt
