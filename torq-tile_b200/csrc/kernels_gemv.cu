// HBM-streaming W4A8 GEMV for decode (m <= 16; more rows run on the tensor-core kernel): no tcgen05, no
// clusters, no shared-memory staging of weights, no scratch memory.  Two kernels share the structure below:
// gemv_w4a8_kernel (m = 1, dp4a) and gemv_mma_kernel (2 <= m <= 16, mma.sync m16n8k32: the 16-row A fragment is a
// decode batch, so every batch size costs nearly what m = 2 does).
//
// A CTA owns one or two groups of 8 consecutive output columns (8 rows of one 128-row block tile of B_packed) and
// loops over such sets when there are more than resident CTAs; its eight warps take interleaved K blocks.  Inside
// a warp lane = (row, 16-byte segment), so one warp-wide 128-bit load covers 512 contiguous bytes of a packed
// block: every 32-byte sector is used whole, once.  A thread holds four weight loads per group at a time: on this
// part a streaming read reaches full bandwidth with many warps that each have a few loads outstanding, not with
// few warps that have many.  The next set's loads are issued as soon as the registers are free, before the
// current set is combined and stored.
// Nibbles are expanded with two logic ops per 8 weights (operands 16*q, as in the tensor-core kernel); the
// zero-point correction uses the int16 partial row sums stored at the tail of every packed block (dp4a kernel) or
// sums the same words against ones (mma kernel).  The segments of a row are combined with warp shuffles and the
// eight warps through shared memory: integer sums, so the result is exact and independent of the split.  The
// epilogue is the GEMM's (reference:
// src/gemm/gemm_i8_i4/gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp/..._4x1vl_rvv.cpp:118-177).
//
// Programmatic dependent launch: the kernel lets its successor start at once and requests its weights before
// waiting for its predecessor, so back-to-back GEMVs (the layers of a decode step) overlap their memory phases.
// Everything after that wait is on the critical path of the chain (a kernel's wait ends only when its
// predecessor has completed), so it is kept short.  Activations, C and D are touched only after the wait.
// TQT_B200_PDL=0 switches this off.
#include <cstdlib>

#include "epilogues.cuh"
#include "ptx_sm100.cuh"

namespace tqt {

int sm_count_cached();
long long *timing_buffer();   // kernels_umma.cu

constexpr uint32_t kGemvThreads = 256;
constexpr uint32_t kGemvWarpRows = 8;   // output columns per warp
constexpr uint32_t kGemvMaxRows = 16;  // activation rows the GEMV takes (decode batch)

struct GemvArgs {
    uint32_t m, n, k;
    const uint8_t *A;  // packed int8 blocks (row-tile 0 only: m <= 16)
    const uint8_t *B;  // packed qsi4cx blocks
    uint32_t b_kblocks_total;
    const void *C;
    size_t ldc;
    void *D;
    size_t ldd;
    const void *bias;
    const float *scale_a;
    const int32_t *zp_a;
    const float *scale_b;
    float cmin, cmax;
    int pdl;
    long long *dbg;   // diagnostic (tqt_cuda_debug_set_timing_buffer): thread 0 of CTAs 0..147 stores clock64 phase stamps, 16 slots per CTA
};

// Phase stamps of the dp4a GEMV (cycles of the CTA's SM clock): 0 kernel entry, 1 first set's weight loads issued,
// 2 griddepcontrol.wait returned, 3 K loop done (activations fetched, dp4a chain), 4 partial sums combined, 5 output stored.
__device__ __forceinline__ void gemv_stamp(const GemvArgs &args, int slot)
{
#ifdef TQT_B200_DIAG   // diagnostic builds only: the six predicated stamps cost a 2.3 us GEMV 1.5 %
    if (args.dbg && threadIdx.x == 0 && blockIdx.x < 148u) args.dbg[blockIdx.x * 16u + slot] = clock64();
#else
    (void)args;
    (void)slot;
#endif
}

// 128-bit streaming load: read-only path, do not keep the line in L1.
__device__ __forceinline__ uint4 ldg_stream(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

constexpr uint32_t kGemvSlices = kGemvThreads / 32;   // warps of a CTA = interleaved K slices
constexpr uint32_t kGemvChunk = 4;                   // loads in flight per thread

// G = 8-column groups a CTA works on at the same time.  With G = 1 a launch of N / 8 CTAs fills up to four
// CTA slots per SM; a decode-sized launch (N = 4096: 512 CTAs on 592 slots) then leaves its successor nowhere
// to become resident, so the successor's weight loads start only when this kernel's CTAs exit and the memory
// phases of back-to-back GEMVs do not overlap.  With G = 2 a CTA streams 16 columns (eight 128-bit loads in
// flight per thread, the activation words shared by both groups), the launch takes two slots per SM, and the
// next GEMV of the chain is resident and has its weights in flight while this one runs its post-wait tail.
//
// Measured on chains of 48 GEMVs (M = 1, K = N = 4096, programmatic dependent launch): G = 2 2.3-2.5 us per GEMV,
// G = 1 3.4 us; the same kernel without the wait for its predecessor 1.85 us, a kernel that only reads the bytes
// 1.2 us.  Holding the loads in flight in shared memory instead of registers (cp.async or bulk copies, to make room
// for the successor's CTAs) was slower in every form tried: a kernel's shared-memory carve-out is sized for its own
// CTAs, so the successor's CTAs did not become resident beside it, and static shared memory of a few KiB alone cost
// the chain 1 us per GEMV.
template <int MR, int G>
constexpr int gemv_min_ctas() { return G == 2 ? 2 : (MR <= 2 ? 4 : (MR <= 8 ? 3 : 2)); }

template <int MR, int G, Dtype TD>
__global__ void __launch_bounds__(kGemvThreads, gemv_min_ctas<MR, G>()) gemv_w4a8_kernel(const GemvArgs args)
{
    constexpr uint32_t S = kGemvSlices, CH = kGemvChunk;
    __shared__ int32_t sRed[(S - 1) * G * kGemvWarpRows * (MR + 1)];
    const uint32_t tid = threadIdx.x, ks = tid >> 5, lane = tid & 31u;
    const uint32_t rr = lane >> 2;                                 // row inside the group
    const uint32_t pos = lane & 3u;                                // physical 16-byte segment
    const uint32_t seg = pos ^ ((rr >> 1) & 3u);                   // logical segment (k = 32*seg .. 32*seg+31); groups start at multiples of 8 rows
    const uint32_t KB = (args.k + 127) / 128;
    const uint32_t T = KB > ks ? (KB - ks + S - 1) / S : 0;        // K blocks of this warp: ks, ks+S, ...
    const uint32_t groups = (args.n + kGemvWarpRows - 1) / kGemvWarpRows;
    const uint32_t sgroups = (groups + G - 1) / G;                 // sets of G groups: the unit a CTA takes

    gemv_stamp(args, 0);
    if (args.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    constexpr size_t kWStep = (size_t)S * kI4CxBlockBytes;
    const uint8_t *wp[G], *rp[G];   // this thread's weight segment / int16 partial row sum in its first K block
    bool gok[G];                    // the group exists (the last set of a launch may be short)
    auto set_group = [&](uint32_t sg) {
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            const uint32_t grp = sg * G + gi;
            gok[gi] = grp < groups;
            const uint32_t row0 = (gok[gi] ? grp : 0u) * kGemvWarpRows, tile = row0 >> 7, r_blk = (row0 & 127u) + rr;
            const uint8_t *blk = args.B + ((size_t)tile * args.b_kblocks_total + ks) * kI4CxBlockBytes;
            wp[gi] = blk + r_blk * 64u + pos * 16u;
            rp[gi] = blk + kI4NibBytes + r_blk * 2u;   // tail of every packed block: the zero-point correction terms
        }
    };
    uint4 w[G][CH];
    int32_t rsv[G][CH];
    auto load_chunk = [&](uint32_t t0) {   // K blocks t0 .. t0 + CH - 1 of this warp
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
#pragma unroll
            for (uint32_t i = 0; i < CH; ++i) {
                const bool ok = gok[gi] && t0 + i < T;
                w[gi][i] = ok ? ldg_stream(wp[gi] + (size_t)(t0 + i) * kWStep) : make_uint4(0, 0, 0, 0);
                rsv[gi][i] = (ok && pos == 0) ? (int32_t)__ldg(reinterpret_cast<const int16_t *>(rp[gi] + (size_t)(t0 + i) * kWStep)) : 0;
            }
        }
    };
    uint32_t sg = blockIdx.x;
    set_group(sg);
    load_chunk(0);
    // per-column constants of the first set: static like the weights, so fetched before the wait
    const bool finisher = ks == 0 && pos == 0;
    float sb[G], bv[G];
    auto load_column_constants = [&](uint32_t sg_) {
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            const uint32_t n = (sg_ * G + gi) * kGemvWarpRows + rr;
            sb[gi] = 0.0f;
            bv[gi] = 0.0f;
            if (finisher && n < args.n) {
                sb[gi] = args.scale_b[n];
                bv[gi] = args.bias ? TdTraits<TD>::load(args.bias, n) : 0.0f;
            }
        }
    };
    load_column_constants(sg);
    gemv_stamp(args, 1);
    // everything else may have been produced by the preceding kernel
    if (args.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    gemv_stamp(args, 2);

    float sa[MR];
    int32_t zp[MR];
#pragma unroll
    for (int mi = 0; mi < MR; ++mi) {
        const bool ok = finisher && (uint32_t)mi < args.m;
        sa[mi] = ok ? args.scale_a[mi] : 0.0f;
        zp[mi] = ok ? args.zp_a[mi] : 0;
    }

    // activation words of row mi for this thread's segment: 16-byte chunks 2*seg and 2*seg+1 of the swizzled row
    const uint8_t *ap = args.A + (size_t)ks * kI8BlockBytes;
    constexpr size_t kAStep = (size_t)S * kI8BlockBytes;

    while (true) {
        int32_t acc[G][MR];
        int32_t rsum[G];   // sum of q over this row's K blocks of this warp (lanes with pos == 0)
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            rsum[gi] = 0;
#pragma unroll
            for (int i = 0; i < MR; ++i) acc[gi][i] = 0;
        }

        for (uint32_t t0 = 0; t0 < T; t0 += CH) {
#pragma unroll
            for (int mi = 0; mi < MR; ++mi) {
                if (MR == 1 || (uint32_t)mi < args.m) {
                    // all activation words of the chunk are requested together: one L1/L2 latency, not CH
                    uint4 av[CH][2];
#pragma unroll
                    for (uint32_t i = 0; i < CH; ++i) {
                        const uint8_t *act = ap + (size_t)(t0 + i) * kAStep;
                        const bool ok = t0 + i < T;
                        av[i][0] = ok ? __ldg(reinterpret_cast<const uint4 *>(act + sw128_byte((uint32_t)mi, seg * 32u)))
                                      : make_uint4(0, 0, 0, 0);
                        av[i][1] = ok ? __ldg(reinterpret_cast<const uint4 *>(act + sw128_byte((uint32_t)mi, seg * 32u + 16u)))
                                      : make_uint4(0, 0, 0, 0);
                    }
#pragma unroll
                    for (uint32_t i = 0; i < CH; ++i) {
                        const uint32_t al[4] = {av[i][0].x, av[i][0].y, av[i][0].z, av[i][0].w};
                        const uint32_t ah[4] = {av[i][1].x, av[i][1].y, av[i][1].z, av[i][1].w};
#pragma unroll
                        for (int gi = 0; gi < G; ++gi) {
                            const uint32_t ws[4] = {w[gi][i].x, w[gi][i].y, w[gi][i].z, w[gi][i].w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const uint32_t lo = (ws[j] << 4) & 0xF0F0F0F0u;   // 16*q for k = 32*seg + 4j .. +3
                                const uint32_t hi = ws[j] & 0xF0F0F0F0u;          // 16*q for k = 32*seg + 16 + 4j .. +3
                                acc[gi][mi] = __dp4a((int)al[j], (int)lo, acc[gi][mi]);
                                acc[gi][mi] = __dp4a((int)ah[j], (int)hi, acc[gi][mi]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
#pragma unroll
                for (uint32_t i = 0; i < CH; ++i) rsum[gi] += rsv[gi][i];   // slots past T hold 0
            }
            if (t0 + CH < T) load_chunk(t0 + CH);
        }

        gemv_stamp(args, 3);
        // request the next set's first chunk before combining this one: the registers are free
        const uint32_t cur = sg;
        const uint32_t next = sg + gridDim.x;
        if (next < sgroups) {
            set_group(next);
            load_chunk(0);
        }

        // combine the four segments of each row (lanes that differ in their low two bits) ...
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
#pragma unroll
            for (int mi = 0; mi < MR; ++mi) {
                int32_t v = acc[gi][mi];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                acc[gi][mi] = v;
            }
        }
        // ... and the eight warps through shared memory
        if (ks > 0 && pos == 0) {
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                int32_t *dst = sRed + (((ks - 1) * G + gi) * kGemvWarpRows + rr) * (MR + 1);
#pragma unroll
                for (int mi = 0; mi < MR; ++mi) dst[mi] = acc[gi][mi];
                dst[MR] = rsum[gi];
            }
        }
        __syncthreads();
        gemv_stamp(args, 4);

        if (finisher) {
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                const uint32_t n = (cur * G + gi) * kGemvWarpRows + rr;
                if (n < args.n) {
#pragma unroll
                    for (uint32_t s2 = 1; s2 < S; ++s2) {
                        const int32_t *src = sRed + (((s2 - 1) * G + gi) * kGemvWarpRows + rr) * (MR + 1);
#pragma unroll
                        for (int mi = 0; mi < MR; ++mi) acc[gi][mi] += src[mi];
                        rsum[gi] += src[MR];
                    }
#pragma unroll
                    for (int mi = 0; mi < MR; ++mi) {
                        if ((uint32_t)mi < args.m) {
                            int32_t a = acc[gi][mi] >> 4;   // operands were 16*q
                            a -= zp[mi] * rsum[gi];
                            const float cv = args.C ? TdTraits<TD>::load(args.C, (size_t)mi * args.ldc + n) : 0.0f;
                            const float v = w4a8_epilogue(a, sa[mi], sb[gi], args.C != nullptr, cv, args.bias != nullptr, bv[gi],
                                                          args.cmin, args.cmax);
                            TdTraits<TD>::store(args.D, (size_t)mi * args.ldd + n, v);
                        }
                    }
                }
            }
        }
        gemv_stamp(args, 5);
        if (next >= sgroups) break;
        sg = next;
        load_column_constants(sg);
        __syncthreads();   // the partial sums in shared memory have been read
    }
}

// ======================================================================================================
// GEMV for 2 <= m <= 16 on mma.sync (m16n8k32, s8 x s8 -> s32), weights streamed through registers.
// The tensor cores here are a convenience, not a throughput need: the 16-row A fragment is exactly a decode
// batch, so one kernel serves every m <= 16 at nearly the cost of m = 2.
//
// A CTA owns a set of 8 G consecutive output columns (G = 1 or 2 groups of 8); warp w takes K blocks w, w+8, ...
// Lane (g, t) = (lane / 4, lane % 4) streams, per group and K block, the 16 bytes of weight row g that hold
// logical segment t (physical position t ^ ((g >> 1) & 3): a warp-wide load still covers 512 contiguous
// bytes), and supplies, for MMA step j, b0 = 16 q[col g][32 t + 4 j ..] and b1 = 16 q[col g][32 t + 16 + 4 j ..]
// (the two masks of word j).  The A fragment takes words j of activation chunks 2t / 2t+1 of rows g / g+8, loaded
// straight from the packed activation rows after the wait for the predecessor: any consistent permutation of k is a
// valid contraction order, and integer sums are exact.  The column sums of the weights (the zero-point correction)
// are accumulated from the same words with dp4a against ones, so the row-sum tails of the packed blocks are not
// read.  The eight warps are combined through shared memory; warp 0 runs the epilogue (reference:
// src/gemm/gemm_i8_i4/gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp/..._4x1vl_rvv.cpp:118-177).  No mbarrier, no scratch
// memory, no staging of weights or activations in shared memory (both were slower in a chain of GEMVs).
//
// All weight loads of a CTA's first set are requested before griddepcontrol.wait.
// ======================================================================================================
constexpr uint32_t kGvRedInts = 5u * 32u;   // per warp and group: [acc0..3, column sum][lane]

__device__ __forceinline__ void mma_s8_16832(int32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int G>
constexpr int gemv_mma_min_ctas() { return 2; }

// Static shared memory: [7 warps][G][reduce].
// R16: the launch has more than 8 activation rows (fragment rows g + 8 exist); their fragments are then fetched
// two K blocks at a time to stay inside the register budget.
template <int G, bool R16, Dtype TD>
__global__ void __launch_bounds__(kGemvThreads, gemv_mma_min_ctas<G>()) gemv_mma_kernel(const GemvArgs args)
{
    constexpr uint32_t S = kGemvSlices, CH = kGemvChunk;
    __shared__ int32_t sRed[(S - 1) * G * kGvRedInts];
    const uint32_t tid = threadIdx.x, ks = tid >> 5, lane = tid & 31u;
    const uint32_t g = lane >> 2, t4 = lane & 3u;
    const uint32_t KB = (args.k + 127) / 128;
    const uint32_t T = KB > ks ? (KB - ks + S - 1) / S : 0;        // K blocks of this warp: ks, ks+S, ...
    const uint32_t groups = (args.n + kGemvWarpRows - 1) / kGemvWarpRows;
    const uint32_t sets = (groups + G - 1) / G;

    if (args.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    constexpr size_t kWStep = (size_t)S * kI4CxBlockBytes;
    const uint32_t wpos = (t4 ^ ((g >> 1) & 3u)) * 16u;   // physical position of logical segment t4 in weight row g
    const uint8_t *wp[G];
    bool gok[G];
    auto set_group = [&](uint32_t sg) {
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            const uint32_t grp = sg * G + gi;
            gok[gi] = grp < groups;
            const uint32_t row0 = (gok[gi] ? grp : 0u) * kGemvWarpRows, tile = row0 >> 7, r_blk = (row0 & 127u) + g;
            wp[gi] = args.B + ((size_t)tile * args.b_kblocks_total + ks) * kI4CxBlockBytes + r_blk * 64u + wpos;
        }
    };
    uint4 w[G][CH];
    auto load_chunk = [&](uint32_t t0) {   // K blocks t0 .. t0 + CH - 1 of this warp
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
#pragma unroll
            for (uint32_t i = 0; i < CH; ++i) {
                const bool ok = gok[gi] && t0 + i < T;
                w[gi][i] = ok ? ldg_stream(wp[gi] + (size_t)(t0 + i) * kWStep) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    uint32_t sg = blockIdx.x;
    set_group(sg);
    load_chunk(0);
    // per-column constants (warp 0 only): requested together with the activations, one round trip for all
    float sb[G][2], bv[G][2];
    auto load_column_constants = [&](uint32_t sg_) {
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint32_t n = (sg_ * G + gi) * kGemvWarpRows + 2u * t4 + c;
                sb[gi][c] = 0.0f;
                bv[gi][c] = 0.0f;
                if (ks == 0 && n < args.n) {
                    sb[gi][c] = args.scale_b[n];
                    bv[gi][c] = args.bias ? TdTraits<TD>::load(args.bias, n) : 0.0f;
                }
            }
        }
    };
    // everything else may have been produced by the preceding kernel
    if (args.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    load_column_constants(sg);

    float sa[2] = {0.0f, 0.0f};
    int32_t zp[2] = {0, 0};
    if (ks == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t row = g + 8u * h;
            if (row < args.m) {
                sa[h] = args.scale_a[row];
                zp[h] = args.zp_a[row];
            }
        }
    }
    const bool row_lo = g < args.m, row_hi = R16 && g + 8u < args.m;   // this lane's fragment rows exist
    const uint32_t a_lo_off = g * 128u + (((2u * t4) ^ g) << 4), a_hi_off = g * 128u + (((2u * t4 + 1u) ^ g) << 4);

    while (true) {
        int32_t acc[G][4], rs[G];   // rs: 16 * sum of q over this lane's words of weight row g
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
            rs[gi] = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[gi][e] = 0;
        }
        for (uint32_t t0 = 0; t0 < T; t0 += CH) {
            // activation fragments, straight from the packed blocks (L2): logical chunks 2 t4 and 2 t4 + 1 of rows g
            // and g + 8 ((g + 8) & 7 = g: same swizzle); a batch is requested whole before its first use
            constexpr uint32_t BA = R16 ? 2u : CH;   // K blocks per batch of fragments
#pragma unroll
            for (uint32_t i0 = 0; i0 < CH; i0 += BA) {
                uint4 fa[BA][2], fb[R16 ? BA : 1][2];
#pragma unroll
                for (uint32_t u = 0; u < BA; ++u) {
                    const uint8_t *ab = args.A + (size_t)(ks + (t0 + i0 + u) * S) * kI8BlockBytes;
                    const bool in = t0 + i0 + u < T;
                    fa[u][0] = (in && row_lo) ? __ldg(reinterpret_cast<const uint4 *>(ab + a_lo_off)) : make_uint4(0, 0, 0, 0);
                    fa[u][1] = (in && row_lo) ? __ldg(reinterpret_cast<const uint4 *>(ab + a_hi_off)) : make_uint4(0, 0, 0, 0);
                    if constexpr (R16) {
                        fb[u][0] = (in && row_hi) ? __ldg(reinterpret_cast<const uint4 *>(ab + 1024u + a_lo_off)) : make_uint4(0, 0, 0, 0);
                        fb[u][1] = (in && row_hi) ? __ldg(reinterpret_cast<const uint4 *>(ab + 1024u + a_hi_off)) : make_uint4(0, 0, 0, 0);
                    }
                }
#pragma unroll
                for (uint32_t u = 0; u < BA; ++u) {
                    const uint32_t i = i0 + u;
                    const uint32_t a0[4] = {fa[u][0].x, fa[u][0].y, fa[u][0].z, fa[u][0].w};
                    const uint32_t a2[4] = {fa[u][1].x, fa[u][1].y, fa[u][1].z, fa[u][1].w};
                    uint32_t a1[4] = {0u, 0u, 0u, 0u}, a3[4] = {0u, 0u, 0u, 0u};
                    if constexpr (R16) {
                        a1[0] = fb[u][0].x; a1[1] = fb[u][0].y; a1[2] = fb[u][0].z; a1[3] = fb[u][0].w;
                        a3[0] = fb[u][1].x; a3[1] = fb[u][1].y; a3[2] = fb[u][1].z; a3[3] = fb[u][1].w;
                    }
#pragma unroll
                    for (int gi = 0; gi < G; ++gi) {
                        const uint32_t ws[4] = {w[gi][i].x, w[gi][i].y, w[gi][i].z, w[gi][i].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint32_t b0 = (ws[j] << 4) & 0xF0F0F0F0u;   // 16*q, k = 32 t4 + 4 j .. + 3
                            const uint32_t b1 = ws[j] & 0xF0F0F0F0u;          // 16*q, k = 32 t4 + 16 + 4 j .. + 3
                            mma_s8_16832(acc[gi], a0[j], a1[j], a2[j], a3[j], b0, b1);
                            rs[gi] = __dp4a((int)b0, 0x01010101, rs[gi]);
                            rs[gi] = __dp4a((int)b1, 0x01010101, rs[gi]);
                        }
                    }
                }
            }
            if (t0 + CH < T) load_chunk(t0 + CH);
        }

        // request the next set's first chunk before combining this one: the registers are free
        const uint32_t cur = sg, next = sg + gridDim.x;
        if (next < sets) {
            set_group(next);
            load_chunk(0);
        }

        // the four lanes of a weight row hold its four segments: after this every lane (g, *) has the sum of row g
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {

            rs[gi] += __shfl_xor_sync(0xffffffffu, rs[gi], 1);
            rs[gi] += __shfl_xor_sync(0xffffffffu, rs[gi], 2);
        }
        // combine the eight warps through shared memory
        if (ks > 0) {
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
                int32_t *dst = sRed + ((ks - 1) * G + gi) * kGvRedInts + lane;
#pragma unroll
                for (int e = 0; e < 4; ++e) dst[e * 32] = acc[gi][e];
                dst[4 * 32] = rs[gi];
            }
        }
        __syncthreads();
        if (ks == 0) {
#pragma unroll
            for (int gi = 0; gi < G; ++gi) {
#pragma unroll
                for (uint32_t s2 = 1; s2 < S; ++s2) {
                    const int32_t *src = sRed + ((s2 - 1) * G + gi) * kGvRedInts + lane;
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[gi][e] += src[e * 32];
                    rs[gi] += src[4 * 32];
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    // this lane's accumulator columns are 2 t4 + c; the sum of weight row r sits in lanes 4 r .. 4 r + 3
                    const int32_t rsum = __shfl_sync(0xffffffffu, rs[gi], (int)((2u * t4 + c) * 4u)) >> 4;
                    const uint32_t n = (cur * G + gi) * kGemvWarpRows + 2u * t4 + c;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t row = g + 8u * h;
                        if (row < args.m && n < args.n) {
                            int32_t a = acc[gi][2 * h + c] >> 4;   // operands were 16*q
                            a -= zp[h] * rsum;
                            const float cv = args.C ? TdTraits<TD>::load(args.C, (size_t)row * args.ldc + n) : 0.0f;
                            const float v = w4a8_epilogue(a, sa[h], sb[gi][c], args.C != nullptr, cv, args.bias != nullptr,
                                                          bv[gi][c], args.cmin, args.cmax);
                            TdTraits<TD>::store(args.D, (size_t)row * args.ldd + n, v);
                        }
                    }
                }
            }
        }
        if (next >= sets) break;
        sg = next;
        load_column_constants(sg);
        __syncthreads();   // the partial sums in shared memory have been read
    }
}

bool pdl_enabled()
{
    static int cached = -1;
    if (cached < 0) {
        const char *e = std::getenv("TQT_B200_PDL");
        cached = (e && e[0] == '0') ? 0 : 1;
    }
    return cached != 0;
}

// TQT_B200_GEMV_G=1|2 forces the number of column groups per CTA (read once); by default two for launches
// that fit the GPU in one round at two CTAs per SM (decode-sized N), one otherwise.
static int gemv_forced_groups()
{
    static const int cached = [] {
        const char *e = std::getenv("TQT_B200_GEMV_G");
        return e ? std::atoi(e) : 0;
    }();
    return cached;
}

template <int MR, int G, Dtype TD>
static Result launch_gemv_t(GemvArgs a, cudaStream_t st)
{
    a.pdl = pdl_enabled() ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    // CTA c owns the sets of G 8-column groups c, c + grid, ...: one set each while they all fit on the GPU at once
    const uint32_t groups = (a.n + kGemvWarpRows - 1) / kGemvWarpRows;
    const uint32_t sgroups = (groups + G - 1) / G;
    const uint32_t resident = (uint32_t)sm_count_cached() * (uint32_t)gemv_min_ctas<MR, G>();
    cfg.gridDim = dim3(sgroups < resident ? sgroups : resident, 1, 1);
    cfg.blockDim = dim3(kGemvThreads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_w4a8_kernel<MR, G, TD>, a);
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

template <int MR, Dtype TD>
static Result launch_gemv_g(const GemvArgs &a, cudaStream_t st)
{
    // two column groups per CTA while the launch then still fits the GPU in one round (decode-sized N)
    const uint32_t groups = (a.n + kGemvWarpRows - 1) / kGemvWarpRows;
    const int forced = gemv_forced_groups();
    const bool two = forced ? forced == 2 : (groups + 1) / 2 <= (uint32_t)sm_count_cached() * 2u;
    if (two) return launch_gemv_t<MR, 2, TD>(a, st);
    return launch_gemv_t<MR, 1, TD>(a, st);
}

// TQT_B200_GEMV_KERNEL=regs|mma forces the dp4a kernel (one row only) or the mma.sync kernel (read once).
static int gemv_forced_kernel()
{
    static const int cached = [] {
        const char *e = std::getenv("TQT_B200_GEMV_KERNEL");
        if (!e) return 0;
        return e[0] == 'r' ? 1 : (e[0] == 'm' ? 2 : 0);
    }();
    return cached;
}

template <int G, bool R16, Dtype TD>
static Result launch_gemv_mma(GemvArgs a, cudaStream_t st)
{
    a.pdl = pdl_enabled() ? 1 : 0;
    const uint32_t groups = (a.n + kGemvWarpRows - 1) / kGemvWarpRows, sets = (groups + G - 1) / G;
    const uint32_t resident = (uint32_t)sm_count_cached() * (uint32_t)gemv_mma_min_ctas<G>();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sets < resident ? sets : resident, 1, 1);
    cfg.blockDim = dim3(kGemvThreads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_mma_kernel<G, R16, TD>, a);
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

template <Dtype TD>
static Result launch_gemv_m(const GemvArgs &a, cudaStream_t st)
{
    // one row: dp4a kernel; a decode batch: mma kernel (TQT_B200_GEMV_KERNEL=mma forces it for one row too)
    const int forced = gemv_forced_kernel(), fg = gemv_forced_groups();
    if (a.m == 1 && forced != 2) return launch_gemv_g<1, TD>(a, st);
    const bool one = fg == 1;
    if (a.m > 8) return one ? launch_gemv_mma<1, true, TD>(a, st) : launch_gemv_mma<2, true, TD>(a, st);
    return one ? launch_gemv_mma<1, false, TD>(a, st) : launch_gemv_mma<2, false, TD>(a, st);
}

Result gemv_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax)
{
    if (g.m == 0 || g.n == 0) return Result{kOk, 0};
    if (g.m > kGemvMaxRows || g.k == 0 || g.k > 65536 || g.n > 0x3fffff00ull) return Result{kUnsupported, 0};
    if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.B) & 15)) return Result{kUnsupported, 0};
    GemvArgs a{};
    a.m = (uint32_t)g.m;
    a.n = (uint32_t)g.n;
    a.k = (uint32_t)g.k;
    a.A = (const uint8_t *)g.A;
    a.B = (const uint8_t *)g.B;
    a.b_kblocks_total = (uint32_t)ceil_div(g.ldb, 128);
    a.C = g.C;
    a.ldc = g.ldc;
    a.D = g.D;
    a.ldd = g.ldd;
    a.bias = g.bias;
    a.scale_a = p.scale_a;
    a.zp_a = p.zp_a;
    a.scale_b = p.scale_b;
    a.cmin = cmin;
    a.cmax = cmax;
    a.dbg = timing_buffer();
    cudaStream_t st = (cudaStream_t)g.stream;
    switch (td) {
        case Dtype::F32: return launch_gemv_m<Dtype::F32>(a, st);
        case Dtype::F16: return launch_gemv_m<Dtype::F16>(a, st);
        default: return launch_gemv_m<Dtype::BF16>(a, st);
    }
}

// Diagnostic: the same launch shape as the GEMV (256 threads, four 128-bit streaming loads per thread
// in flight, programmatic dependent launch) with the arithmetic removed: what a kernel that only
// reads `bytes` can reach, the ceiling the GEMV is compared against at small sizes.
__global__ void __launch_bounds__(kGemvThreads, 4) stream_read_kernel(const uint4 *src, size_t n16, uint32_t *sink, int pdl)
{
    if (pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t acc = 0;
    bool waited = false;
    for (size_t base = (size_t)blockIdx.x * (kGemvChunk * kGemvThreads) + threadIdx.x; base < n16;
         base += (size_t)gridDim.x * (kGemvChunk * kGemvThreads)) {
        uint4 v[kGemvChunk];
#pragma unroll
        for (uint32_t i = 0; i < kGemvChunk; ++i)
            v[i] = (base + i * kGemvThreads < n16) ? ldg_stream(src + base + i * kGemvThreads) : make_uint4(0, 0, 0, 0);
        if (pdl && !waited) {   // as in the GEMV: first loads requested, then wait for the predecessor
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
        }
#pragma unroll
        for (uint32_t i = 0; i < kGemvChunk; ++i) acc ^= v[i].x ^ v[i].y ^ v[i].z ^ v[i].w;
    }
    if (pdl && !waited) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (acc == 0x9e3779b9u && sink) sink[threadIdx.x & 31u] = acc;   // keeps the loads alive; practically never taken
}

Result stream_read(const void *src, size_t bytes, void *sink, void *stream)
{
    if ((reinterpret_cast<uintptr_t>(src) & 15) || bytes < 16) return Result{kInvalid, 0};
    const size_t n16 = bytes / 16;
    const size_t per_cta = (size_t)kGemvChunk * kGemvThreads;
    const size_t want = (n16 + per_cta - 1) / per_cta, resident = (size_t)sm_count_cached() * 4;
    const int pdl = pdl_enabled() ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(want < resident ? want : resident), 1, 1);
    cfg.blockDim = dim3(kGemvThreads, 1, 1);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, stream_read_kernel, (const uint4 *)src, n16, (uint32_t *)sink, pdl);
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

}  // namespace tqt
