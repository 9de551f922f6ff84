// CTA-pair (cta_group::2) tensor-core GEMMs for sm_100a.
//
// Shared memory bandwidth (128 B/clk per SM), not the tensor pipe, bounds a single-CTA 8-bit GEMM:
// per 128-deep K step a 128x256 tile moves 48 KB of operands into shared memory and the MMA reads
// 48 KB back.  Two CTAs of a cluster that issue one tcgen05.mma.cta_group::2 each hold only half of
// the N-side operand, and the int4 weights can be expanded into TENSOR memory (the M-side operand
// of a "TS" MMA) instead of shared memory.  Two kernels:
//
//   gemm_pair_i8_kernel     int8 x int8: pair tile 256 (M) x 256 (N); per CTA and K step 16 KB of A
//                           and 16 KB of B through shared memory; s32 / requantised int8 epilogues.
//   gemm_pair_w4a8_kernel   W4A8 with the roles swapped: the M side of the MMA is the WEIGHT matrix
//                           (256 output channels per pair, 128 per CTA), expanded from int4 to int8
//                           (= 16*q) in registers and written to tensor memory with tcgen05.st; the
//                           N side is 192 activation rows (96 per CTA) straight from the packed LHS
//                           blocks.  The accumulator is D^T: lane = output channel, column = row of A,
//                           so scale_b / bias / row sums are per-thread constants in the epilogue.
//                           Tensor memory: 2 x 192 accumulator columns + 4 x 32 operand columns = 512;
//                           shared memory: 8 stages of (8448 B of nibbles + 12 KiB of activations).
//
// Protocol inside a pair (leader = cluster rank 0): every CTA loads its own operands with bulk copies
// on local mbarriers; readiness of the peer's operands reaches the leader through remote mbarrier
// arrives (a relay warp for int8, the converter warps for W4A8); the leader's MMA completion is
// broadcast to both CTAs' barriers with tcgen05.commit (an arrive broadcast, no data copy).  All
// waits are bounded; teardown is a hardware cluster barrier that every path reaches.
//
// Reference semantics of the epilogues: see kernels_umma.cu.
#include "epilogues.cuh"
#include "ptx_sm100.cuh"
#include "umma_args.cuh"

namespace tqt {

#define TQT_PTIMED(slot, call)                                  \
    ([&]() -> bool {                                            \
        if (!args.dbg) return (call);                           \
        const long long _t0 = clock64();                        \
        const bool _r = (call);                                 \
        wcyc[slot] += clock64() - _t0;                          \
        return _r;                                              \
    }())

// ======================================================================================================
// int8 x int8
// ======================================================================================================
constexpr uint32_t kI8Stages = 6;
constexpr uint32_t kI8Threads = 320;   // warp 0 producer, warp 1 MMA / relay, warps 2..9 epilogue
constexpr uint32_t kI8Smem = 1024 + kI8Stages * 32768 + 8 * 3 * 128 * 4 + 256;

template <EpiKind EK>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kI8Threads, 1) gemm_pair_i8_kernel(const UmmaArgs args)
{
    using OutT = typename OutType<EK, Dtype::F32>::type;
    constexpr uint32_t S = kI8Stages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sA = smem;                         // S x 16 KiB: this CTA's 128 rows of A
    uint8_t *sB = sA + S * 16384;               // S x 16 KiB: this CTA's half of the N-side operand
    int32_t *sColAll = reinterpret_cast<int32_t *>(sB + S * 16384);   // [8 warps][3][128]
    uint64_t *bars = reinterpret_cast<uint64_t *>(sColAll + 8 * 3 * 128);
    constexpr uint32_t kFull = 0, kPeerFull = S, kEmpty = 2 * S, kTmemFull = 3 * S, kTmemEmpty = 3 * S + 2;
    uint32_t *sTmemBase = reinterpret_cast<uint32_t *>(bars + 3 * S + 4);
    volatile int *sAbort = reinterpret_cast<volatile int *>(sTmemBase + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto BAR = [&](uint32_t idx) { return bar0 + idx * 8u; };

    const uint32_t tiles_m = (args.m + 127) / 128, pmc = (tiles_m + 1) / 2;
    const uint32_t nblocks = (args.n + 127) / 128, tnc = (nblocks + 1) / 2;
    const uint32_t num_tiles = pmc * tnc;
    const uint32_t KB = (args.k + 127) / 128;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            ptx::mbar_init(BAR(kFull + s), 1);
            ptx::mbar_init(BAR(kPeerFull + s), 1);
            ptx::mbar_init(BAR(kEmpty + s), 1);
        }
        for (uint32_t e = 0; e < 2; ++e) {
            ptx::mbar_init(BAR(kTmemFull + e), 1);
            ptx::mbar_init(BAR(kTmemEmpty + e), 16);   // 8 epilogue warps of each CTA
        }
        *sAbort = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(sTmemBase), 512);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();   // the peer's barriers exist before anything arrives on them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *sTmemBase;
    long long wcyc[3] = {0, 0, 0};
    const long long t_role0 = args.dbg ? clock64() : 0;

    if (warp == 0) {
        // ===================== producer (both CTAs) =====================
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t t = pair; t < num_tiles && ok; t += npairs) {
            const uint32_t pm = t % pmc, tn = t / pmc;
            const uint32_t nblk = min(2u, nblocks - tn * 2);
            const uint32_t mtile = pm * 2 + rank;
            const bool a_valid = mtile < tiles_m;
            const uint32_t b_bytes = nblk == 2 ? 16384u : 8192u;
            const uint8_t *a_src = args.A + (size_t)mtile * args.a_kblocks_total * kI8BlockBytes;
            const uint8_t *b_src = nblk == 2 ? args.B + (size_t)(tn * 2 + rank) * args.b_kblocks_total * kI8BlockBytes
                                             : args.B + (size_t)(tn * 2) * args.b_kblocks_total * kI8BlockBytes + rank * 8192u;
            for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                const uint32_t s = it % S, ph = (it / S) & 1u;
                if (!TQT_PTIMED(0, ptx::mbar_wait_cluster(BAR(kEmpty + s), ph ^ 1u, sAbort, args.fault, kFaultProducerWait))) {
                    ok = false;
                    break;
                }
                if (lane == 0) ptx::mbar_arrive_expect_tx(BAR(kFull + s), (a_valid ? 16384u : 0u) + b_bytes);
                __syncwarp();
                // two lanes issue one bulk copy each in the same instruction
                if (lane == 0) {
                    ptx::bulk_g2s(ptx::smem_u32(sB + s * 16384), b_src + (size_t)kb * kI8BlockBytes, b_bytes, BAR(kFull + s));
                } else if (lane == 1 && a_valid) {
                    ptx::bulk_g2s(ptx::smem_u32(sA + s * 16384), a_src + (size_t)kb * kI8BlockBytes, 16384u, BAR(kFull + s));
                }
                __syncwarp();
            }
        }
        if (!ok) {
            const uint32_t pending = it < S ? it : S;
            for (uint32_t i = 0; i < pending; ++i) {
                const uint32_t j = it - 1 - i;
                const uint32_t s = j % S, ph = (j / S) & 1u;
                const long long t0 = clock64();
                while (!ptx::mbar_try_wait(BAR(kFull + s), ph)) {
                    if (clock64() - t0 > ptx::kWaitLimitCycles) {
                        if (args.fault) atomicCAS(args.fault, 0u, (unsigned)kFaultDrainWait);
                        break;
                    }
                }
            }
        }
    } else if (warp == 1 && rank == 0) {
        // ===================== MMA issuer (leader CTA) =====================
        const uint32_t idesc256 = ptx::make_idesc(2u, 1u, 1u, 256, 256);
        const uint32_t idesc128 = ptx::make_idesc(2u, 1u, 1u, 256, 128);
        uint32_t it = 0, ti = 0;
        bool ok = true;
        for (uint32_t t = pair; t < num_tiles && ok; t += npairs, ++ti) {
            const uint32_t tn = t / pmc;
            const uint32_t nblk = min(2u, nblocks - tn * 2);
            const uint32_t idesc = nblk == 2 ? idesc256 : idesc128;
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            if (!TQT_PTIMED(0, ptx::mbar_wait_cluster(BAR(kTmemEmpty + acc), pha ^ 1u, sAbort, args.fault, kFaultMmaWaitTmem))) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * 256u;
            for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                const uint32_t s = it % S, ph = (it / S) & 1u;
                if (!TQT_PTIMED(1, ptx::mbar_wait(BAR(kFull + s), ph, sAbort, args.fault, kFaultMmaWaitFull, true)) ||
                    !TQT_PTIMED(2, ptx::mbar_wait_cluster(BAR(kPeerFull + s), ph, sAbort, args.fault, kFaultMmaWaitFull, true))) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                if (lane == 0) {
                    const uint64_t a_desc = ptx::make_desc_k_sw128(ptx::smem_u32(sA + s * 16384));
                    const uint64_t b_desc = ptx::make_desc_k_sw128(ptx::smem_u32(sB + s * 16384));
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j)
                        ptx::mma_i8_ss_pair(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc, (kb | j) ? 1u : 0u);
                    ptx::tc_commit_pair(BAR(kEmpty + s), 3);
                    if (kb == KB - 1) ptx::tc_commit_pair(BAR(kTmemFull + acc), 3);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ===================== relay (peer CTA): tells the leader that this CTA's stage has landed =====
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t t = pair; t < num_tiles && ok; t += npairs) {
            for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                const uint32_t s = it % S, ph = (it / S) & 1u;
                if (!TQT_PTIMED(1, ptx::mbar_wait(BAR(kFull + s), ph, sAbort, args.fault, kFaultMmaWaitFull, true))) {
                    ok = false;
                    break;
                }
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(BAR(kPeerFull + s), 0));
                __syncwarp();
            }
        }
    } else {
        // ===================== epilogue (8 warps per CTA) =====================
        const uint32_t quad = warp & 3u, half = (warp - 2u) >> 2;   // TMEM lane quadrant, column half
        int32_t *sCol = sColAll + (warp - 2u) * 384u;
        uint32_t ti = 0;
        bool ok = true;
        for (uint32_t t = pair; t < num_tiles && ok; t += npairs, ++ti) {
            const uint32_t pm = t % pmc, tn = t / pmc;
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            const uint32_t n0 = tn * 256u + half * 128u;
            const uint32_t ncols = args.n > n0 ? min(128u, args.n - n0) : 0u;
            const size_t mrow = (size_t)(pm * 2 + rank) * 128u + quad * 32u + lane;
            const bool row_ok = mrow < args.m;
            __syncwarp();
            if constexpr (EK == EpiKind::Req8) {
                for (uint32_t c = lane; c < 128u; c += 32u) {
                    const bool cok = c < ncols;
                    int32_t mult = 0, rsh = 0;
                    if (cok) requant_column(args.rq_scale_a, args.scale_b[args.rq_per_tensor ? 0 : n0 + c], args.rq_scale_d, &mult, &rsh);
                    sCol[c] = mult;
                    sCol[128 + c] = rsh;
                    sCol[256 + c] = (cok && args.bias) ? static_cast<const int32_t *>(args.bias)[n0 + c] : 0;
                }
            }
            __syncwarp();
            if (!TQT_PTIMED(0, ptx::mbar_wait_cluster(BAR(kTmemFull + acc), pha, sAbort, args.fault, kFaultEpilogueWait))) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            const uint32_t t_addr = tmem_base + acc * 256u + half * 128u + ((quad * 32u) << 16);
            const uint32_t nchunks = (ncols + 31u) / 32u;
            for (uint32_t ch = 0; ch < nchunks; ++ch) {
                uint32_t r[32];
                __syncwarp();
                const long long tl0 = args.dbg ? clock64() : 0;
                ptx::tmem_ld_32x32b_x32(t_addr + ch * 32u, r);
                ptx::tmem_wait_ld();
                if (args.dbg) wcyc[2] += clock64() - tl0;
                if (row_ok) {
                    const uint32_t c0 = ch * 32u;
                    const uint32_t nvalid = min(32u, ncols - c0);
                    alignas(16) OutT out[32];
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) {
                        const uint32_t c = c0 + j;
                        if constexpr (EK == EpiKind::S32) {
                            int32_t v = (int32_t)r[j];
                            if (args.C && j < nvalid)
                                v = (int32_t)((uint32_t)v + (uint32_t) static_cast<const int32_t *>(args.C)[mrow * args.ldc + n0 + c]);
                            out[j] = max(args.cmin_i, min(args.cmax_i, v));
                        } else {
                            uint32_t u = r[j];
                            if (args.C && j < nvalid) u += (uint32_t) static_cast<const int32_t *>(args.C)[mrow * args.ldc + n0 + c];
                            u += (uint32_t)sCol[256 + c];
                            out[j] = (int8_t)requant_value((int32_t)u, sCol[c], sCol[128 + c], args.rq_zp_d, args.cmin_i, args.cmax_i);
                        }
                    }
                    OutT *dst = static_cast<OutT *>(args.D) + mrow * args.ldd + n0 + c0;
                    if (args.vec_store && nvalid == 32u) {
                        constexpr uint32_t nvec = 32u * sizeof(OutT) / 16u;
#pragma unroll
                        for (uint32_t v = 0; v < nvec; ++v) reinterpret_cast<uint4 *>(dst)[v] = reinterpret_cast<const uint4 *>(out)[v];
                    } else {
#pragma unroll
                        for (uint32_t j = 0; j < 32; ++j)
                            if (j < nvalid) dst[j] = out[j];
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0)
                    ptx::mbar_arrive(BAR(kTmemEmpty + acc));
                else
                    ptx::mbar_arrive_cluster(ptx::mapa(BAR(kTmemEmpty + acc), 0));
            }
        }
    }

    if (args.dbg && lane == 0 && (warp == 0 || warp == 1 || warp == 2)) {
        long long *d = args.dbg + (size_t)blockIdx.x * 16 + (warp == 0 ? 0 : warp == 1 ? 4 : 8);
        d[0] = wcyc[0];
        d[1] = wcyc[1];
        d[2] = wcyc[2];
        d[3] = clock64() - t_role0;
    }
    // ---- teardown: both CTAs arrive, then tensor memory is released ----
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, 512);
    }
}

// ======================================================================================================
// W4A8, weights through tensor memory
// ======================================================================================================
constexpr uint32_t kW4Stages = 8;          // shared-memory stages (bulk copies run this far ahead)
constexpr uint32_t kW4StagesSingle = 6;    // single-CTA variant: 24 KiB of activations per stage
constexpr uint32_t kW4TStages = 4;         // tensor-memory operand stages (4 x 32 columns)
constexpr uint32_t kW4MT = 192;            // activation rows per pair tile (MMA N), 96 per CTA
constexpr uint32_t kW4Threads = 576;       // warp 0 producer, 1 MMA, 2..9 epilogue, 10..17 converters
constexpr uint32_t kW4NibBytes = 8448, kW4ActBytes = 96 * 128;
// (padded to more than half of an SM's shared memory: one CTA per SM, each owns all 512 TMEM columns)
constexpr uint32_t kW4SmemUsed = 1024 + kW4Stages * (kW4ActBytes + kW4NibBytes) + 8 * 2 * 96 * 4 + 2 * 2 * 128 * 4 + 512;
constexpr uint32_t kW4Smem = kW4SmemUsed > 120 * 1024 ? kW4SmemUsed : 120 * 1024;
constexpr uint32_t kW4SmemSingle = 1024 + kW4StagesSingle * (192 * 128 + kW4NibBytes) + 8 * 2 * 96 * 4 + 2 * 2 * 128 * 4 + 512;

template <Dtype TD, bool PAIR>
__device__ __forceinline__ void w4a8_ts_body(const UmmaArgs &args)
{
    using OutT = typename TdTraits<TD>::type;
    constexpr uint32_t S = PAIR ? kW4Stages : kW4StagesSingle;
    constexpr uint32_t kActRows = PAIR ? 96u : 192u;        // activation rows this CTA stages per K step
    constexpr uint32_t kActBytes = kActRows * 128u;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sAct = smem;                              // S x 12 (pair) or 24 KiB; both multiples of 1024
    uint8_t *sNib = sAct + S * kActBytes;            // S x 8448 B
    float *sRowAll = reinterpret_cast<float *>(sNib + S * kW4NibBytes);   // [8 warps][scale_a 96 | zp_a 96]
    int32_t *sRsum = reinterpret_cast<int32_t *>(sRowAll + 8 * 192);      // [2 accumulators][2 converter sets][128]
    uint64_t *bars = reinterpret_cast<uint64_t *>(sRsum + 512);
    constexpr uint32_t T = kW4TStages;
    // K steps are committed in groups of two (it >> 1): tcgen05.commit after MMAs that take their M-side
    // operand from tensor memory costs a pipeline drain, so one commit per group releases two
    // shared-memory stages and two tensor-memory operand stages together.
    constexpr uint32_t NG = S / 2;   // shared-memory stage groups; the tensor-memory stages form T / 2 = 2 groups
    constexpr uint32_t kFull = 0, kGroupDone = S, kConvFull = 2 * S, kTmemFull = 2 * S + 2 * T,
                       kTmemEmpty = kTmemFull + 2, kRsumFull = kTmemFull + 4, kRsumEmpty = kTmemFull + 6;
    uint32_t *sTmemBase = reinterpret_cast<uint32_t *>(bars + kTmemFull + 8);
    volatile int *sAbort = reinterpret_cast<volatile int *>(sTmemBase + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;
    const uint32_t pair = PAIR ? blockIdx.x >> 1 : blockIdx.x, npairs = PAIR ? gridDim.x >> 1 : gridDim.x;
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto BAR = [&](uint32_t idx) { return bar0 + idx * 8u; };

    const uint32_t tiles_m128 = (args.m + 127) / 128;          // 128-row blocks that exist in A_packed
    const uint32_t tmc = (args.m + kW4MT - 1) / kW4MT;         // 192-row tiles of the activations
    const uint32_t nblocks = (args.n + 127) / 128, tnc = PAIR ? (nblocks + 1) / 2 : nblocks;
    const uint32_t num_tiles = tmc * tnc;
    const uint32_t KB = (args.k + 127) / 128;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) ptx::mbar_init(BAR(kFull + s), 1);
        for (uint32_t g = 0; g < NG; ++g) ptx::mbar_init(BAR(kGroupDone + g), 1);
        for (uint32_t s = 0; s < T; ++s) ptx::mbar_init(BAR(kConvFull + s), PAIR ? 8 : 4);   // 4 converter warps per CTA
        for (uint32_t e = 0; e < 2; ++e) {
            ptx::mbar_init(BAR(kTmemFull + e), 1);
            ptx::mbar_init(BAR(kTmemEmpty + e), PAIR ? 16 : 8);
            ptx::mbar_init(BAR(kRsumFull + e), 8);   // 8 converter warps
            ptx::mbar_init(BAR(kRsumEmpty + e), 8);
        }
        *sAbort = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        if constexpr (PAIR) {
            ptx::tmem_alloc_pair(ptx::smem_u32(sTmemBase), 512);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(ptx::smem_u32(sTmemBase), 512);
            ptx::tmem_relinquish();
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) ptx::cluster_sync_all();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *sTmemBase;
    const uint32_t tmem_a = tmem_base + 2 * kW4MT;   // operand stages after the two accumulators
    long long wcyc[3] = {0, 0, 0};
    const long long t_role0 = args.dbg ? clock64() : 0;

    if (warp == 0) {
        // ===================== producer (both CTAs) =====================
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t t = pair; t < num_tiles && ok; t += npairs) {
            const uint32_t tm = t % tmc, tn = t / tmc;
            const uint32_t nb = PAIR ? tn * 2 + rank : tn;
            const bool nib_valid = nb < nblocks;
            const uint8_t *nib_src = args.B + (size_t)nb * args.b_kblocks_total * kI4CxBlockBytes;
            // this CTA's activation rows [a0, a0 + kActRows) = at most two pieces of 128-row blocks
            const uint32_t a0 = tm * kW4MT + rank * 96u;
            const uint32_t blk1 = a0 >> 7, off1 = a0 & 127u;
            const uint32_t rows1 = min(kActRows, 128u - off1), rows2 = kActRows - rows1;
            const bool v1 = blk1 < tiles_m128, v2 = rows2 > 0 && (blk1 + 1) < tiles_m128;
            const uint8_t *act1 = args.A + (size_t)blk1 * args.a_kblocks_total * kI8BlockBytes + off1 * 128u;
            const uint8_t *act2 = args.A + (size_t)(blk1 + 1) * args.a_kblocks_total * kI8BlockBytes;
            const uint32_t tx = (nib_valid ? kW4NibBytes : 0u) + (v1 ? rows1 * 128u : 0u) + (v2 ? rows2 * 128u : 0u);
            for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                const uint32_t s = it % S, G = it >> 1;
                if ((it & 1u) == 0u) {   // first K step of a group: the group that used these two stages last is done
                    if (!TQT_PTIMED(0, ptx::mbar_wait_cluster(BAR(kGroupDone + G % NG), ((G / NG) & 1u) ^ 1u, sAbort, args.fault,
                                                              kFaultProducerWait))) {
                        ok = false;
                        break;
                    }
                }
                if (lane == 0) ptx::mbar_arrive_expect_tx(BAR(kFull + s), tx);
                __syncwarp();
                // three lanes issue one bulk copy each in the same instruction
                if (lane == 0) {
                    if (nib_valid)
                        ptx::bulk_g2s(ptx::smem_u32(sNib + s * kW4NibBytes), nib_src + (size_t)kb * kI4CxBlockBytes, kW4NibBytes,
                                      BAR(kFull + s));
                } else if (lane == 1) {
                    if (v1)
                        ptx::bulk_g2s(ptx::smem_u32(sAct + s * kActBytes), act1 + (size_t)kb * kI8BlockBytes, rows1 * 128u,
                                      BAR(kFull + s));
                } else if (lane == 2) {
                    if (v2)
                        ptx::bulk_g2s(ptx::smem_u32(sAct + s * kActBytes + rows1 * 128u), act2 + (size_t)kb * kI8BlockBytes,
                                      rows2 * 128u, BAR(kFull + s));
                }
                __syncwarp();
            }
        }
        if (!ok) {
            const uint32_t pending = it < S ? it : S;
            for (uint32_t i = 0; i < pending; ++i) {
                const uint32_t j = it - 1 - i;
                const uint32_t s = j % S, ph = (j / S) & 1u;
                const long long t0 = clock64();
                while (!ptx::mbar_try_wait(BAR(kFull + s), ph)) {
                    if (clock64() - t0 > ptx::kWaitLimitCycles) {
                        if (args.fault) atomicCAS(args.fault, 0u, (unsigned)kFaultDrainWait);
                        break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer (leader CTA only; the peer's warp 1 idles) =====================
        if (rank == 0) {
            const uint32_t idesc = ptx::make_idesc(2u, 1u, 1u, PAIR ? 256 : 128, kW4MT);
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (uint32_t t = pair; t < num_tiles && ok; t += npairs, ++ti) {
                const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
                if (!TQT_PTIMED(0, ptx::mbar_wait_cluster(BAR(kTmemEmpty + acc), pha ^ 1u, sAbort, args.fault, kFaultMmaWaitTmem))) {
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kW4MT;
                for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                    const uint32_t s = it % S, ts = it % T, pht = (it / T) & 1u;
                    // all eight converter warps have written their rows of operand stage ts (which also
                    // means both CTAs' activation halves of shared-memory stage s have landed)
                    if (!TQT_PTIMED(1, ptx::mbar_wait_cluster(BAR(kConvFull + ts), pht, sAbort, args.fault, kFaultMmaWaitFull, true))) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    if (lane == 0) {
                        const uint64_t b_desc = ptx::make_desc_k_sw128(ptx::smem_u32(sAct + s * kActBytes));
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            if constexpr (PAIR)
                                ptx::mma_i8_ts_pair(d_tmem, tmem_a + ts * 32u + j * 8u, b_desc + 2 * j, idesc, (kb | j) ? 1u : 0u);
                            else
                                ptx::mma_i8_ts(d_tmem, tmem_a + ts * 32u + j * 8u, b_desc + 2 * j, idesc, (kb | j) ? 1u : 0u);
                        }
                        const uint32_t G = it >> 1;
                        if constexpr (PAIR) {
                            if (it & 1u) ptx::tc_commit_pair(BAR(kGroupDone + G % NG), 3);
                            if (kb == KB - 1) ptx::tc_commit_pair(BAR(kTmemFull + acc), 3);
                        } else {
                            if (it & 1u) ptx::tc_commit(BAR(kGroupDone + G % NG));
                            if (kb == KB - 1) ptx::tc_commit(BAR(kTmemFull + acc));
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp < 10) {
        // ===================== epilogue (8 warps per CTA): D^T, lane = output channel ==================
        // Per-channel values (scale_b, bias, row sum) are per-thread constants; the per-row values
        // (scale_a, zero_point_a) of a 32-column strip are loaded one per lane and broadcast with
        // shuffles, so the epilogue makes no shared-memory reads that would queue behind the MMA's.
        const uint32_t quad = warp & 3u, half = (warp - 2u) >> 2;
        const uint32_t row = quad * 32u + lane;             // weight row inside this CTA's block
        uint32_t ti = 0;
        bool ok = true;
        for (uint32_t t = pair; t < num_tiles && ok; t += npairs, ++ti) {
            const uint32_t tm = t % tmc, tn = t / tmc;
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            const uint32_t n = (PAIR ? tn * 2 + rank : tn) * 128u + row;
            const bool n_ok = n < args.n;
            const uint32_t m0 = tm * kW4MT + half * 96u;
            const uint32_t mcols = args.m > m0 ? min(96u, args.m - m0) : 0u;
            const float sb = n_ok ? args.scale_b[n] : 0.0f;
            const float bv = (n_ok && args.bias) ? TdTraits<TD>::load(args.bias, n) : 0.0f;
            if (!TQT_PTIMED(0, ptx::mbar_wait_cluster(BAR(kTmemFull + acc), pha, sAbort, args.fault, kFaultEpilogueWait)) ||
                !TQT_PTIMED(1, ptx::mbar_wait(BAR(kRsumFull + acc), pha, sAbort, args.fault, kFaultEpilogueWait))) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            const int32_t rs = sRsum[acc * 256 + row] + sRsum[acc * 256 + 128 + row];
            const uint32_t t_addr = tmem_base + acc * kW4MT + half * 96u + ((quad * 32u) << 16);
            const uint32_t nchunks = (mcols + 31u) / 32u;
            for (uint32_t ch = 0; ch < nchunks; ++ch) {
                const uint32_t c0 = ch * 32u;
                const uint32_t nvalid = min(32u, mcols - c0);
                const float sa_l = lane < nvalid ? __ldg(args.scale_a + m0 + c0 + lane) : 0.0f;
                const int32_t zp_l = lane < nvalid ? __ldg(args.zp_a + m0 + c0 + lane) : 0;
                uint32_t r[32];
                __syncwarp();
                const long long tl0 = args.dbg ? clock64() : 0;
                ptx::tmem_ld_32x32b_x32(t_addr + c0, r);
                ptx::tmem_wait_ld();
                if (args.dbg) wcyc[2] += clock64() - tl0;
                OutT *dcol = static_cast<OutT *>(args.D) + (size_t)(m0 + c0) * args.ldd + n;
#pragma unroll
                for (uint32_t j = 0; j < 32; ++j) {
                    const float sa = __shfl_sync(0xffffffffu, sa_l, j);
                    const int32_t zp = __shfl_sync(0xffffffffu, zp_l, j);
                    // operands were 16*q: the accumulator is an exact multiple of 16
                    const int32_t a = (((int32_t)r[j]) >> 4) - zp * rs;
                    if (n_ok && j < nvalid) {
                        float cv = 0.0f;
                        if (args.C) cv = TdTraits<TD>::load(args.C, (size_t)(m0 + c0 + j) * args.ldc + n);
                        const float v = w4a8_epilogue(a, sa, sb, args.C != nullptr, cv, args.bias != nullptr, bv, args.cmin_f,
                                                      args.cmax_f);
                        dcol[(size_t)j * args.ldd] = cvt_out<OutT>(v);   // the warp writes 32 consecutive channels
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0)
                    ptx::mbar_arrive(BAR(kTmemEmpty + acc));
                else
                    ptx::mbar_arrive_cluster(ptx::mapa(BAR(kTmemEmpty + acc), 0));
                ptx::mbar_arrive(BAR(kRsumEmpty + acc));
            }
        }
    } else {
        // ===================== converters (warps 10..17): int4 -> int8 (16*q) into tensor memory ========
        // Two warps per tensor-memory lane quadrant: set 0 (warps 10..13) takes the even K steps, set 1
        // (warps 14..17) the odd ones.  Inside a warp the tensor-memory store of step i stays in flight
        // while step i+2 is fetched and expanded; only then does the warp wait for the store and
        // announce step i.
        const uint32_t quad = warp & 3u, cset = (warp - 10u) >> 2;
        const uint32_t row = quad * 32u + lane;
        const uint32_t swz_in = (row >> 1) & 3u;
        const uint32_t conv_full_leader = ptx::mapa(BAR(kConvFull), 0);   // + 8 * s
        auto announce = [&](uint32_t ts) {
            ptx::tmem_wait_st();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0)
                    ptx::mbar_arrive(BAR(kConvFull + ts));
                else
                    ptx::mbar_arrive_cluster(conv_full_leader + ts * 8u);
            }
        };
        uint32_t it = 0, ti = 0;
        bool ok = true;
        bool pending = false;      // a tensor-memory store has been issued but not announced
        uint32_t pending_s = 0;
        for (uint32_t t = pair; t < num_tiles && ok; t += npairs, ++ti) {
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            int32_t rsum = 0;
            for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                if ((it & 1u) != cset) continue;
                const uint32_t s = it % S, ph = (it / S) & 1u, ts = it % T;
                if (!TQT_PTIMED(0, ptx::mbar_wait(BAR(kFull + s), ph, sAbort, args.fault, kFaultConverterWait))) {
                    ok = false;
                    break;
                }
                const uint8_t *nrow = sNib + s * kW4NibBytes + row * 64u;
                uint32_t regs[32];
#pragma unroll
                for (uint32_t seg = 0; seg < 4; ++seg) {
                    const uint4 w = *reinterpret_cast<const uint4 *>(nrow + ((seg ^ swz_in) << 4));
                    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        regs[seg * 8 + j] = (ws[j] << 4) & 0xF0F0F0F0u;       // k = 32 seg + 4 j .. + 3
                        regs[seg * 8 + 4 + j] = ws[j] & 0xF0F0F0F0u;          // k = 32 seg + 16 + 4 j .. + 3
                    }
                }
                rsum += (int32_t) reinterpret_cast<const int16_t *>(sNib + s * kW4NibBytes + kI4NibBytes)[row];
                if (pending) announce(pending_s);
                // the MMAs of the group two groups back read this tensor-memory stage: they must be done
                const uint32_t G = it >> 1;
                if (G >= 2u) {
                    const uint32_t Gp = G - 2u;
                    if (!TQT_PTIMED(2, ptx::mbar_wait_cluster(BAR(kGroupDone + Gp % NG), (Gp / NG) & 1u, sAbort, args.fault,
                                                              kFaultConverterWait))) {
                        ok = false;
                        break;
                    }
                }
                __syncwarp();
                ptx::tmem_st_32x32b_x32(tmem_a + ts * 32u + ((quad * 32u) << 16), regs);
                pending = true;
                pending_s = ts;
            }
            if (!ok) break;
            if (pending) {   // the tile's last step must be visible before the leader can finish the tile
                announce(pending_s);
                pending = false;
            }
            if (!TQT_PTIMED(1, ptx::mbar_wait(BAR(kRsumEmpty + acc), pha ^ 1u, sAbort, args.fault, kFaultConverterWait))) {
                ok = false;
                break;
            }
            sRsum[acc * 256 + cset * 128 + row] = rsum;
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(BAR(kRsumFull + acc));
        }
        if (pending) announce(pending_s);
    }

    if (args.dbg && lane == 0 && (warp == 0 || warp == 1 || warp == 2 || warp == 10)) {
        long long *d = args.dbg + (size_t)blockIdx.x * 16 + (warp == 0 ? 0 : warp == 1 ? 4 : warp == 2 ? 8 : 12);
        d[0] = wcyc[0];
        d[1] = wcyc[1];
        d[2] = wcyc[2];
        d[3] = clock64() - t_role0;
    }
    ptx::tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) ptx::cluster_sync_all();
    if (warp == 1) {
        ptx::tc_fence_after();
        if constexpr (PAIR)
            ptx::tmem_dealloc_pair(tmem_base, 512);
        else
            ptx::tmem_dealloc(tmem_base, 512);
    }
}

template <Dtype TD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kW4Threads, 1) gemm_pair_w4a8_kernel(const UmmaArgs args)
{
    w4a8_ts_body<TD, true>(args);
}

// Same kernel on one CTA (cta_group::1): the CTA stages all 192 activation rows itself.
template <Dtype TD>
__global__ void __launch_bounds__(kW4Threads, 1) gemm_ts_w4a8_kernel(const UmmaArgs args)
{
    w4a8_ts_body<TD, false>(args);
}


// ---- host side ------------------------------------------------------------------------------------------
template <class Kern>
static Result launch_pair(Kern kern, const UmmaArgs &a, uint32_t num_tiles, uint32_t threads, uint32_t smem, cudaStream_t st,
                          bool *attr_set)
{
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
        attr_set[dev] = true;
    }
    const uint32_t max_pairs = (uint32_t)sm_count_cached() / 2;
    const uint32_t pairs = num_tiles < max_pairs ? num_tiles : max_pairs;
    kern<<<pairs * 2, threads, smem, st>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

Result pair_gemm_i8(const UmmaArgs &a, bool requant, cudaStream_t st)
{
    const uint32_t tiles = (((a.m + 127) / 128 + 1) / 2) * ((((a.n + 127) / 128) + 1) / 2);
    static bool set_s32[64] = {false}, set_req[64] = {false};
    if (requant) return launch_pair(gemm_pair_i8_kernel<EpiKind::Req8>, a, tiles, kI8Threads, kI8Smem, st, set_req);
    return launch_pair(gemm_pair_i8_kernel<EpiKind::S32>, a, tiles, kI8Threads, kI8Smem, st, set_s32);
}

template <class Kern>
static Result launch_single(Kern kern, const UmmaArgs &a, uint32_t num_tiles, uint32_t threads, uint32_t smem, cudaStream_t st,
                            bool *attr_set)
{
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
        attr_set[dev] = true;
    }
    const uint32_t sms = (uint32_t)sm_count_cached();
    kern<<<num_tiles < sms ? num_tiles : sms, threads, smem, st>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

Result ts_gemm_w4a8(const UmmaArgs &a, Dtype td, cudaStream_t st)
{
    const uint32_t tiles = ((a.m + kW4MT - 1) / kW4MT) * ((a.n + 127) / 128);
    static bool set0[64] = {false}, set1[64] = {false}, set2[64] = {false};
    switch (td) {
        case Dtype::F32: return launch_single(gemm_ts_w4a8_kernel<Dtype::F32>, a, tiles, kW4Threads, kW4SmemSingle, st, set0);
        case Dtype::F16: return launch_single(gemm_ts_w4a8_kernel<Dtype::F16>, a, tiles, kW4Threads, kW4SmemSingle, st, set1);
        default: return launch_single(gemm_ts_w4a8_kernel<Dtype::BF16>, a, tiles, kW4Threads, kW4SmemSingle, st, set2);
    }
}

Result pair_gemm_w4a8(const UmmaArgs &a, Dtype td, cudaStream_t st)
{
    const uint32_t tiles = ((a.m + kW4MT - 1) / kW4MT) * ((((a.n + 127) / 128) + 1) / 2);
    static bool set0[64] = {false}, set1[64] = {false}, set2[64] = {false};
    switch (td) {
        case Dtype::F32: return launch_pair(gemm_pair_w4a8_kernel<Dtype::F32>, a, tiles, kW4Threads, kW4Smem, st, set0);
        case Dtype::F16: return launch_pair(gemm_pair_w4a8_kernel<Dtype::F16>, a, tiles, kW4Threads, kW4Smem, st, set1);
        default: return launch_pair(gemm_pair_w4a8_kernel<Dtype::BF16>, a, tiles, kW4Threads, kW4Smem, st, set2);
    }
}

}  // namespace tqt
