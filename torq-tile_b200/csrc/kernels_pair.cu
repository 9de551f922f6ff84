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
#include <cuda.h>   // tensor-map types and enumerators only: the encode function is looked up at run time

#include <cstdlib>
#include <type_traits>

#include "epilogues.cuh"
#include "ptx_sm100.cuh"
#include "quant_row.cuh"
#include "umma_args.cuh"

namespace tqt {

// Role timing (cycles spent in each role's waits) and the per-group clock64 traces exist only in builds with
// -DTQT_B200_DIAG: the timed form of a wait duplicates its polling loop, and the kernels' hot loops are sensitive to code
// size (a few predicated diagnostic branches in the converter loop cost the C3 GEMM 8 %).
#ifdef TQT_B200_DIAG
#define TQT_DIAG_ON(args) ((args).dbg != nullptr)
#else
#define TQT_DIAG_ON(args) false
#endif
#define TQT_PTIMED(slot, call)                                  \
    ([&]() -> bool {                                            \
        if (!TQT_DIAG_ON(args)) return (call);                  \
        const long long _t0 = clock64();                        \
        const bool _r = (call);                                 \
        wcyc[slot] += clock64() - _t0;                          \
        return _r;                                              \
    }())

// ======================================================================================================
// int8 x int8
// ======================================================================================================
constexpr uint32_t kI8Stages = 6;
constexpr uint32_t kI8Threads = 384;   // warp 0 producer (even K steps), warp 1 MMA / relay, warps 2..9 epilogue, warp 10 producer (odd K steps), warp 11 second MMA issuer
constexpr uint32_t kI8Smem = 1024 + kI8Stages * 32768 + 8 * 3 * 128 * 4 + 256;

// Work items of the int8 CTA-pair kernel.  Item w is a pair tile (256 x 256: two 128-column blocks of the N side), except
// that the tiles of a last, at most half-full wave are split into two items of one block each (256 x 128): a one-block
// MMA costs ~0.6 of a two-block one, so the tail wave takes 0.6 of a full wave's time instead of all of it, on twice as
// many CTA pairs.  No reduction is involved: the halves are independent output columns.
struct I8Work {
    uint32_t pm;     // pair row-tile
    uint32_t bn0;    // first 128-column block of the N side
    uint32_t nblk;   // blocks: 2, or 1 (ragged last block, or half of a split tile)
};

struct I8Split {
    uint32_t full;   // items below this index are whole tiles
    uint32_t count;  // work items in all
    bool split;
};

__device__ __forceinline__ I8Split i8_split(uint32_t num_tiles, uint32_t npairs, bool allow)
{
    I8Split sp;
    sp.full = (num_tiles / npairs) * npairs;
    const uint32_t rem = num_tiles - sp.full;
    sp.split = allow && rem > 0 && 2u * rem <= npairs;
    sp.count = sp.split ? sp.full + 2u * rem : num_tiles;
    return sp;
}

// false: the item is empty (the second half of a tile whose second block lies beyond n); every role skips it alike
__device__ __forceinline__ bool i8_work(uint32_t w, const I8Split &sp, uint32_t pmc, uint32_t tnc, uint32_t band, uint32_t nblocks,
                                        bool b_whole, I8Work &o)
{
    uint32_t t = w, h = 2u;
    if (sp.split && w >= sp.full) {
        t = sp.full + ((w - sp.full) >> 1);
        h = (w - sp.full) & 1u;
    }
    uint32_t tn;
    tile_coords(t, pmc, tnc, band, o.pm, tn);
    if (h == 2u) {
        o.bn0 = tn * 2u;
        o.nblk = b_whole ? 2u : min(2u, nblocks - tn * 2u);
        return true;
    }
    o.bn0 = tn * 2u + h;
    o.nblk = 1u;
    return o.bn0 < nblocks;
}

// TMA = true: an operand whose args.a_src / args.b_src is not kSrcBlocks comes straight from the caller's row-major
// matrix through a tiled TMA load (one 128 x 128-byte box per stage, 128-byte swizzle: the box lands in exactly the
// layout a packed block has); cells outside the matrix read as zero, so ragged edges need no packing either.  A
// K-major box ([rows, k], k contiguous) is what a packed block holds; an MN-major box of B ([k, n], n contiguous)
// is consumed with the instruction descriptor's b_major bit and K slices 32 rows (4 KiB) apart.
template <EpiKind EK, Dtype TD, bool TMA>
__device__ __forceinline__ void pair_i8_body(const UmmaArgs &args, const TmaOperands *maps)
{
    using OutT = typename OutType<EK, TD>::type;
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
    volatile uint32_t *sIssued = reinterpret_cast<volatile uint32_t *>(sTmemBase + 3);   // K steps issued so far: whose turn it is

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto BAR = [&](uint32_t idx) { return bar0 + idx * 8u; };

    const uint32_t tiles_m = (args.m + 127) / 128, pmc = (tiles_m + 1) / 2;
    const uint32_t nblocks = (args.n + 127) / 128, tnc = (nblocks + 1) / 2;
    const uint32_t num_tiles = pmc * tnc;
    constexpr bool kFloat = EK == EpiKind::Float;   // 16-bit floating-point operands (kind::f16), f32 accumulators
    constexpr uint32_t kElem = kFloat ? 2u : 1u;
    const uint32_t KB = (args.k * kElem + 127) / 128;   // K blocks of 128 bytes per row
    // a B fetched by tiled TMA loads is always taken two blocks at a time (a box beyond the matrix is zeros); its tiles are not split
    const bool b_whole = TMA && args.b_src != kSrcBlocks;
    const I8Split sp = i8_split(num_tiles, npairs, !b_whole);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            ptx::mbar_init(BAR(kFull + s), 1);
            ptx::mbar_init(BAR(kPeerFull + s), 1);
            ptx::mbar_init(BAR(kEmpty + s), 1);
        }
        for (uint32_t e = 0; e < 2; ++e) {
            ptx::mbar_init(BAR(kTmemFull + e), 2);     // one commit per issuing thread
            ptx::mbar_init(BAR(kTmemEmpty + e), 16);   // 8 epilogue warps of each CTA
        }
        sAbort[0] = 0;
        sAbort[1] = (int)args.wait_shift;
        *sIssued = 0u;
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
    const long long t_role0 = TQT_DIAG_ON(args) ? clock64() : 0;

    if (warp == 0 || warp == 10) {
        // ===================== producers (both CTAs) =====================
        // The issue of a bulk copy costs its warp a few hundred cycles whatever its size (measured: one
        // warp sustains one set of copies per ~400-500 cycles, n warps n times that, up to ~72 B/clk per
        // SM), so two warps issue alternate K steps: warp 0 the even ones, warp 10 the odd ones.
        const uint32_t pw = warp == 0 ? 0u : 1u;
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t w = pair; w < sp.count && ok; w += npairs) {
            I8Work wk;
            if (!i8_work(w, sp, pmc, tnc, args.band_m, nblocks, b_whole, wk)) continue;
            const uint32_t pm = wk.pm, nblk = wk.nblk;
            const bool b_tma = b_whole, a_tma = TMA && args.a_src != kSrcBlocks;
            const uint32_t mtile = pm * 2 + rank;
            const bool a_valid = mtile < tiles_m;
            const uint32_t b_bytes = nblk == 2 ? 16384u : 8192u;
            const uint8_t *a_src = args.A + (size_t)mtile * args.a_kblocks_total * kI8BlockBytes;
            const size_t bbb = args.b_block_bytes;   // 16 KiB, or 16 KiB + the block's row sums
            const uint8_t *b_src = nblk == 2 ? args.B + (size_t)(wk.bn0 + rank) * args.b_kblocks_total * bbb
                                             : args.B + (size_t)wk.bn0 * args.b_kblocks_total * bbb + rank * 8192u;
            for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                if ((it & 1u) != pw) continue;
                const uint32_t s = it % S, ph = (it / S) & 1u;
                if (!TQT_PTIMED(0, ptx::mbar_wait_cluster(BAR(kEmpty + s), ph ^ 1u, sAbort, args.fault, kFaultProducerWait))) {
                    ok = false;
                    break;
                }
                if (lane == 0) ptx::mbar_arrive_expect_tx(BAR(kFull + s), (a_valid ? 16384u : 0u) + b_bytes);
                __syncwarp();
                // two lanes issue one copy each in the same instruction
                if (lane == 0) {
                    if (b_tma) {
                        const int32_t rows0 = (int32_t)((wk.bn0 + rank) * 128u), k0 = (int32_t)(kb * 128u);
                        if (args.b_src == kSrcTmaMn) {
                            // B stored [k, n]: x runs along n.  int8: one box of 128 columns x 128 k rows; 16-bit types: the
                            // first of two boxes of 64 columns (128 bytes) x 64 k rows (lane 2 issues the second)
                            if constexpr (kFloat)
                                ptx::tma_load_2d(ptx::smem_u32(sB + s * 16384), &maps->b, rows0 * 2, (int32_t)(kb * 64u), BAR(kFull + s));
                            else
                                ptx::tma_load_2d(ptx::smem_u32(sB + s * 16384), &maps->b, rows0, k0, BAR(kFull + s));
                        } else {
                            ptx::tma_load_2d(ptx::smem_u32(sB + s * 16384), &maps->b, k0, rows0, BAR(kFull + s));
                        }
                    } else {
                        ptx::bulk_g2s(ptx::smem_u32(sB + s * 16384), b_src + (size_t)kb * bbb, b_bytes, BAR(kFull + s));
                    }
                } else if (lane == 1 && a_valid) {
                    if (a_tma)
                        ptx::tma_load_2d(ptx::smem_u32(sA + s * 16384), &maps->a, (int32_t)(kb * 128u), (int32_t)(mtile * 128u),
                                         BAR(kFull + s));
                    else
                        ptx::bulk_g2s(ptx::smem_u32(sA + s * 16384), a_src + (size_t)kb * kI8BlockBytes, 16384u, BAR(kFull + s));
                } else if (kFloat && lane == 2 && b_tma && args.b_src == kSrcTmaMn) {
                    const int32_t cols1 = (int32_t)(((wk.bn0 + rank) * 128u + 64u) * 2u);   // the second 64 columns, in bytes
                    ptx::tma_load_2d(ptx::smem_u32(sB + s * 16384 + 8192), &maps->b, cols1, (int32_t)(kb * 64u), BAR(kFull + s));
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
                    if (clock64() - t0 > ptx::wait_limit(sAbort)) {
                        if (args.fault) atomicCAS(args.fault, 0u, (unsigned)kFaultDrainWait);
                        break;
                    }
                }
            }
        }
    } else if ((warp == 1 || warp == 11) && rank == 0) {
        // ===================== MMA issuers (one thread each, leader CTA) =====================
        // A K step occupies the pipe for ~680 cycles; one thread that waits for the step's two barriers (own stage
        // landed, peer's stage landed), fences, issues the four MMAs and commits needs longer than that, and the pipe's
        // queue does not cover the difference.  Two threads in different SM sub-partitions therefore take the K steps in
        // turn (the counter sIssued hands the turn over, so the MMAs enter the pipe in step order: the first MMA of a
        // tile overwrites the accumulator, and floating-point accumulation keeps one order): while one commits and tests
        // its next step's barriers the other is issuing.  Each thread commits its own steps; the accumulator-full
        // barrier takes one commit from each.  The four MMAs of a step go out in one instruction block from precomputed
        // descriptor words, and the next step's barriers are tested after this step's MMAs and read after its commit.
        static_assert(S % 2u == 0u, "the two issuing threads keep to the stages of their own parity");
        const uint32_t who = warp == 1 ? 0u : 1u;
        if (lane == 0) {
            const bool b_mn = TMA && args.b_src == kSrcTmaMn;
            const uint32_t ffmt = args.in_bf16 ? 1u : 0u;
            const uint32_t idesc256 = (kFloat ? ptx::make_idesc(1u, ffmt, ffmt, 256, 256) : ptx::make_idesc(2u, 1u, 1u, 256, 256)) |
                                      (b_mn ? ptx::kIdescBMajorMn : 0u);
            const uint32_t idesc128 = kFloat ? ptx::make_idesc(1u, ffmt, ffmt, 256, 128) : ptx::make_idesc(2u, 1u, 1u, 256, 128);
            // a 16-bit MN-major stage is two column groups of 64 (128 bytes wide, 64 k rows each) 8 KiB apart
            const uint64_t a_desc0 = ptx::make_desc_k_sw128(ptx::smem_u32(sA)),
                           b_desc0 = (kFloat && b_mn) ? ptx::make_desc_sw128(ptx::smem_u32(sB), 8192u, 1024u)
                                                      : ptx::make_desc_k_sw128(ptx::smem_u32(sB));
            const uint32_t a_lo0 = (uint32_t)a_desc0, a_hi = (uint32_t)(a_desc0 >> 32);
            const uint32_t b_lo0 = (uint32_t)b_desc0, b_hi = (uint32_t)(b_desc0 >> 32);
            const uint32_t peer_tmem_full = ptx::mapa(BAR(kTmemFull), 1);
            uint32_t it = 0, ti = 0, s = who, ph = 0;   // it = K steps of the items before this one; s, ph = this thread's next stage
            bool ok = true, ready = false;
            for (uint32_t w = pair; w < sp.count && ok; w += npairs) {
                I8Work wk;
                if (!i8_work(w, sp, pmc, tnc, args.band_m, nblocks, b_whole, wk)) continue;
                const uint32_t idesc = wk.nblk == 2 ? idesc256 : idesc128;
                const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
                if (!TQT_PTIMED(0, ptx::mbar_wait(BAR(kTmemEmpty + acc), pha ^ 1u, sAbort, args.fault, kFaultMmaWaitTmem))) {
                    ok = false;
                    break;
                }
                const uint32_t d_tmem = tmem_base + acc * 256u;
                const uint32_t kb_first = (it & 1u) ^ who;
                if (kb_first >= KB) {
                    // a one-step item that is the other thread's: only keep the accumulator-full barrier's count (the
                    // wait above paces this: the barrier's previous phase has been consumed)
                    ptx::mbar_arrive(BAR(kTmemFull + acc));
                    ptx::mbar_arrive_cluster(peer_tmem_full + acc * 8u);
                }
                for (uint32_t kb = kb_first; kb < KB; kb += 2u) {
                    const uint32_t step = it + kb;
                    if (!ready && (!TQT_PTIMED(1, ptx::mbar_wait(BAR(kFull + s), ph, sAbort, args.fault, kFaultMmaWaitFull, 0u)) ||
                                   !TQT_PTIMED(2, ptx::mbar_wait(BAR(kPeerFull + s), ph, sAbort, args.fault, kFaultMmaWaitFull, 0u)))) {
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    if (*sIssued != step) {   // this thread's turn comes when the other one has issued step - 1
                        const long long t0 = clock64();
                        while (*sIssued != step) {
                            if (*sAbort || clock64() - t0 > ptx::wait_limit(sAbort)) {
                                if (!*sAbort && args.fault) atomicCAS(args.fault, 0u, (unsigned)kFaultMmaWaitFull);
                                *sAbort = 1;
                                ok = false;
                                break;
                            }
                        }
                        if (!ok) break;
                    }
                    if constexpr (kFloat) {
                        if (b_mn)   // K slices of 16 rows of 128 bytes
                            ptx::mma_f16_ss_pair_group4<128>(d_tmem, a_lo0 + s * 1024u, a_hi, b_lo0 + s * 1024u, b_hi, idesc, kb);
                        else
                            ptx::mma_f16_ss_pair_group4(d_tmem, a_lo0 + s * 1024u, a_hi, b_lo0 + s * 1024u, b_hi, idesc, kb);
                    } else if (b_mn)
                        ptx::mma_i8_ss_pair_group4<256>(d_tmem, a_lo0 + s * 1024u, a_hi, b_lo0 + s * 1024u, b_hi, idesc, kb);
                    else
                        ptx::mma_i8_ss_pair_group4(d_tmem, a_lo0 + s * 1024u, a_hi, b_lo0 + s * 1024u, b_hi, idesc, kb);   // 16 KiB stages = 1024 units
                    asm volatile("" ::: "memory");
                    *sIssued = step + 1u;
                    // this thread's next step's stage (a phase seen complete stays complete until this thread commits it free again)
                    const uint32_t s1 = s + 2u >= S ? s + 2u - S : s + 2u, ph1 = s + 2u >= S ? ph ^ 1u : ph;
                    const bool next_ready = ptx::mbar_test_wait(BAR(kFull + s1), ph1) && ptx::mbar_test_wait(BAR(kPeerFull + s1), ph1);
                    ptx::tc_commit_pair(BAR(kEmpty + s), 3);
                    if (kb + 2u >= KB) ptx::tc_commit_pair(BAR(kTmemFull + acc), 3);
                    ready = next_ready;
                    s = s1;
                    ph = ph1;
                }
                it += KB;
                ++ti;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ===================== relay (peer CTA): tells the leader that this CTA's stage has landed =====
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t w = pair; w < sp.count && ok; w += npairs) {
            I8Work wk;
            if (!i8_work(w, sp, pmc, tnc, args.band_m, nblocks, b_whole, wk)) continue;
            for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                const uint32_t s = it % S, ph = (it / S) & 1u;
                if (!TQT_PTIMED(1, ptx::mbar_wait(BAR(kFull + s), ph, sAbort, args.fault, kFaultMmaWaitFull))) {
                    ok = false;
                    break;
                }
                if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(BAR(kPeerFull + s), 0));
                __syncwarp();
            }
        }
    } else if (warp == 11) {
        // the peer CTA's second-issuer warp has no role
    } else {
        // ===================== epilogue (8 warps per CTA) =====================
        const uint32_t quad = warp & 3u, half = (warp - 2u) >> 2;   // TMEM lane quadrant, column half
        int32_t *sCol = sColAll + (warp - 2u) * 384u;
        uint32_t ti = 0;
        bool ok = true;
        for (uint32_t w = pair; w < sp.count && ok; w += npairs) {
            I8Work wk;
            if (!i8_work(w, sp, pmc, tnc, args.band_m, nblocks, b_whole, wk)) continue;
            const uint32_t pm = wk.pm;
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            ++ti;
            // this warp's column half exists when the item has two blocks (or is the first of one)
            const uint32_t n0 = (wk.bn0 + half) * 128u;
            const uint32_t ncols = (half < wk.nblk && args.n > n0) ? min(128u, args.n - n0) : 0u;
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
            // dynamic-activation W8A8 with float output: per column the row sum of B (from the packed blocks' tails),
            // scale_b and the bias; per row (= this thread) scale_a and zero_point_a
            float row_sa = 0.0f;
            int32_t row_zp = 0;
            if constexpr (EK == EpiKind::DxCx) {
                const uint32_t blk = wk.bn0 + half;   // this warp's 128 columns are one 128-row block tile of B
                for (uint32_t c = lane; c < 128u; c += 32u) {
                    const bool cok = c < ncols;
                    int32_t rsum = 0;
                    if (TMA && args.b_src == kSrcTmaK) {
                        // row-major B [n, ldb] carries no row sums: add up the row (16-byte aligned by the tensor map's rules)
                        if (cok) {
                            const uint8_t *brow = args.B + (size_t)(n0 + c) * args.b_ld;
                            uint32_t kk = 0;
                            for (; kk + 16u <= args.k; kk += 16u) {
                                const uint4 v = *reinterpret_cast<const uint4 *>(brow + kk);
                                rsum = __dp4a((int)v.x, 0x01010101, rsum);
                                rsum = __dp4a((int)v.y, 0x01010101, rsum);
                                rsum = __dp4a((int)v.z, 0x01010101, rsum);
                                rsum = __dp4a((int)v.w, 0x01010101, rsum);
                            }
                            for (; kk < args.k; ++kk) rsum += (int32_t)(int8_t)brow[kk];
                        }
                    } else if (cok) {
                        const uint8_t *tail = args.B + (size_t)blk * args.b_kblocks_total * args.b_block_bytes + kI8BlockBytes + c * 2u;
                        for (uint32_t kb = 0; kb < KB; ++kb)
                            rsum += (int32_t) * reinterpret_cast<const int16_t *>(tail + (size_t)kb * args.b_block_bytes);
                    }
                    sCol[c] = rsum;
                    sCol[128 + c] = cok ? __float_as_int(args.scale_b[n0 + c]) : 0;
                    float bv = 0.0f;
                    if (cok && args.bias) bv = TdTraits<TD>::load(args.bias, n0 + c);
                    sCol[256 + c] = __float_as_int(bv);
                }
                if (row_ok) {
                    row_sa = args.scale_a[mrow];
                    row_zp = args.zp_a[mrow];
                }
            }
            // unquantised GEMM: bias per column (staged as float bits) or per row (this thread's constant)
            float row_bias_f = 0.0f;
            if constexpr (EK == EpiKind::Float) {
                for (uint32_t c = lane; c < 128u; c += 32u) {
                    float bv = 0.0f;
                    if (c < ncols && args.bias && !args.bias_per_row) bv = TdTraits<TD>::load(args.bias, n0 + c);
                    sCol[256 + c] = __float_as_int(bv);
                }
                if (row_ok && args.bias && args.bias_per_row) row_bias_f = TdTraits<TD>::load(args.bias, mrow);
            }
            // per-row requantisation (Mx1 bias types): this thread's row has one multiplier, shift and bias
            int32_t row_mult = 0, row_rsh = 0, row_bias = 0;
            if constexpr (EK == EpiKind::Req8Row) {
                if (row_ok) {
                    requant_column(args.rq_scale_rows[args.rq_per_tensor ? 0 : mrow], args.rq_scale_a, args.rq_scale_d, &row_mult,
                                   &row_rsh);
                    if (args.bias) row_bias = static_cast<const int32_t *>(args.bias)[mrow];
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
            const bool has_bias = args.bias != nullptr;
            for (uint32_t ch = 0; ch < nchunks; ++ch) {
                uint32_t r[32];
                __syncwarp();
                const long long tl0 = TQT_DIAG_ON(args) ? clock64() : 0;
                ptx::tmem_ld_32x32b_x32(t_addr + ch * 32u, r);
                ptx::tmem_wait_ld();
                if (TQT_DIAG_ON(args)) wcyc[2] += clock64() - tl0;
                if (row_ok) {
                    const uint32_t c0 = ch * 32u;
                    const uint32_t nvalid = min(32u, ncols - c0);
                    alignas(16) OutT out[32];
                    if constexpr (EK != EpiKind::DxCx && EK != EpiKind::Float) {
                        // the optional C operand: one uniform branch per strip, so the loop below has none
                        if (args.C) {
                            const int32_t *crow = static_cast<const int32_t *>(args.C) + mrow * args.ldc + n0 + c0;
#pragma unroll
                            for (uint32_t j = 0; j < 32; ++j)
                                if (j < nvalid) r[j] += (uint32_t)crow[j];
                        }
                    }
#pragma unroll
                    for (uint32_t j = 0; j < 32; ++j) {
                        const uint32_t c = c0 + j;
                        if constexpr (EK == EpiKind::S32) {
                            const int32_t v = (int32_t)r[j];
                            out[j] = max(args.cmin_i, min(args.cmax_i, v));
                        } else if constexpr (EK == EpiKind::Float) {
                            // + C, + bias, clamp in f32, one narrowing (test/common/reference_gemm.cpp:38-57); nothing is
                            // added where the caller passed no C / no bias (x + 0 would turn -0 into +0)
                            float v = __uint_as_float(r[j]);
                            if (args.C && j < nvalid) v = __fadd_rn(v, TdTraits<TD>::load(args.C, mrow * args.ldc + n0 + c));
                            if (has_bias) v = __fadd_rn(v, args.bias_per_row ? row_bias_f : __int_as_float(sCol[256 + c]));
                            v = fminf(fmaxf(v, args.cmin_f), args.cmax_f);
                            out[j] = cvt_out<OutT>(v);
                        } else if constexpr (EK == EpiKind::DxCx) {
                            // acc - zp_a * rowsum(b), then r = (float)acc * (scale_b * scale_a); f32: + bias, clamp;
                            // f16: narrow first, then add the bias and clamp in f16 (as EpiDxCx in epilogues.cuh)
                            const int32_t a = (int32_t)(r[j] - (uint32_t)row_zp * (uint32_t)sCol[c]);
                            const float sc = __fmul_rn(__int_as_float(sCol[128 + c]), row_sa);
                            float v = __fmul_rn(__int2float_rn(a), sc);
                            const float bv = __int_as_float(sCol[256 + c]);
                            if constexpr (TD == Dtype::F32) {
                                v = has_bias ? __fadd_rn(v, bv) : v;
                                v = v < args.cmin_f ? args.cmin_f : v;
                                v = v > args.cmax_f ? args.cmax_f : v;
                                out[j] = v;
                            } else {
                                float h = __half2float(__float2half_rn(v));
                                h = has_bias ? __half2float(__float2half_rn(__fadd_rn(h, bv))) : h;
                                h = h < args.cmin_f ? args.cmin_f : h;
                                h = h > args.cmax_f ? args.cmax_f : h;
                                out[j] = __float2half_rn(h);
                            }
                        } else if constexpr (EK == EpiKind::Req8Row) {
                            uint32_t u = r[j];
                            u += (uint32_t)row_bias;
                            out[j] = (int8_t)requant_value((int32_t)u, row_mult, row_rsh, args.rq_zp_d, args.cmin_i, args.cmax_i);
                        } else {
                            uint32_t u = r[j];
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

    if (TQT_DIAG_ON(args) && lane == 0 && (warp == 0 || warp == 1 || warp == 2)) {
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

template <EpiKind EK, Dtype TD = Dtype::F32>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kI8Threads, 1) gemm_pair_i8_kernel(const UmmaArgs args)
{
    pair_i8_body<EK, TD, false>(args, nullptr);
}

// Operands in the caller's own row-major layouts: the tensor maps travel as a kernel parameter.
template <EpiKind EK, Dtype TD = Dtype::F32>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kI8Threads, 1)
    gemm_pair_i8_tma_kernel(const UmmaArgs args, const __grid_constant__ TmaOperands maps)
{
    pair_i8_body<EK, TD, true>(args, &maps);
}

// ======================================================================================================
// int4 weights through tensor memory: W4A8 (kind::i8) and W4A16 (kind::f16)
// ======================================================================================================
enum class TsKind : int { W4A8 = 0, W4A16 = 1 };

constexpr uint32_t kTsMT = 192;            // activation rows per tile (MMA N) by default; 96 per CTA in a pair
constexpr uint32_t kTsMTWide = 256;        // CTA pairs, launches of at most one tile per pair: one accumulator of 256 columns
// Warp roles: 0 producer (step 0 of each group), 1 MMA issuer, 2..9 epilogue, then the converter sets of four warps
// each (set c expands the K steps c, c + sets, c + 2 sets, ... numbered through the whole launch), then the producer of
// step 1 and the second MMA issuer (CTA pairs).  Packed W4A8 has two converter sets (640 threads); W4A16, whose expansion
// is heavier (an f16 per weight, block scales), and the row-major nibble order (byte permutes, row sums by dp4a) three
// (768 threads): 3.86 -> 3.62 ms at the 8192 x 8192 x 28672 W4A16 shape, while a third set changed nothing for packed W4A8.
template <TsKind KD, bool UNP = false>
__host__ __device__ constexpr uint32_t ts_sets() { return (KD == TsKind::W4A16 || UNP) ? 3u : 2u; }
template <TsKind KD, bool UNP = false>
__host__ __device__ constexpr uint32_t ts_threads() { return 32u * (10u + 4u * ts_sets<KD, UNP>() + 2u); }
constexpr uint32_t kTsMaxSets = 3;
constexpr uint32_t kTsT = 4;               // tensor-memory operand stages (4 x 32 columns)

// WIDE (CTA pairs only): 256 activation rows per tile on one accumulator, for launches of at most one tile per pair.
template <TsKind KD, bool PAIR, bool WIDE>
struct TsCfg {
    static_assert(PAIR || !WIDE, "the wide tile exists for CTA pairs only");
    static constexpr bool kF16 = KD == TsKind::W4A16;
    static constexpr uint32_t kMT = WIDE ? kTsMTWide : kTsMT;      // activation rows per tile (MMA N)
    static constexpr uint32_t NG = PAIR ? (WIDE ? 4u : 5u) : 3u;   // shared-memory stage groups (two K steps each)
    static constexpr uint32_t S = NG * 2u;
    static constexpr uint32_t kActRows = PAIR ? kMT / 2u : kMT;    // activation rows this CTA stages per K step
    static constexpr uint32_t kActBytes = kActRows * 128u;         // stage stride
    static constexpr uint32_t kNibGroupBytes = kF16 ? 8192u : 2u * 8448u;   // int4 bytes per group of two K steps
    static constexpr uint32_t kUsed = 1024u + S * kActBytes + NG * kNibGroupBytes + 2u * kTsMaxSets * 128u * 4u + 512u;
    // more than half of an SM's shared memory: one CTA per SM, which owns all 512 tensor-memory columns
    static constexpr uint32_t kSmem = kUsed > 120u * 1024u ? kUsed : 120u * 1024u;
};

// Waits: every mbarrier a thread waits on lives in its own CTA's shared memory, also those that the peer CTA
// arrives on (relaxed remote arrives) or that a multicast tcgen05.commit completes, so the waits use the
// CTA-scope try_wait: the cluster-scope acquire form costs about 200 cycles per call even on a completed phase,
// which the MMA issuer paid twice per group of eight MMAs.  What the barriers order is tensor-memory traffic, and
// that is fenced by tcgen05.wait::st / tcgen05.fence on both sides, not by the barrier's memory scope.
// A K step is 128 int8 (W4A8) or 64 f16 (W4A16): 128 bytes per activation row and 32 tensor-memory
// columns per weight row either way.  Steps are handled in groups of two: one tcgen05.commit per group
// releases two shared-memory stages and two tensor-memory operand stages (a commit after MMAs that
// read their M-side operand from tensor memory drains the MMA pipeline, so they are kept rare).
// REPL: the epilogue also stores into the output replicas (fused all-gather).  A separate instantiation: with the
// replica stores compiled into the common kernel, even as a branch never taken, every launch ran 10 % slower
// (code size: the strip loop is unrolled 32 times).
// The two 4-bit values (k = 2 t, 2 t + 1 of an 8-k word) as the low nibbles of the two halves of a word.  Packed qsi4c2
// blocks order a word's nibbles (k0,k2,k4,k6,k1,k3,k5,k7) so that one shift and mask does it; row-major weights hold them
// in k order.
template <bool SEQUENTIAL>
__device__ __forceinline__ uint32_t nib_pair(uint32_t w, uint32_t t)
{
    if (SEQUENTIAL) {
        const uint32_t x = w >> (8u * t);
        return (x & 0xFu) | ((x << 12) & 0x000F0000u);
    }
    return (w >> (4u * t)) & 0x000F000Fu;
}

// UNP (CTA pairs, 192-row tiles only): the operands stay in the caller's row-major layouts and every stage is fetched by
// tiled TMA loads through the two tensor maps in `maps`: activations int8 / f16 [m, lda] as boxes of 128 bytes x 96 rows
// with the 128-byte swizzle (what a slice of a packed block looks like), weights as nibbles [n, ldb / 2 bytes] in the
// reference's unpacked encoding (byte = (q_hi + 8) << 4 | (q_lo + 8), consecutive k in consecutive nibbles) as boxes of
// 64 bytes x 128 rows with the 64-byte swizzle, which puts 16-byte segment s of row r at position s ^ ((r >> 1) & 3)
// like a packed block.  The converters decode that nibble order and add up the row sums themselves (the packed
// blocks carry them in their tails); cells outside the matrices arrive as zero bytes.
// Grid-wide barrier for a launch whose CTAs are all resident (a cooperative launch): sense reversal on two words of
// device memory, [arrivals, generation].  Thread 0 of every CTA arrives; the last arrival clears the count and advances
// the generation, the others poll the generation with a bounded wait.  Returns false when the wait ran out (the
// caller then skips its work and tears down).  Writes made before the barrier by any thread of any CTA are visible to
// every thread after it, to bulk copies too (fence.proxy.async).
__device__ __forceinline__ bool grid_barrier(unsigned int *sync, unsigned int nblocks, volatile int *sAbort, unsigned int *fault)
{
    __syncthreads();
    __shared__ int s_ok;
    if (threadIdx.x == 0) {
        int ok = 1;
        unsigned int gen;
        asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(gen) : "l"(sync + 1) : "memory");
        __threadfence();
        if (atomicAdd(sync, 1u) == nblocks - 1u) {
            atomicExch(sync, 0u);
            __threadfence();
            atomicAdd(sync + 1, 1u);
        } else {
            const long long t0 = clock64();
            unsigned int now;
            while (true) {
                asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(now) : "l"(sync + 1) : "memory");
                if (now != gen) break;
                if (clock64() - t0 > ptx::wait_limit(sAbort)) {
                    if (fault) atomicCAS(fault, 0u, (unsigned)kFaultGridBarrier);
                    ok = 0;
                    break;
                }
                __nanosleep(32);
            }
        }
        __threadfence();
        s_ok = ok;
    }
    __syncthreads();
    asm volatile("fence.proxy.async;" ::: "memory");
    return s_ok != 0;
}

template <TsKind KD, Dtype TD, bool PAIR, bool WIDE, bool REPL, bool UNP = false, bool FUSEQ = false>
__device__ __forceinline__ void ts_body(const UmmaArgs &args, const TmaOperands *maps = nullptr)
{
    static_assert(!UNP || (PAIR && !WIDE && !REPL), "row-major operands: CTA pairs with 192-row tiles only");
    static_assert(!FUSEQ || (KD == TsKind::W4A8 && PAIR && !WIDE && !REPL && !UNP), "fused quantiser: W4A8 CTA pairs, 192-row tiles");
    using Cfg = TsCfg<KD, PAIR, WIDE>;
    using OutT = typename TdTraits<TD>::type;
    constexpr bool kF16 = Cfg::kF16;
    constexpr uint32_t S = Cfg::S, NG = Cfg::NG, T = kTsT;
    constexpr uint32_t kActBytes = Cfg::kActBytes;
    // activation rows per tile: 192 (two accumulators), or 256 for a CTA pair when the host found that every pair
    // then gets at most one tile (one accumulator of 256 columns at column 0; the operand stages stay at 384)
    constexpr uint32_t mt = Cfg::kMT, kActRows = Cfg::kActRows;
    constexpr uint32_t kStepK = kF16 ? 64u : 128u;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sAct = smem;                                   // S x 12 or 24 KiB (multiples of 1024)
    uint8_t *sNib = sAct + S * kActBytes;                   // NG groups of packed int4
    int32_t *sRsum = reinterpret_cast<int32_t *>(sNib + NG * Cfg::kNibGroupBytes);   // [2 accumulators][converter sets][128]
    constexpr uint32_t kSets = ts_sets<KD, UNP>(), kProd1Warp = 10u + 4u * kSets, kIssuer1Warp = kProd1Warp + 1u;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sRsum + 2u * kTsMaxSets * 128u);
    constexpr uint32_t kFull = 0, kGroupDone = S, kConvFull = S + NG, kTmemFull = S + NG + T, kTmemEmpty = kTmemFull + 2,
                       kRsumFull = kTmemFull + 4, kRsumEmpty = kTmemFull + 6;
    uint32_t *sTmemBase = reinterpret_cast<uint32_t *>(bars + kTmemFull + 8);
    volatile int *sAbort = reinterpret_cast<volatile int *>(sTmemBase + 1);
    // CTA pairs issue their MMAs from two threads that take the groups in turn (warp 1 the even ones, the last warp the
    // odd ones): sIssued counts the groups issued so far and hands the turn over
    constexpr bool kDual = PAIR;
    volatile uint32_t *sIssued = reinterpret_cast<volatile uint32_t *>(sTmemBase + 3);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;
    const uint32_t pair = PAIR ? blockIdx.x >> 1 : blockIdx.x, npairs = PAIR ? gridDim.x >> 1 : gridDim.x;
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto BAR = [&](uint32_t idx) { return bar0 + idx * 8u; };

    if (args.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the successor may start its own prologue
    const uint32_t tiles_m128 = (args.m + 127) / 128;          // 128-row blocks that exist in A_packed
    const uint32_t tmc = (args.m + mt - 1) / mt;               // row tiles of the activations
    const uint32_t nblocks = (args.n + 127) / 128, tnc = PAIR ? (nblocks + 1) / 2 : nblocks;
    const uint32_t num_tiles = tmc * tnc;
    const uint32_t ksteps = (args.k + kStepK - 1) / kStepK;    // K steps per tile
    const uint32_t ngroups = (ksteps + 1) / 2;                 // groups per tile (the last may hold one step)

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) ptx::mbar_init(BAR(kFull + s), 1);
        for (uint32_t g = 0; g < NG; ++g) ptx::mbar_init(BAR(kGroupDone + g), 1);
        for (uint32_t s = 0; s < 2; ++s) ptx::mbar_init(BAR(kConvFull + s), PAIR ? 16 : 8);   // per group slot: two steps announced by four converter warps each, per CTA
        for (uint32_t e = 0; e < 2; ++e) {
            ptx::mbar_init(BAR(kTmemFull + e), kDual ? 2 : 1);   // one commit per issuing thread
            ptx::mbar_init(BAR(kTmemEmpty + e), PAIR ? 16 : 8);
            ptx::mbar_init(BAR(kRsumFull + e), 4u * kSets);   // the converter warps
            ptx::mbar_init(BAR(kRsumEmpty + e), 8);
        }
        sAbort[0] = 0;
        sAbort[1] = (int)args.wait_shift;
        *sIssued = 0u;
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
    const uint32_t tmem_a = tmem_base + 2 * kTsMT;   // operand stages after the two accumulators
    // Programmatic dependent launch: barriers, tensor memory and the cluster handshake above overlap the tail of
    // the preceding kernel (the activation quantiser); everything below reads what it produced.
    if (args.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    long long wcyc[3] = {0, 0, 0};
    const long long t_role0 = TQT_DIAG_ON(args) ? clock64() : 0;
    // how long a waiting thread may stay suspended in hardware before it polls again: the waits on the critical
    // loop (issuer <-> converters) poll often, the others sleep long
    // diagnostic: with inject bit 6 the timing buffer of pair 0's leader CTA receives a per-step timeline instead
    // (2048 int64: [0,512) issuer, [512,1024) converter warp 10, [1024,1536) converter warp 14, [1536,2048) epilogue warp 2)
    long long *trace = (TQT_DIAG_ON(args) && (args.inject & 64u) && blockIdx.x == 0) ? args.dbg : nullptr;
    long long *trace_peer = (TQT_DIAG_ON(args) && (args.inject & 64u) && blockIdx.x == 1) ? args.dbg + 1536 : nullptr;   // peer CTA: converter warp 12
    const uint32_t hint_mma = (args.inject & 16u) ? 0u : ptx::kTryWaitSuspendNs;
    const uint32_t hint_conv = (args.inject & 32u) ? 0u : ptx::kTryWaitSuspendNs;
    bool conv_failed = false;   // a converter warp whose waits ran out does not help with the epilogue
    bool run_roles = true;
    if constexpr (FUSEQ) {
        // Phase 0: every warp of the grid quantises rows of the activations into the packed A operand this kernel is
        // about to read (one row per warp at a time), then all CTAs meet at a grid-wide barrier.
        // rows are dealt round-robin over the CTAs first, so that few rows still spread over every SM
        const uint32_t gw = warp * gridDim.x + blockIdx.x, nw = gridDim.x * (blockDim.x / 32u);
        uint8_t *a_out = const_cast<uint8_t *>(args.A);
        float *sa_out = const_cast<float *>(args.scale_a);
        int32_t *zp_out = const_cast<int32_t *>(args.zp_a);
        for (size_t row = gw; row < args.m; row += nw) {
            if (args.q_bf16)
                quant_row_warp<Dtype::BF16, true>(row, args.k, args.q_in, args.q_lda, a_out, 0, args.a_kblocks_total, sa_out, zp_out, lane);
            else
                quant_row_warp<Dtype::F16, true>(row, args.k, args.q_in, args.q_lda, a_out, 0, args.a_kblocks_total, sa_out, zp_out, lane);
        }
        asm volatile("fence.proxy.async;" ::: "memory");   // the packed rows are read by bulk copies after the barrier
        run_roles = grid_barrier(args.grid_sync, gridDim.x, sAbort, args.fault);
    }

    if (!run_roles) {
        // the grid barrier ran out: nothing was started, fall through to the teardown
    } else if (warp == 0 || warp == kProd1Warp) {
        // ===================== producers (both CTAs) =====================
        // The issue of a bulk copy costs its warp a few hundred cycles whatever its size (measured: one
        // warp sustains one set of copies per ~400-500 cycles, n warps n times that, up to ~72 B/clk per
        // SM), so the two K steps of a group are issued by two warps: warp 0 step 0, the warp after the converters step 1.
        const uint32_t ph = warp == 0 ? 0u : 1u;
        uint32_t Gc = 0;   // groups issued so far
        uint32_t withheld = 0xffffffffu;   // group whose stage this warp left without copies and arrive (test knob)
        bool ok = true;
        for (uint32_t t = pair; t < num_tiles && ok; t += npairs) {
            uint32_t tm, tn;
            tile_coords(t, tmc, tnc, args.band_m, tm, tn);
            const uint32_t nb = PAIR ? tn * 2 + rank : tn;
            const bool nib_valid = nb < nblocks;
            const uint8_t *nib_src = args.B + (size_t)nb * args.b_kblocks_total * (kF16 ? kI4C2BlockBytes : kI4CxBlockBytes);
            // this CTA's activation rows [a0, a0 + kActRows) = at most two pieces of 128-row blocks
            const uint32_t a0 = tm * mt + rank * kActRows;
            const uint32_t blk1 = a0 >> 7, off1 = a0 & 127u;
            const uint32_t rows1 = min(kActRows, 128u - off1), rows2 = kActRows - rows1;
            const bool v1 = blk1 < tiles_m128, v2 = rows2 > 0 && (blk1 + 1) < tiles_m128;
            const uint8_t *act1 = args.A + (size_t)blk1 * args.a_kblocks_total * kI8BlockBytes + off1 * 128u;
            const uint8_t *act2 = args.A + (size_t)(blk1 + 1) * args.a_kblocks_total * kI8BlockBytes;
            const uint32_t act_tx = (v1 ? rows1 * 128u : 0u) + (v2 ? rows2 * 128u : 0u);
            for (uint32_t g = 0; g < ngroups && ok; ++g, ++Gc) {
                const uint32_t gs = Gc % NG;
                if (!TQT_PTIMED(0, ptx::mbar_wait(BAR(kGroupDone + gs), ((Gc / NG) & 1u) ^ 1u, sAbort, args.fault,
                                                          kFaultProducerWait))) {
                    ok = false;
                    break;
                }
                // every group runs both of its steps so that all barriers advance in lockstep; when the tile
                // has an odd number of K steps the last one is empty (no bytes, no MMAs)
                {
                    const uint32_t h = ph;
                    const uint32_t s = gs * 2 + h, ks = g * 2 + h;
                    if (ks >= ksteps) {
                        if (lane == 0) ptx::mbar_arrive(BAR(kFull + s));
                        __syncwarp();
                        continue;
                    }
                    if ((args.inject & 1u) && Gc == 0 && ph == 0) {   // host-made failure: see UmmaArgs::inject
                        withheld = 0;
                        continue;
                    }
                    // W4A8: every step brings its own 128-k block of nibbles; W4A16: the group's single block rides on step 0
                    const bool nib_now = nib_valid && (!kF16 || h == 0);
                    const uint32_t nib_bytes = kF16 ? 8192u : 8448u;
                    if constexpr (UNP) {
                        // boxes always count in full, cells beyond the matrices included
                        if (lane == 0) ptx::mbar_arrive_expect_tx(BAR(kFull + s), kActBytes + (nib_now ? 8192u : 0u));
                        __syncwarp();
                        if (lane == 0) {
                            if (nib_now)   // 64 bytes of nibbles = 128 k: x counts bytes of the row
                                ptx::tma_load_2d(ptx::smem_u32(sNib + gs * Cfg::kNibGroupBytes + (kF16 ? 0u : h * 8192u)), &maps->b,
                                                 (int32_t)((kF16 ? g : ks) * 64u), (int32_t)(nb * 128u), BAR(kFull + s));
                        } else if (lane == 1) {
                            ptx::tma_load_2d(ptx::smem_u32(sAct + s * kActBytes), &maps->a, (int32_t)(ks * 128u), (int32_t)a0, BAR(kFull + s));
                        }
                        __syncwarp();
                        continue;
                    }
                    if (lane == 0) ptx::mbar_arrive_expect_tx(BAR(kFull + s), act_tx + (nib_now ? nib_bytes : 0u));
                    __syncwarp();
                    // three lanes issue one bulk copy each in the same instruction
                    if (lane == 0) {
                        if (nib_now)
                            ptx::bulk_g2s(ptx::smem_u32(sNib + gs * Cfg::kNibGroupBytes + (kF16 ? 0u : h * 8448u)),
                                          nib_src + (size_t)(kF16 ? g : ks) * nib_bytes, nib_bytes, BAR(kFull + s));
                    } else if (lane == 1) {
                        if (v1)
                            ptx::bulk_g2s(ptx::smem_u32(sAct + s * kActBytes), act1 + (size_t)ks * kI8BlockBytes, rows1 * 128u,
                                          BAR(kFull + s));
                    } else if (lane == 2) {
                        if (v2)
                            ptx::bulk_g2s(ptx::smem_u32(sAct + s * kActBytes + rows1 * 128u), act2 + (size_t)ks * kI8BlockBytes,
                                          rows2 * 128u, BAR(kFull + s));
                    }
                    __syncwarp();
                }
            }
        }
        if (!ok) {
            // bail-out: the copies this warp has issued must have landed before the CTA returns its shared
            // memory.  Each of the last NG groups owns one stage of this warp: wait (bounded) for its barrier.
            const uint32_t pending = Gc < NG ? Gc : NG;
            for (uint32_t i = 0; i < pending; ++i) {
                const uint32_t G = Gc - 1u - i;
                if (G == withheld) continue;
                const uint32_t s = (G % NG) * 2u + ph, phs = (G / NG) & 1u;
                const long long t0 = clock64();
                while (!ptx::mbar_try_wait(BAR(kFull + s), phs)) {
                    if (clock64() - t0 > ptx::wait_limit(sAbort)) {
                        if (args.fault) atomicCAS(args.fault, 0u, (unsigned)kFaultDrainWait);
                        break;
                    }
                }
            }
        }
    } else if (warp == 1 || warp == kIssuer1Warp) {
        // ===================== MMA issuers (one thread each, leader CTA; the rest of the warps idle) ==========
        // A group of eight MMAs occupies the tensor pipe for ~820 cycles (M256 x N192 x K32: 102.5 each).  One thread
        // that waits for the operands, fences, issues the eight MMAs and commits needs longer than that per group
        // (measured with clock64 stamps: wait + fence 150-450 cycles even on a barrier that completed long ago, the
        // eight issues 500-880 because they block once the pipe's queue is full, the commit 120-240) and the queue
        // does not hold enough MMAs to cover its other work, so the pipe ran dry for a part of every group.  CTA pairs
        // therefore issue from two threads in different SM sub-partitions that take the groups in turn: while one
        // commits and waits for its next group's operands the other is already issuing.  The turn is handed over through
        // a counter in shared memory, so the MMAs enter the pipe in group order (the first MMA of a tile overwrites the
        // accumulator, and floating-point accumulation stays in one order).  Each thread commits its own groups; the
        // accumulator-full barrier takes one commit from each.
        const uint32_t who = warp == 1 ? 0u : 1u;
        if (rank == 0 && lane == 0 && (kDual || who == 0u)) {
            const uint32_t idesc = kF16 ? ptx::make_idesc(1u, 0u, 0u, PAIR ? 256 : 128, mt)
                                        : ptx::make_idesc(2u, 1u, 1u, PAIR ? 256 : 128, mt);
            const uint64_t desc0 = ptx::make_desc_k_sw128(ptx::smem_u32(sAct));
            const uint32_t desc0_lo = (uint32_t)desc0, desc0_hi = (uint32_t)(desc0 >> 32);
            constexpr uint32_t kDescStage = kActBytes >> 4;   // descriptor address field counts 16-byte units
            constexpr uint32_t kStride = kDual ? 2u : 1u;     // this thread takes every kStride-th group
            const uint32_t peer_tmem_full = (PAIR && kDual) ? ptx::mapa(BAR(kTmemFull), 1) : 0u;
            uint32_t ti = 0, G0 = 0;   // G0 = groups of the tiles before this one
            uint32_t gs = kDual ? who : 0u;   // this thread's current group modulo NG, carried along
            bool ok = true;
            // Whether this thread's next group's operands are ready is tested one group ahead: the test is issued after the
            // current group's MMAs and its result read after the commit, so its latency (~150-250 cycles even on a phase
            // that completed long ago) is off the issuing thread's critical path.  A phase seen complete stays
            // complete: the converters can only arrive for it again after the MMAs that are about to be issued.
            bool ready = false;
            for (uint32_t t = pair; t < num_tiles && ok; t += npairs, ++ti, G0 += ngroups) {
                const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
                if (!TQT_PTIMED(0, ptx::mbar_wait(BAR(kTmemEmpty + acc), pha ^ 1u, sAbort, args.fault, kFaultMmaWaitTmem))) {
                    ok = false;
                    break;
                }
                const uint32_t d_tmem = tmem_base + acc * mt;
                const uint32_t g_first = kDual ? ((G0 & 1u) ^ who) : 0u;
                if (g_first >= ngroups) {
                    // a one-group tile that is the other thread's: only keep the accumulator-full barrier's count
                    // (the wait above paces this: the barrier's previous phase has been consumed)
                    if constexpr (PAIR && kDual) {
                        ptx::mbar_arrive(BAR(kTmemFull + acc));
                        ptx::mbar_arrive_cluster(peer_tmem_full + acc * 8u);
                    }
                    continue;
                }
                for (uint32_t g = g_first; g < ngroups; g += kStride) {
                    const uint32_t Gc = G0 + g, slot = Gc & 1u;
                    const bool tr = trace && who == 0u && Gc < 64u;   // diagnostic trace: first 64 groups of pair 0
                    if (tr) trace[Gc * 8 + 0] = clock64();
                    // all converter warps of both steps have written operand stages 2 slot, 2 slot + 1 (which also
                    // means the activation rows of the two shared-memory stages have landed, in both CTAs of a pair)
                    if (!ready && !TQT_PTIMED(1, ptx::mbar_wait(BAR(kConvFull + slot), (Gc >> 1) & 1u, sAbort, args.fault,
                                                                kFaultMmaWaitFull, hint_mma))) {
                        ok = false;
                        break;
                    }
                    if (tr) trace[Gc * 8 + 4] = trace[Gc * 8 + 5] = clock64();
                    ptx::tc_fence_after();
                    if constexpr (kDual) {
                        // this thread's turn: the other one has issued group Gc - 1
                        if (*sIssued != Gc) {
                            const long long t0 = clock64();
                            while (*sIssued != Gc) {
                                if (*sAbort || clock64() - t0 > ptx::wait_limit(sAbort)) {
                                    if (!*sAbort && args.fault) atomicCAS(args.fault, 0u, (unsigned)kFaultMmaWaitFull);
                                    *sAbort = 1;
                                    ok = false;
                                    break;
                                }
                            }
                            if (!ok) break;
                        }
                    }
                    if (tr) trace[Gc * 8 + 1] = clock64();
                    const uint32_t two = (ksteps - g * 2u) >= 2u ? 1u : 0u;
                    const uint32_t dlo = desc0_lo + gs * 2u * kDescStage, a_t = tmem_a + slot * 64u;
                    if constexpr (kF16) {
                        if constexpr (PAIR) ptx::mma_f16_ts_pair_group8(d_tmem, a_t, dlo, desc0_hi, kDescStage, idesc, g, two);
                        else ptx::mma_f16_ts_group8(d_tmem, a_t, dlo, desc0_hi, kDescStage, idesc, g, two);
                    } else {
                        if constexpr (PAIR) ptx::mma_i8_ts_pair_group8(d_tmem, a_t, dlo, desc0_hi, kDescStage, idesc, g, two);
                        else ptx::mma_i8_ts_group8(d_tmem, a_t, dlo, desc0_hi, kDescStage, idesc, g, two);
                    }
                    if constexpr (kDual) {
                        asm volatile("" ::: "memory");
                        *sIssued = Gc + 1u;
                    }
                    if (tr) trace[Gc * 8 + 2] = clock64();
                    // this thread's next group's barrier (same parity formula with Gc + kStride): tested between the
                    // MMAs and the commit, read at the top of the next iteration
                    const uint32_t Gn = Gc + kStride;
                    const bool next_ready = ptx::mbar_test_wait(BAR(kConvFull + (Gn & 1u)), (Gn >> 1) & 1u);
                    const bool last_mine = g + kStride >= ngroups;
                    if constexpr (PAIR) {
                        ptx::tc_commit_pair(BAR(kGroupDone + gs), 3);
                        if (last_mine) ptx::tc_commit_pair(BAR(kTmemFull + acc), 3);
                    } else {
                        ptx::tc_commit(BAR(kGroupDone + gs));
                        if (last_mine) ptx::tc_commit(BAR(kTmemFull + acc));
                    }
                    if (tr) trace[Gc * 8 + 3] = clock64();
                    ready = next_ready;
                    gs += kStride;
                    if (gs >= NG) gs -= NG;
                }
            }
        }
        __syncwarp();
    } else if (warp >= 10) {
        // ===================== converters (warps 10 ..): int4 -> MMA operand type, into tensor memory ========
        // Sets of four warps, one per tensor-memory lane quadrant.  The K steps are numbered through the whole launch
        // (2 * group + step) and set c takes the steps c, c + sets, ...: with two sets (packed W4A8) set 0 has step 0 of
        // every group and set 1 step 1; with three every set meets both.  A step is fetched and expanded into registers
        // before the warp waits for its tensor-memory stage to be free; the store is then announced at once (deferring the
        // announcement past the next step's expansion, to hide the store latency, would put that expansion on the MMAs'
        // critical path).
        const uint32_t quad = warp & 3u, cset = (warp - 10u) >> 2;
        const uint32_t row = quad * 32u + lane;
        const uint32_t swz_in = (row >> 1) & 3u;
        const uint32_t conv_full_leader = PAIR ? ptx::mapa(BAR(kConvFull), 0) : 0u;   // + 8 * group slot
        const bool word_scale = kF16 && (args.bl & 7u) == 0u;   // W4A16: one scale per 8-k word (bl a multiple of 8)
        const int bl_shift = (kF16 && args.bl && (args.bl & (args.bl - 1u)) == 0u) ? (int)__ffs((int)args.bl) - 1 : -1;
        // the last window of a row may read up to 7 entries past the row's k / bl scales: only when that stays
        // inside the row stride (ldsb a multiple of 8 covers it) and the base is 16-byte aligned
        const bool sc_vec = kF16 && bl_shift >= 3 && (args.ldsb & 7u) == 0u && (reinterpret_cast<uintptr_t>(args.scale_blk) & 15u) == 0u;
        auto announce = [&](uint32_t ts) {   // ts = operand stage; its group slot's barrier counts both steps
            ptx::tmem_wait_st();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0)
                    ptx::mbar_arrive(BAR(kConvFull + (ts >> 1)));
                else
                    ptx::mbar_arrive_cluster(conv_full_leader + (ts >> 1) * 8u);
            }
        };
        uint32_t Gc = 0, ti = 0;
        bool ok = true;
        // A wait on an mbarrier costs 150-300 cycles even when its phase completed long ago, and a converter warp has two
        // per step (its shared-memory stage has landed; the MMAs that read its tensor-memory stage are done).  Both are
        // therefore tested ahead of their use, so that the test's latency runs under the expansion: the next step's
        // stage at the end of the current step, the tensor-memory stage at the top of the step.  A phase seen complete
        // stays complete until this warp's own announcement lets the pipeline advance.
        bool full_ready = false;
        uint32_t gs = 0, phs = 0;   // Gc % NG and (Gc / NG) & 1, carried along instead of divided out every step
        uint32_t own = cset;        // the next K step this warp expands: steps are numbered 2 Gc + h through the launch
        for (uint32_t t = pair; t < num_tiles && ok; t += npairs, ++ti) {
            uint32_t tm_unused, tn;
            tile_coords(t, tmc, tnc, args.band_m, tm_unused, tn);
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            const size_t nrow = (size_t)(PAIR ? tn * 2 + rank : tn) * 128u + row;
            int32_t rsum = 0;
            // W4A16 block scales: scale_b[nrow, k / bl].  When bl is a power of two >= 8 and the rows of scale_b
            // are 16-byte aligned, one 128-bit load fetches the eight scales that cover the next 8 * bl values of
            // k (four K steps at bl = 32) and stays cached in registers; otherwise eight scalar loads per step.
            uint4 sc_win = make_uint4(0, 0, 0, 0);
            uint32_t sc_base = 0xffffffffu;
            auto load_scales = [&](uint32_t step, bool valid, __half(&sc)[8]) {
                const uint32_t kb0 = step * 64u;
                const bool n_ok = nrow < args.n;
                const __half *srow = args.scale_blk + nrow * args.ldsb;
                if (sc_vec) {
                    const uint32_t sh = (uint32_t)bl_shift & 31u;   // sc_vec implies bl_shift >= 3
                    const uint32_t i0 = kb0 >> sh;
                    const uint32_t base = i0 & ~7u;
                    if (base != sc_base) {
                        sc_win = (valid && n_ok) ? __ldg(reinterpret_cast<const uint4 *>(srow + base)) : make_uint4(0, 0, 0, 0);
                        sc_base = base;
                    }
                    const unsigned long long lo = ((unsigned long long)sc_win.y << 32) | sc_win.x;
                    const unsigned long long hi = ((unsigned long long)sc_win.w << 32) | sc_win.z;
#pragma unroll
                    for (uint32_t w = 0; w < 8; ++w) {
                        const uint32_t k0 = kb0 + w * 8u;
                        const uint32_t idx = (k0 >> sh) - base;   // 0..7 (entries past k / bl are never selected for k0 < k)
                        const unsigned long long v = (idx & 4u) ? hi : lo;
                        const unsigned short bits = (unsigned short)(v >> (16u * (idx & 3u)));
                        sc[w] = (valid && k0 < args.k) ? __ushort_as_half(bits) : __ushort_as_half((unsigned short)0);
                    }
                } else {
#pragma unroll
                    for (uint32_t w = 0; w < 8; ++w) {
                        const uint32_t k0 = kb0 + w * 8u;
                        const uint32_t bi = bl_shift >= 0 ? (k0 >> ((uint32_t)bl_shift & 31u)) : (k0 / args.bl);
                        sc[w] = (valid && word_scale && n_ok && k0 < args.k) ? __ldg(srow + bi) : __ushort_as_half((unsigned short)0);
                    }
                }
            };
            for (uint32_t g = 0; g < ngroups && ok; ++g, ++Gc, gs = gs + 1u == NG ? 0u : gs + 1u, phs ^= (gs == 0u ? 1u : 0u)) {
                if ((own >> 1) != Gc) continue;   // neither step of this group is this set's
                const uint32_t h = own & 1u, s = gs * 2 + h, ts = (Gc & 1u) * 2 + h;
                own += kSets;
                // the same for the group two back (its MMAs free this tensor-memory stage) and for this warp's next step
                const uint32_t gs_p = gs >= 2u ? gs - 2u : gs + NG - 2u, ph_p = gs >= 2u ? phs : phs ^ 1u;
                const uint32_t h_n = own & 1u, gs_n1 = gs + (own >> 1) - Gc;   // one or two groups on
                const uint32_t gs_n = gs_n1 >= NG ? gs_n1 - NG : gs_n1, ph_n = gs_n1 >= NG ? phs ^ 1u : phs;
                const bool step_valid = g * 2 + h < ksteps;
                long long *ctr = (trace && lane == 0 && quad == 2 && cset < 2u && h == cset && Gc < 64u) ? trace + 512 + cset * 512 + Gc * 4 : nullptr;
                if (trace_peer && lane == 0 && quad == 2 && cset == 0 && Gc < 64u) ctr = trace_peer + Gc * 4;
                if (ctr) ctr[0] = clock64();
                // W4A16: the block scales of a step (one per 8-k word) do not depend on the barriers; they were
                // requested during the previous step of this warp (or are requested here, for a tile's first step)
                __half sc8[8];
                if constexpr (kF16) load_scales(g * 2 + h, step_valid, sc8);
                const bool done_ready = Gc < 2u || ptx::mbar_test_wait(BAR(kGroupDone + gs_p), ph_p);
                if (!full_ready && !TQT_PTIMED(0, ptx::mbar_wait(BAR(kFull + s), phs, sAbort, args.fault, kFaultConverterWait))) {
                    ok = false;
                    break;
                }
                if (kF16 && h == 1) {   // the group's nibbles arrived with step 0
                    if (!TQT_PTIMED(0, ptx::mbar_wait(BAR(kFull + gs * 2), phs, sAbort, args.fault, kFaultConverterWait))) {
                        ok = false;
                        break;
                    }
                }
                if (!step_valid) {   // empty step of an odd tile: keep the barrier in step, nothing to convert
                    // like a real step, it may only be announced once the group that used this operand stage
                    // before is done: otherwise two announcements could fall into one phase of the barrier
                    full_ready = false;   // the next step's stage has not been tested
                    if (Gc >= 2u) {
                        if (!TQT_PTIMED(2, ptx::mbar_wait(BAR(kGroupDone + gs_p), ph_p, sAbort, args.fault,
                                                                  kFaultConverterWait))) {
                            ok = false;
                            break;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) {
                        if (rank == 0)
                            ptx::mbar_arrive(BAR(kConvFull + (ts >> 1)));
                        else
                            ptx::mbar_arrive_cluster(conv_full_leader + (ts >> 1) * 8u);
                    }
                    continue;
                }
                uint32_t regs[32];
                if constexpr (!kF16 && UNP) {
                    // Row-major nibbles: word j of segment seg holds k = 32 seg + 8 j .. + 7, low nibble first, as u = q + 8.
                    // L / H = the even / odd k as bytes 16 u; two byte permutes put them in k order and 16 u - 128 = 16 q
                    // is an exclusive-or with 0x80 (no carries: 16 u <= 240).  sum u = dp4a of the nibble bytes with ones.
                    const uint8_t *nrowp = sNib + gs * Cfg::kNibGroupBytes + h * 8192u + row * 64u;
                    const uint32_t kv = min(128u, args.k - (g * 2u + h) * 128u);   // k values of this step that exist
                    int32_t usum = 0;
#pragma unroll
                    for (uint32_t seg = 0; seg < 4; ++seg) {
                        const uint4 w = *reinterpret_cast<const uint4 *>(nrowp + ((seg ^ swz_in) << 4));
                        uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            if (kv < 128u) {   // the ragged last step: nibbles beyond k (zero bytes from the copy) become u = 8, q = 0
                                const uint32_t k0 = seg * 32u + j * 8u;
                                const uint32_t nv = kv > k0 ? min(8u, kv - k0) : 0u;
                                const uint32_t mask = nv >= 8u ? 0xffffffffu : ((1u << (4u * nv)) - 1u);
                                ws[j] = (ws[j] & mask) | (0x88888888u & ~mask);
                            }
                            const uint32_t lo = (ws[j] << 4) & 0xF0F0F0F0u, hi = ws[j] & 0xF0F0F0F0u;
                            regs[seg * 8 + 2 * j] = __byte_perm(lo, hi, 0x5140) ^ 0x80808080u;       // k = 32 seg + 8 j .. + 3
                            regs[seg * 8 + 2 * j + 1] = __byte_perm(lo, hi, 0x7362) ^ 0x80808080u;   // k = 32 seg + 8 j + 4 .. + 7
                            usum = __dp4a((int)((lo >> 4) + (hi >> 4)), 0x01010101, usum);
                        }
                    }
                    rsum += usum - 8 * 128;   // sum q = sum u - 8 per nibble (the masked ones hold u = 8)
                } else if constexpr (!kF16) {
                    const uint8_t *blk = sNib + gs * Cfg::kNibGroupBytes + h * 8448u;
                    const uint8_t *nrowp = blk + row * 64u;
#pragma unroll
                    for (uint32_t seg = 0; seg < 4; ++seg) {
                        const uint4 w = *reinterpret_cast<const uint4 *>(nrowp + ((seg ^ swz_in) << 4));
                        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            regs[seg * 8 + j] = (ws[j] << 4) & 0xF0F0F0F0u;       // k = 32 seg + 4 j .. + 3
                            regs[seg * 8 + 4 + j] = ws[j] & 0xF0F0F0F0u;          // k = 32 seg + 16 + 4 j .. + 3
                        }
                    }
                    rsum += (int32_t) reinterpret_cast<const int16_t *>(blk + kI4NibBytes)[row];
                } else {
                    // 64 k of this step = segments 2h, 2h+1 of the 128-k block; each word holds 8 k as nibbles
                    // (k0,k2,k4,k6,k1,k3,k5,k7) so that (w >> 4t) & 0x000F000F = (k2t, k2t+1).  nibble u = q + 8;
                    // 0x6400 | u is the f16 1024 + u, so q = that - 1032 exactly, and q * scale is rounded once.
                    const uint8_t *nrowp = sNib + gs * Cfg::kNibGroupBytes + row * 64u;
                    const bool n_ok = nrow < args.n;
                    const uint32_t kbase = (g * 2 + h) * 64u;
                    const __half *srow = args.scale_blk + nrow * args.ldsb;
                    const __half2 k1032 = __float2half2_rn(1032.0f);
                    if (word_scale) {
                        // common case (block length a multiple of 8): branch-free, one scale per 8-k word
#pragma unroll
                        for (uint32_t sg = 0; sg < 2; ++sg) {
                            const uint4 w4 = *reinterpret_cast<const uint4 *>(nrowp + (((2 * h + sg) ^ swz_in) << 4));
                            const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                            for (uint32_t wi = 0; wi < 4; ++wi) {
                                const __half2 sc2 = __half2half2(sc8[sg * 4 + wi]);
#pragma unroll
                                for (uint32_t tt = 0; tt < 4; ++tt) {
                                    const uint32_t bits = nib_pair<UNP>(ws[wi], tt) | 0x64006400u;
                                    const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&bits), k1032), sc2);
                                    regs[sg * 16 + wi * 4 + tt] = *reinterpret_cast<const uint32_t *>(&v);
                                }
                            }
                        }
                    } else {
                        // block lengths 2, 4, 6, ...: one scale per pair of k (a pair never straddles blocks)
#pragma unroll
                        for (uint32_t sg = 0; sg < 2; ++sg) {
                            const uint4 w4 = *reinterpret_cast<const uint4 *>(nrowp + (((2 * h + sg) ^ swz_in) << 4));
                            const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                            for (uint32_t wi = 0; wi < 4; ++wi) {
#pragma unroll
                                for (uint32_t tt = 0; tt < 4; ++tt) {
                                    const uint32_t kk = kbase + sg * 32u + wi * 8u + 2 * tt;
                                    const __half2 sc2 = (n_ok && kk < args.k) ? __half2half2(__ldg(srow + kk / args.bl))
                                                                              : __float2half2_rn(0.0f);
                                    const uint32_t bits = nib_pair<UNP>(ws[wi], tt) | 0x64006400u;
                                    const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&bits), k1032), sc2);
                                    regs[sg * 16 + wi * 4 + tt] = *reinterpret_cast<const uint32_t *>(&v);
                                }
                            }
                        }
                    }
                }
                if (ctr) ctr[1] = clock64();
                full_ready = ptx::mbar_test_wait(BAR(kFull + gs_n * 2u + h_n), ph_n);
                // the MMAs of the group two groups back read this tensor-memory stage: they must be done
                if (!done_ready) {
                    if (!TQT_PTIMED(2, ptx::mbar_wait(BAR(kGroupDone + gs_p), ph_p, sAbort, args.fault,
                                                              kFaultConverterWait, hint_conv))) {
                        ok = false;
                        break;
                    }
                }
                __syncwarp();
                if (ctr) ctr[2] = clock64();
                ptx::tmem_st_32x32b_x32(tmem_a + ts * 32u + ((quad * 32u) << 16), regs);
                announce(ts);
                if (ctr) ctr[3] = clock64();
            }
            if (!ok) break;
            if constexpr (!kF16) {
                if (!TQT_PTIMED(1, ptx::mbar_wait(BAR(kRsumEmpty + acc), pha ^ 1u, sAbort, args.fault, kFaultConverterWait))) {
                    ok = false;
                    break;
                }
                sRsum[(acc * kSets + cset) * 128u + row] = rsum;
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(BAR(kRsumFull + acc));
            }
        }
        conv_failed = !ok;
    }

    if (run_roles && warp >= 2 && warp < 18 && !conv_failed) {
        // ===================== epilogue (8 warps per CTA): D^T, lane = output channel ==================
        // The converter warps, idle once the last K step of their last tile is in tensor memory, come here
        // too and take the upper half of that tile's column strips: the epilogue of the last tile overlaps no
        // mainloop (it is the whole tail of a launch, and half of a single-wave launch), so it is spread over
        // sixteen warps instead of eight.  Warp w and helper warp w + 8 share a lane quadrant and a column half.
        // Per-channel values (scale_b, bias, row sum) are per-thread constants; the per-row values
        // (scale_a, zero_point_a) of a 32-column strip are loaded one per lane and broadcast with
        // shuffles, so the epilogue makes no shared-memory reads that would queue behind the MMA's.
        const bool helper = warp >= 10;
        const uint32_t ew = helper ? warp - 8u : warp;
        const uint32_t quad = ew & 3u, half = (ew - 2u) >> 2;
        const uint32_t row = quad * 32u + lane;             // weight row inside this CTA's block
        constexpr bool replicate = REPL;
        const bool has_c = args.C != nullptr, has_bias = args.bias != nullptr;
        const uint32_t my_tiles = pair < num_tiles ? (num_tiles - pair + npairs - 1) / npairs : 0u;
        uint32_t ti = helper ? (my_tiles ? my_tiles - 1u : 0u) : 0u;   // helpers: the last tile only
        bool ok = true;
        for (uint32_t t = pair + ti * npairs; t < num_tiles && ok; t += npairs, ++ti) {
            const bool last = ti + 1u == my_tiles;
            uint32_t tm, tn;
            tile_coords(t, tmc, tnc, args.band_m, tm, tn);
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            const uint32_t n = (PAIR ? tn * 2 + rank : tn) * 128u + row;
            const bool n_ok = n < args.n;
            const uint32_t hcols = mt / 2u;   // accumulator columns (activation rows) of this warp's half
            const uint32_t m0 = tm * mt + half * hcols;
            const uint32_t mcols = args.m > m0 ? min(hcols, args.m - m0) : 0u;
            float sb = 0.0f;
            if constexpr (!kF16) sb = n_ok ? args.scale_b[n] : 0.0f;
            const float bv = (n_ok && args.bias) ? TdTraits<TD>::load(args.bias, n) : 0.0f;
            if (!(helper ? ptx::mbar_wait(BAR(kTmemFull + acc), pha, sAbort, args.fault, kFaultEpilogueWait)
                         : TQT_PTIMED(0, ptx::mbar_wait(BAR(kTmemFull + acc), pha, sAbort, args.fault, kFaultEpilogueWait)))) {
                ok = false;
                break;
            }
            int32_t rs = 0;
            if constexpr (!kF16) {
                if (!(helper ? ptx::mbar_wait(BAR(kRsumFull + acc), pha, sAbort, args.fault, kFaultEpilogueWait)
                             : TQT_PTIMED(1, ptx::mbar_wait(BAR(kRsumFull + acc), pha, sAbort, args.fault, kFaultEpilogueWait)))) {
                    ok = false;
                    break;
                }
                rs = 0;
#pragma unroll
                for (uint32_t c = 0; c < kSets; ++c) rs += sRsum[(acc * kSets + c) * 128u + row];
            }
            ptx::tc_fence_after();
            const uint32_t t_addr = tmem_base + acc * mt + half * hcols + ((quad * 32u) << 16);
            const uint32_t nchunks = (mcols + 31u) / 32u;
            // the last tile's strips are split between this warp and its helper
            const uint32_t split = (nchunks + 1u) / 2u;
            const uint32_t ch_begin = helper ? split : 0u, ch_end = (last && !helper) ? split : nchunks;
            for (uint32_t ch = ch_begin; ch < ch_end; ++ch) {
                const uint32_t c0 = ch * 32u;
                const uint32_t nvalid = min(32u, mcols - c0);
                float sa_l = 0.0f;
                int32_t zp_l = 0;
                if constexpr (!kF16) {
                    if constexpr (FUSEQ) {   // written by this launch's phase 0: coherent loads
                        sa_l = lane < nvalid ? args.scale_a[m0 + c0 + lane] : 0.0f;
                        zp_l = lane < nvalid ? args.zp_a[m0 + c0 + lane] : 0;
                    } else {
                        sa_l = lane < nvalid ? __ldg(args.scale_a + m0 + c0 + lane) : 0.0f;
                        zp_l = lane < nvalid ? __ldg(args.zp_a + m0 + c0 + lane) : 0;
                    }
                }
                __syncwarp();
                OutT *dcol = static_cast<OutT *>(args.D) + (size_t)(m0 + c0) * args.ldd + n;
                // Eight columns at a time in a rolled loop: the strip's code is a quarter of the fully unrolled
                // form.  The kernel's warps share one instruction cache, and the MMA issuer, whose instruction
                // stream is the bottleneck of the mainloop, slowed down whenever the epilogue's code grew.
#pragma unroll 1
                for (uint32_t q8 = 0; q8 < 32u && q8 < nvalid; q8 += 8u) {
                    uint32_t r[8];
                    const long long tl0 = TQT_DIAG_ON(args) ? clock64() : 0;
                    ptx::tmem_ld_32x32b_x8(t_addr + c0 + q8, r);
                    ptx::tmem_wait_ld();
                    if (TQT_DIAG_ON(args)) wcyc[2] += clock64() - tl0;
                    constexpr bool kRepl = replicate;
#pragma unroll
                    for (uint32_t jj = 0; jj < 8; ++jj) {
                        const uint32_t j = q8 + jj;
                        float v;
                        if constexpr (!kF16) {
                            const float sa = __shfl_sync(0xffffffffu, sa_l, j);
                            const int32_t zp = __shfl_sync(0xffffffffu, zp_l, j);
                            // operands were 16*q: the accumulator is an exact multiple of 16
                            const int32_t a = (((int32_t)r[jj]) >> 4) - zp * rs;
                            v = __fmul_rn(__fmul_rn(__int2float_rn(a), sa), sb);
                        } else {
                            v = __uint_as_float(r[jj]);
                        }
                        // branch-free per element: selects and a predicated load / store instead of three branches
                        const bool live = n_ok && j < nvalid;
                        float cv = 0.0f;
                        if (has_c && live) cv = TdTraits<TD>::load(args.C, (size_t)(m0 + c0 + j) * args.ldc + n);
                        v = has_c ? __fadd_rn(v, cv) : v;
                        v = has_bias ? __fadd_rn(v, bv) : v;
                        v = fminf(fmaxf(v, args.cmin_f), args.cmax_f);
                        const OutT o = cvt_out<OutT>(v);
                        OutT *dst = dcol + (size_t)j * args.ldd;
                        if (live) *dst = o;   // the warp writes 32 consecutive channels
                        if constexpr (kRepl) {
                            if (live) {
                                for (uint32_t rp = 0; rp < args.n_replicas; ++rp)
                                    *reinterpret_cast<OutT *>(reinterpret_cast<char *>(dst) + args.replica_delta[rp]) = o;
                            }
                        }
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0 && !helper) {   // nobody waits for these after the last tile; helpers never arrive
                if (rank == 0)
                    ptx::mbar_arrive(BAR(kTmemEmpty + acc));
                else
                    ptx::mbar_arrive_cluster(ptx::mapa(BAR(kTmemEmpty + acc), 0));
                if constexpr (!kF16) ptx::mbar_arrive(BAR(kRsumEmpty + acc));
            }
        }
    }

    if (TQT_DIAG_ON(args) && !(args.inject & 64u) && lane == 0 && (warp == 0 || warp == 1 || warp == 2 || warp == 10)) {
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

template <TsKind KD, Dtype TD, bool WIDE, bool REPL>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(ts_threads<KD>(), 1) gemm_ts_pair_kernel(const UmmaArgs args)
{
    ts_body<KD, TD, true, WIDE, REPL>(args);
}

// W4A8 with the activation quantiser in front of the mainloop (one launch; needs every CTA resident: cooperative launch).
template <Dtype TD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(ts_threads<TsKind::W4A8>(), 1) gemm_ts_pair_fusedq_kernel(const UmmaArgs args)
{
    ts_body<TsKind::W4A8, TD, true, false, false, false, true>(args);
}

// Row-major operands: the tensor maps travel as a kernel parameter.
template <TsKind KD, Dtype TD>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(ts_threads<KD, true>(), 1)
    gemm_ts_pair_tma_kernel(const UmmaArgs args, const __grid_constant__ TmaOperands maps)
{
    ts_body<KD, TD, true, false, false, true>(args, &maps);
}

// Same kernel on one CTA (cta_group::1): the CTA stages all 192 activation rows itself.
template <TsKind KD, Dtype TD>
__global__ void __launch_bounds__(ts_threads<KD>(), 1) gemm_ts_kernel(const UmmaArgs args)
{
    ts_body<KD, TD, false, false, false>(args);
}

// ---- host side ------------------------------------------------------------------------------------------
template <class Kern, class... Extra>
static Result launch_grid(Kern kern, const UmmaArgs &a, uint32_t num_tiles, bool pair, uint32_t threads, uint32_t smem,
                          cudaStream_t st, bool *attr_set, const Extra &...extra)
{
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
        attr_set[dev] = true;
    }
    uint32_t sms = (uint32_t)sm_count_cached();
    static const int sm_limit = [] {   // diagnostic: run on fewer SMs (TQT_B200_SM_LIMIT), e.g. to separate per-SM from shared limits
        const char *e = std::getenv("TQT_B200_SM_LIMIT");
        return e ? std::atoi(e) : 0;
    }();
    if (sm_limit > 1 && (uint32_t)sm_limit < sms) sms = (uint32_t)sm_limit;
    uint32_t grid;
    if (pair) {
        const uint32_t max_pairs = sms / 2;
        grid = 2 * (num_tiles < max_pairs ? num_tiles : max_pairs);
    } else {
        grid = num_tiles < sms ? num_tiles : sms;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;   // only kernels that execute griddepcontrol.wait set pdl
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a, extra...);
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

// Pair tiles of an int8 x int8 launch, as the number of CTA pairs worth launching: a problem with so few tiles that
// twice as many pairs still fit the GPU runs as half tiles (see I8Work), which the kernel derives from its grid size.
static uint32_t i8_launch_items(const UmmaArgs &a, bool b_whole)
{
    const uint32_t tiles = (((a.m + 127) / 128 + 1) / 2) * ((((a.n + 127) / 128) + 1) / 2);
    const uint32_t max_pairs = (uint32_t)sm_count_cached() / 2;
    return (!b_whole && 2u * tiles <= max_pairs) ? 2u * tiles : tiles;
}

Result pair_gemm_i8_dxcx(const UmmaArgs &a, Dtype td, cudaStream_t st)
{
    const uint32_t tiles = i8_launch_items(a, false);
    static bool set_f32[64] = {false}, set_f16[64] = {false};
    if (td == Dtype::F32)
        return launch_grid(gemm_pair_i8_kernel<EpiKind::DxCx, Dtype::F32>, a, tiles, true, kI8Threads, kI8Smem, st, set_f32);
    return launch_grid(gemm_pair_i8_kernel<EpiKind::DxCx, Dtype::F16>, a, tiles, true, kI8Threads, kI8Smem, st, set_f16);
}

Result pair_gemm_i8_rows(const UmmaArgs &a, cudaStream_t st)
{
    const uint32_t tiles = i8_launch_items(a, false);
    static bool set_row[64] = {false};
    return launch_grid(gemm_pair_i8_kernel<EpiKind::Req8Row>, a, tiles, true, kI8Threads, kI8Smem, st, set_row);
}

Result pair_gemm_i8(const UmmaArgs &a, bool requant, cudaStream_t st)
{
    const uint32_t tiles = i8_launch_items(a, false);
    static bool set_s32[64] = {false}, set_req[64] = {false};
    note_kernel(kKernelPairBlocks);
    if (requant) return launch_grid(gemm_pair_i8_kernel<EpiKind::Req8>, a, tiles, true, kI8Threads, kI8Smem, st, set_req);
    return launch_grid(gemm_pair_i8_kernel<EpiKind::S32>, a, tiles, true, kI8Threads, kI8Smem, st, set_s32);
}

// ---- tensor maps for row-major operands -------------------------------------------------------------------
// cuTensorMapEncodeTiled is a driver entry point: it is looked up through the runtime, so the library links no driver
// library and still loads on machines without one.
using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn()
{
    static const EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// int8 matrix [outer, inner] with `inner` contiguous and rows `stride` bytes apart, read in boxes of 128 x 128 bytes
// with the 128-byte swizzle.  The base and the stride must be multiples of 16 bytes.
// A byte matrix [outer, inner bytes] with rows `stride` bytes apart, read in boxes of box_inner bytes x box_outer rows;
// box_inner 128 takes the 128-byte swizzle, 64 the 64-byte one.
static bool encode_byte_map(TmaDesc *out, const void *base, size_t inner, size_t outer, size_t stride, uint32_t box_inner,
                            uint32_t box_outer)
{
    static_assert(sizeof(CUtensorMap) == sizeof(TmaDesc), "tensor map size");
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn || (reinterpret_cast<uintptr_t>(base) & 15) || (stride & 15) || stride == 0 || inner == 0 || outer == 0 ||
        inner > 0xffffffffull || outer > 0xffffffffull)
        return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {stride};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    return fn(reinterpret_cast<CUtensorMap *>(out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box,
              estr, CU_TENSOR_MAP_INTERLEAVE_NONE, box_inner == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool encode_i8_map(TmaDesc *out, const void *base, size_t inner, size_t outer, size_t stride)
{
    return encode_byte_map(out, base, inner, outer, stride, 128, 128);
}

// int8 x int8 with at least one operand in the caller's row-major layout.  a.a_src / a.b_src say how each operand is
// stored; a.A / a.lda_elems (a.B / a.ldb_elems) describe the row-major ones.  kUnsupported when a matrix cannot be
// described by a tensor map (base or row stride not a multiple of 16 bytes): the caller falls back to the generic kernel.
Result pair_gemm_i8_tma(const UmmaArgs &a_in, EpiKind ek, Dtype td, size_t lda, size_t ldb, cudaStream_t st)
{
    UmmaArgs a = a_in;
    a.b_ld = ldb;
    TmaOperands maps{};
    if (a.a_src == kSrcTmaK && !encode_i8_map(&maps.a, a.A, a.k, a.m, lda)) return Result{kUnsupported, 0};
    if (a.b_src == kSrcTmaK && !encode_i8_map(&maps.b, a.B, a.k, a.n, ldb)) return Result{kUnsupported, 0};
    if (a.b_src == kSrcTmaMn && !encode_i8_map(&maps.b, a.B, a.n, a.k, ldb)) return Result{kUnsupported, 0};
    const uint32_t tiles = i8_launch_items(a, a.b_src != kSrcBlocks);
    static bool set_s32[64] = {false}, set_req[64] = {false}, set_row[64] = {false}, set_f32[64] = {false}, set_f16[64] = {false};
    note_kernel(kKernelPairTma);
    switch (ek) {
        case EpiKind::DxCx:
            if (a.b_src == kSrcTmaMn) return Result{kUnsupported, 0};   // the row sums are taken along rows of B^T
            if (td == Dtype::F32)
                return launch_grid(gemm_pair_i8_tma_kernel<EpiKind::DxCx, Dtype::F32>, a, tiles, true, kI8Threads, kI8Smem, st, set_f32, maps);
            if (td == Dtype::F16)
                return launch_grid(gemm_pair_i8_tma_kernel<EpiKind::DxCx, Dtype::F16>, a, tiles, true, kI8Threads, kI8Smem, st, set_f16, maps);
            return Result{kUnsupported, 0};
        case EpiKind::S32: return launch_grid(gemm_pair_i8_tma_kernel<EpiKind::S32>, a, tiles, true, kI8Threads, kI8Smem, st, set_s32, maps);
        case EpiKind::Req8: return launch_grid(gemm_pair_i8_tma_kernel<EpiKind::Req8>, a, tiles, true, kI8Threads, kI8Smem, st, set_req, maps);
        case EpiKind::Req8Row:
            return launch_grid(gemm_pair_i8_tma_kernel<EpiKind::Req8Row>, a, tiles, true, kI8Threads, kI8Smem, st, set_row, maps);
        default: return Result{kUnsupported, 0};
    }
}

// Unquantised f16 / bf16 GEMM: the same kernel with kind::f16 MMAs and the float epilogue.  Operands packed (128-row blocks
// of 64 elements per row) or row-major [rows, k] through tensor maps.
Result pair_gemm_f16(const UmmaArgs &a_in, bool bf16, Dtype td, bool bias_per_row, size_t lda, size_t ldb, cudaStream_t st)
{
    UmmaArgs a = a_in;
    a.in_bf16 = bf16 ? 1 : 0;
    a.bias_per_row = bias_per_row ? 1 : 0;
    TmaOperands maps{};
    if (a.a_src == kSrcTmaK && !encode_i8_map(&maps.a, a.A, (size_t)a.k * 2, a.m, lda * 2)) return Result{kUnsupported, 0};
    if (a.b_src == kSrcTmaK && !encode_i8_map(&maps.b, a.B, (size_t)a.k * 2, a.n, ldb * 2)) return Result{kUnsupported, 0};
    if (a.b_src == kSrcTmaMn && !encode_byte_map(&maps.b, a.B, (size_t)a.n * 2, a.k, ldb * 2, 128, 64)) return Result{kUnsupported, 0};
    const uint32_t tiles = i8_launch_items(a, a.b_src != kSrcBlocks);
    static bool set_f32[64] = {false}, set_f16[64] = {false}, set_bf16[64] = {false};
    note_kernel(a.a_src == kSrcBlocks && a.b_src == kSrcBlocks ? kKernelPairBlocks : kKernelPairTma);
    switch (td) {
        case Dtype::F32: return launch_grid(gemm_pair_i8_tma_kernel<EpiKind::Float, Dtype::F32>, a, tiles, true, kI8Threads, kI8Smem, st, set_f32, maps);
        case Dtype::F16: return launch_grid(gemm_pair_i8_tma_kernel<EpiKind::Float, Dtype::F16>, a, tiles, true, kI8Threads, kI8Smem, st, set_f16, maps);
        default: return launch_grid(gemm_pair_i8_tma_kernel<EpiKind::Float, Dtype::BF16>, a, tiles, true, kI8Threads, kI8Smem, st, set_bf16, maps);
    }
}

template <TsKind KD, Dtype TD>
static Result launch_ts(const UmmaArgs &a_in, bool pair, cudaStream_t st)
{
    const uint32_t nblocks = (a_in.n + 127) / 128;
    // a CTA pair may take 256 activation rows per tile when that makes the launch a single wave (every pair at
    // most one tile) and 192-row tiles would need a second one: sharded shapes such as 2048 x 1792 on 74 pairs
    UmmaArgs a = a_in;
    uint32_t mt = kTsMT;
    if (pair) {
        const uint32_t tnc = (nblocks + 1) / 2, pairs = (uint32_t)sm_count_cached() / 2;
        const uint32_t t192 = ((a.m + kTsMT - 1) / kTsMT) * tnc, t256 = ((a.m + kTsMTWide - 1) / kTsMTWide) * tnc;
        if (t192 > pairs && t256 <= pairs) mt = kTsMTWide;
    }
    a.mt = mt;
    a.pdl = pdl_enabled() ? 1 : 0;
    const uint32_t tiles = ((a.m + mt - 1) / mt) * (pair ? (nblocks + 1) / 2 : nblocks);
    static bool set_p[64] = {false}, set_s[64] = {false}, set_w[64] = {false}, set_pr[64] = {false}, set_wr[64] = {false};
    constexpr uint32_t kSmemN = TsCfg<KD, true, false>::kSmem, kSmemW = TsCfg<KD, true, true>::kSmem;
    if (a.n_replicas) {   // output replicas: CTA-pair kernels only
        if (!pair) return Result{kUnsupported, 0};
        if (mt == kTsMTWide) return launch_grid(gemm_ts_pair_kernel<KD, TD, true, true>, a, tiles, true, ts_threads<KD>(), kSmemW, st, set_wr);
        return launch_grid(gemm_ts_pair_kernel<KD, TD, false, true>, a, tiles, true, ts_threads<KD>(), kSmemN, st, set_pr);
    }
    if (pair && mt == kTsMTWide) return launch_grid(gemm_ts_pair_kernel<KD, TD, true, false>, a, tiles, true, ts_threads<KD>(), kSmemW, st, set_w);
    if (pair) return launch_grid(gemm_ts_pair_kernel<KD, TD, false, false>, a, tiles, true, ts_threads<KD>(), kSmemN, st, set_p);
    return launch_grid(gemm_ts_kernel<KD, TD>, a, tiles, false, ts_threads<KD>(), TsCfg<KD, false, false>::kSmem, st, set_s);
}

Result ts_gemm_w4a8(const UmmaArgs &a, Dtype td, bool pair, cudaStream_t st)
{
    switch (td) {
        case Dtype::F32: return launch_ts<TsKind::W4A8, Dtype::F32>(a, pair, st);
        case Dtype::F16: return launch_ts<TsKind::W4A8, Dtype::F16>(a, pair, st);
        default: return launch_ts<TsKind::W4A8, Dtype::BF16>(a, pair, st);
    }
}

Result ts_gemm_w4a16(const UmmaArgs &a, Dtype td, bool pair, cudaStream_t st)
{
    if (td == Dtype::F16) return launch_ts<TsKind::W4A16, Dtype::F16>(a, pair, st);
    return launch_ts<TsKind::W4A16, Dtype::F32>(a, pair, st);
}

// ---- W4A8 with the activation quantiser fused in front (one cooperative launch) -----------------------------------
// The grid barrier's two words live in a file-scope device array (the library allocates nothing); its address is looked
// up once per device.  Two fused launches must not run at the same time on one device (they would share the barrier):
// launches on one stream never do.
static __device__ __align__(256) unsigned int g_fused_sync[64];

static unsigned int *fused_sync_ptr()
{
    static unsigned int *cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    unsigned int *p = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
    if (!p) {
        void *addr = nullptr;
        if (cudaGetSymbolAddress(&addr, g_fused_sync) != cudaSuccess) return nullptr;
        p = static_cast<unsigned int *>(addr);
        __atomic_store_n(&cache[dev], p, __ATOMIC_RELEASE);
    }
    return p;
}

template <Dtype TD>
static Result launch_fusedq(const UmmaArgs &a, uint32_t tiles, cudaStream_t st)
{
    auto kern = gemm_ts_pair_fusedq_kernel<TD>;
    constexpr uint32_t smem = TsCfg<TsKind::W4A8, true, false>::kSmem;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
        attr_set[dev] = true;
    }
    const uint32_t max_pairs = (uint32_t)sm_count_cached() / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (tiles < max_pairs ? tiles : max_pairs), 1, 1);
    cfg.blockDim = dim3(ts_threads<TsKind::W4A8>(), 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;   // every CTA resident: the kernel's CTAs wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return Result{kUnsupported, (int)e};   // the caller falls back to two launches
    }
    note_kernel(kKernelTsFusedQuant);
    return Result{kOk, 0};
}

// kUnsupported: the caller runs the quantiser and the GEMM as two launches.
Result ts_gemm_w4a8_fusedq(const UmmaArgs &a_in, Dtype td, const void *q_in, size_t q_lda, bool q_bf16, cudaStream_t st)
{
    UmmaArgs a = a_in;
    const uint32_t nblocks = (a.n + 127) / 128, tnc = (nblocks + 1) / 2, pairs = (uint32_t)sm_count_cached() / 2;
    const uint32_t t192 = ((a.m + kTsMT - 1) / kTsMT) * tnc, t256 = ((a.m + kTsMTWide - 1) / kTsMTWide) * tnc;
    if (t192 > pairs && t256 <= pairs) return Result{kUnsupported, 0};   // the single-wave wide tile has no fused form
    if (a.n_replicas || a.k > 4096 || a.k % 16 || q_lda % 8 || (reinterpret_cast<uintptr_t>(q_in) & 15)) return Result{kUnsupported, 0};
    a.mt = kTsMT;
    a.pdl = 0;
    a.q_in = q_in;
    a.q_lda = q_lda;
    a.q_bf16 = q_bf16 ? 1 : 0;
    a.grid_sync = fused_sync_ptr();
    if (!a.grid_sync) return Result{kUnsupported, 0};
    switch (td) {
        case Dtype::F32: return launch_fusedq<Dtype::F32>(a, t192, st);
        case Dtype::F16: return launch_fusedq<Dtype::F16>(a, t192, st);
        default: return launch_fusedq<Dtype::BF16>(a, t192, st);
    }
}

// int4 weights with row-major operands (the reference's unpacked "t" kernel types): activations [m, lda] of a_elem bytes
// per element, weights as nibbles [n, ldb / 2 bytes].  kUnsupported when a tensor map cannot describe an operand.
template <TsKind KD, Dtype TD>
static Result launch_ts_tma(const UmmaArgs &a_in, const TmaOperands &maps, cudaStream_t st)
{
    UmmaArgs a = a_in;
    a.mt = kTsMT;
    a.pdl = 0;
    const uint32_t nblocks = (a.n + 127) / 128;
    const uint32_t tiles = ((a.m + kTsMT - 1) / kTsMT) * ((nblocks + 1) / 2);
    static bool set_attr[64] = {false};
    note_kernel(kKernelTsTma);
    return launch_grid(gemm_ts_pair_tma_kernel<KD, TD>, a, tiles, true, ts_threads<KD, true>(), TsCfg<KD, true, false>::kSmem, st, set_attr, maps);
}

Result ts_gemm_unpacked(const UmmaArgs &a, bool w4a16, Dtype td, size_t lda, size_t ldb, cudaStream_t st)
{
    TmaOperands maps{};
    const size_t a_elem = w4a16 ? 2 : 1;
    constexpr uint32_t kActRowsPair = kTsMT / 2;
    if (!encode_byte_map(&maps.a, a.A, (size_t)a.k * a_elem, a.m, lda * a_elem, 128, kActRowsPair)) return Result{kUnsupported, 0};
    if ((a.k & 1u) || (ldb & 1u) || !encode_byte_map(&maps.b, a.B, a.k / 2, a.n, ldb / 2, 64, 128)) return Result{kUnsupported, 0};
    if (w4a16) {
        if (td == Dtype::F16) return launch_ts_tma<TsKind::W4A16, Dtype::F16>(a, maps, st);
        if (td == Dtype::F32) return launch_ts_tma<TsKind::W4A16, Dtype::F32>(a, maps, st);
        return Result{kUnsupported, 0};
    }
    switch (td) {
        case Dtype::F32: return launch_ts_tma<TsKind::W4A8, Dtype::F32>(a, maps, st);
        case Dtype::F16: return launch_ts_tma<TsKind::W4A8, Dtype::F16>(a, maps, st);
        default: return launch_ts_tma<TsKind::W4A8, Dtype::BF16>(a, maps, st);
    }
}

}  // namespace tqt
