// Tensor-core GEMM for sm_100a: bulk-copy (TMA) producer -> shared-memory ring -> tcgen05.mma with
// accumulators in tensor memory -> fused epilogue, as one persistent, warp-specialised kernel.
//
// CTA tile 128 (M) x 256 (N), K step 128.  Operands arrive as the pre-swizzled 128-row blocks the
// packers write, so one bulk copy per block lands them in shared memory exactly as the MMA reads
// them (K-major, 128-byte swizzle); no tensor maps are needed.
//
// Warp roles (one CTA per SM):
//   warp 0       producer: waits for a free stage, issues the bulk copies of the next K step
//   warp 1       MMA issuer: owns tensor memory (512 columns = two 128x256 accumulators), issues
//                tcgen05.mma from one lane and commits completion to the stage / accumulator barriers
//   warps 2-5    epilogue: tcgen05.ld of the finished accumulator, fused arithmetic, global stores;
//                runs on accumulator i while the mainloop fills accumulator i+1
//   warps 6-9    (int4 weights only) converters: expand packed int4 to the MMA operand type in
//                shared memory (int8 = 16*q for W4A8, f16 = q*scale for W4A16) and add up row sums
//
// Reference semantics implemented by the epilogues:
//   s32     src/gemm/gemm_i8_i8/gemm_clamp_i32_i8p_i8p/..._4x1vl_rvv.cpp (D = clamp(C + A*B))
//   requant src/gemm/gemm_i8_i8/gemm_1xnbias_reqi32toi8_clamp_qai8_qai8p_qsi8cxp/..._4x1vl_rvv.cpp:121-241
//   W4A8    src/gemm/gemm_i8_i4/gemm_1xnbias_clamp_*_qai8dxp_qsi4cxp/..._4x1vl_rvv.cpp:118-238
//   W4A16   src/gemm/gemm_f16_i4/gemm_1xnbias_clamp_*_f16p_qsi4c2p/..._8x2vl_rvv.cpp:127-283
//
// Every wait is bounded (ptx::mbar_wait); a wait that runs out records a code in the device fault
// word, the CTA stops issuing work, drains its copies, frees tensor memory and returns.
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "epilogues.cuh"
#include "ptx_sm100.cuh"
#include "umma_args.cuh"

namespace tqt {

// Diagnostic (builds with -DTQT_B200_DIAG only): when a timing buffer is installed (tqt_cuda_debug_set_timing_buffer) each
// role adds up the cycles it spends inside its waits; slot meaning is listed where the buffer is written.
#ifdef TQT_B200_DIAG
#define TQT_DIAG_ON(args) ((args).dbg != nullptr)
#else
#define TQT_DIAG_ON(args) false
#endif
#define TQT_TIMED(slot, call)                                   \
    ([&]() -> bool {                                            \
        if (!TQT_DIAG_ON(args)) return (call);                  \
        const long long _t0 = clock64();                        \
        const bool _r = (call);                                 \
        wcyc[slot] += clock64() - _t0;                          \
        return _r;                                              \
    }())

static std::atomic<unsigned> g_wait_shift{0}, g_inject{0};
void set_failure_injection(unsigned wait_shift, unsigned flags)
{
    g_wait_shift.store(wait_shift > 20 ? 20 : wait_shift);
    g_inject.store(flags);
}
static std::atomic<long long *> g_timing_buffer{nullptr};
void set_timing_buffer(void *p) { g_timing_buffer.store(static_cast<long long *>(p)); }
long long *timing_buffer() { return g_timing_buffer.load(std::memory_order_relaxed); }

template <BMode BM>
struct ModeCfg;
template <>
struct ModeCfg<BMode::I8> {
    static constexpr uint32_t kStages = 4, kExp = 0;
    static constexpr uint32_t kABytes = 16384, kBBlock = 16384, kBStage = 32768;
    static constexpr uint32_t kThreads = 192;
};
template <>
struct ModeCfg<BMode::I4Cx> {
    static constexpr uint32_t kStages = 4, kExp = 2;
    static constexpr uint32_t kABytes = 16384, kBBlock = 8448, kBStage = 2 * 8448;
    static constexpr uint32_t kThreads = 320;
};
template <>
struct ModeCfg<BMode::I4C2> {
    static constexpr uint32_t kStages = 3, kExp = 2;
    static constexpr uint32_t kABytes = 32768, kBBlock = 8192, kBStage = 2 * 8192;
    static constexpr uint32_t kThreads = 320;
};

constexpr uint32_t kExpBytes = 32768;                 // one expanded B operand buffer (256 rows x 128 B)
constexpr uint32_t kColParamBytes = 4 * 3 * 256 * 4;  // per-column epilogue parameters, one private copy per epilogue warp
constexpr uint32_t kRsumBytes = 2 * 256 * 4;          // row sums of B, one set per accumulator
constexpr uint32_t kBarrierBytes = 256;

template <BMode BM>
constexpr uint32_t umma_smem_bytes()
{
    using Cfg = ModeCfg<BM>;
    return 1024 /* alignment slack */ + Cfg::kStages * Cfg::kABytes + Cfg::kExp * kExpBytes + Cfg::kStages * Cfg::kBStage +
           kColParamBytes + kRsumBytes + kBarrierBytes;
}

template <BMode BM, EpiKind EK, Dtype TD>
__global__ void __launch_bounds__(ModeCfg<BM>::kThreads, 1) gemm_umma_kernel(const UmmaArgs args)
{
    using Cfg = ModeCfg<BM>;
    using OutT = typename OutType<EK, TD>::type;
    constexpr uint32_t S = Cfg::kStages;
    constexpr uint32_t E = Cfg::kExp;
    constexpr bool kConv = (BM != BMode::I8);
    constexpr bool kF16 = (BM == BMode::I4C2);

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sA = smem;                                   // S x kABytes
    uint8_t *sExp = sA + S * Cfg::kABytes;                // E x 32 KiB (1024-aligned)
    uint8_t *sB = sExp + E * kExpBytes;                   // S x kBStage (operand itself in I8 mode)
    float *sColAll = reinterpret_cast<float *>(sB + S * Cfg::kBStage);  // [4 warps][3][256]
    int32_t *sRsum = reinterpret_cast<int32_t *>(sColAll + 4 * 3 * 256);  // [2][256]
    uint64_t *bars = reinterpret_cast<uint64_t *>(sRsum + 2 * 256);
    // barrier indices
    constexpr uint32_t kFull = 0, kEmpty = 4, kConvFull = 8, kConvEmpty = 10, kTmemFull = 12, kTmemEmpty = 14,
                       kRsumFull = 16;
    uint32_t *sTmemBase = reinterpret_cast<uint32_t *>(bars + 20);
    volatile int *sAbort = reinterpret_cast<volatile int *>(sTmemBase + 1);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = ptx::smem_u32(bars);
    auto BAR = [&](uint32_t idx) { return bar0 + idx * 8u; };

    const uint32_t tiles_m = (args.m + 127) / 128;
    const uint32_t nblocks = (args.n + 127) / 128;       // 128-column blocks of B
    const uint32_t tiles_n = (nblocks + 1) / 2;
    const uint32_t num_tiles = tiles_m * tiles_n;
    const uint32_t KB = (args.k + 127) / 128;            // K steps of 128
    const uint32_t a_blocks_k = kF16 ? (args.k + 63) / 64 : KB;  // A blocks along k that hold data

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            ptx::mbar_init(BAR(kFull + s), 1);
            ptx::mbar_init(BAR(kEmpty + s), kConv ? 5 : 1);
        }
        for (uint32_t e = 0; e < 2; ++e) {
            ptx::mbar_init(BAR(kConvFull + e), 4);
            ptx::mbar_init(BAR(kConvEmpty + e), 1);
            ptx::mbar_init(BAR(kTmemFull + e), 1);
            ptx::mbar_init(BAR(kTmemEmpty + e), 4);
            ptx::mbar_init(BAR(kRsumFull + e), 4);
        }
        sAbort[0] = 0;
        sAbort[1] = (int)args.wait_shift;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(sTmemBase), 512);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *sTmemBase;
    long long wcyc[3] = {0, 0, 0};
    const long long t_role0 = TQT_DIAG_ON(args) ? clock64() : 0;

    if (warp == 0) {
        // ===================== producer =====================
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const uint32_t tm = t % tiles_m, tn = t / tiles_m;
            const uint32_t nblk = min(2u, nblocks - tn * 2);
            for (uint32_t kb = 0; kb < KB; ++kb, ++it) {
                const uint32_t s = it % S, ph = (it / S) & 1u;
                if (!TQT_TIMED(0, ptx::mbar_wait(BAR(kEmpty + s), ph ^ 1u, sAbort, args.fault, kFaultProducerWait))) {
                    ok = false;
                    break;
                }
                // lane 0 arms the barrier; lanes 0..nblk issue one bulk copy each in the same instruction
                uint32_t a_bytes = Cfg::kABytes;
                const uint8_t *a_src;
                if (kF16) {
                    const uint32_t nsub = min(2u, a_blocks_k - kb * 2);
                    a_bytes = nsub * 16384u;
                    a_src = args.A + ((size_t)tm * args.a_kblocks_total + kb * 2) * kF16BlockBytes;
                } else {
                    a_src = args.A + ((size_t)tm * args.a_kblocks_total + kb) * kI8BlockBytes;
                }
                if (lane == 0) ptx::mbar_arrive_expect_tx(BAR(kFull + s), a_bytes + nblk * Cfg::kBBlock);
                __syncwarp();
                if (lane == 0) {
                    ptx::bulk_g2s(ptx::smem_u32(sA + s * Cfg::kABytes), a_src, a_bytes, BAR(kFull + s));
                } else if (lane <= nblk) {
                    const uint32_t j = lane - 1;
                    const uint8_t *b_src = args.B + ((size_t)(tn * 2 + j) * args.b_kblocks_total + kb) * Cfg::kBBlock;
                    ptx::bulk_g2s(ptx::smem_u32(sB + s * Cfg::kBStage + j * Cfg::kBBlock), b_src, Cfg::kBBlock, BAR(kFull + s));
                }
                __syncwarp();
            }
        }
        if (!ok) {
            // Bail-out: let the copies already issued land before the CTA gives its shared memory back.
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
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        constexpr uint32_t dfmt = kF16 ? 1u : 2u;
        constexpr uint32_t ifmt = kF16 ? 0u : 1u;
        const uint32_t idesc256 = ptx::make_idesc(dfmt, ifmt, ifmt, 128, 256);
        const uint32_t idesc128 = ptx::make_idesc(dfmt, ifmt, ifmt, 128, 128);
        uint32_t it = 0, xit = 0, ti = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++ti) {
            const uint32_t tn = t / tiles_m;
            const uint32_t nblk = min(2u, nblocks - tn * 2);
            const uint32_t idesc = nblk == 2 ? idesc256 : idesc128;
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            if (!TQT_TIMED(0, ptx::mbar_wait(BAR(kTmemEmpty + acc), pha ^ 1u, sAbort, args.fault, kFaultMmaWaitTmem))) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * 256u;
            for (uint32_t kb = 0; kb < KB && ok; ++kb, ++it) {
                const uint32_t s = it % S, ph = (it / S) & 1u;
                if (!TQT_TIMED(1, ptx::mbar_wait(BAR(kFull + s), ph, sAbort, args.fault, kFaultMmaWaitFull))) {
                    ok = false;
                    break;
                }
                const uint32_t nsub = kF16 ? min(2u, a_blocks_k - kb * 2) : 1u;
                for (uint32_t h = 0; h < nsub; ++h) {
                    uint32_t b_addr;
                    uint32_t e = 0;
                    if (kConv) {
                        e = xit % 2u;
                        const uint32_t phe = (xit / 2u) & 1u;
                        if (!TQT_TIMED(2, ptx::mbar_wait(BAR(kConvFull + e), phe, sAbort, args.fault, kFaultMmaWaitFull))) {
                            ok = false;
                            break;
                        }
                        b_addr = ptx::smem_u32(sExp + e * kExpBytes);
                    } else {
                        b_addr = ptx::smem_u32(sB + s * Cfg::kBStage);
                    }
                    ptx::tc_fence_after();
                    if (lane == 0) {
                        const uint64_t a_desc = ptx::make_desc_k_sw128(ptx::smem_u32(sA + s * Cfg::kABytes + h * 16384u));
                        const uint64_t b_desc = ptx::make_desc_k_sw128(b_addr);
#pragma unroll
                        for (uint32_t j = 0; j < 4; ++j) {
                            // 32 bytes of K per instruction (32 int8 or 16 f16): +2 in the 16-byte address field
                            const uint32_t accum = (kb | h | j) ? 1u : 0u;
                            if (kF16)
                                ptx::mma_f16_ss(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc, accum);
                            else
                                ptx::mma_i8_ss(d_tmem, a_desc + 2 * j, b_desc + 2 * j, idesc, accum);
                        }
                        if (kConv) ptx::tc_commit(BAR(kConvEmpty + e));
                    }
                    __syncwarp();
                    if (kConv) ++xit;
                }
                if (!ok) break;
                if (lane == 0) {
                    ptx::tc_commit(BAR(kEmpty + s));
                    if (kb == KB - 1) ptx::tc_commit(BAR(kTmemFull + acc));
                }
                __syncwarp();
            }
        }
    } else if (warp < 6) {
        // ===================== epilogue =====================
        // The four epilogue warps work independently (no CTA-level barrier inside the loop, so a
        // warp that bails out cannot strand the others): each keeps a private copy of the tile's
        // per-column parameters.
        const uint32_t quad = warp & 3u;             // tensor-memory lane quadrant this warp may read
        const uint32_t row_in_tile = quad * 32u + lane;
        float *sColF = sColAll + (warp - 2u) * 768u;
        int32_t *sColI = reinterpret_cast<int32_t *>(sColF);
        uint32_t ti = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++ti) {
            const uint32_t tm = t % tiles_m, tn = t / tiles_m;
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            const uint32_t n0 = tn * 256u;
            const uint32_t ncols = min(256u, args.n - n0);
            const size_t mrow = (size_t)tm * 128u + row_in_tile;
            const bool row_ok = mrow < args.m;

            __syncwarp();  // every lane is done with the previous tile's parameters
            for (uint32_t c = lane; c < 256u; c += 32u) {
                const bool cok = c < ncols;
                const uint32_t n = n0 + c;
                if constexpr (EK == EpiKind::Req8) {
                    int32_t mult = 0, rsh = 0;
                    if (cok)
                        requant_column(args.rq_scale_a, args.scale_b[args.rq_per_tensor ? 0 : n], args.rq_scale_d, &mult, &rsh);
                    sColI[c] = mult;
                    sColI[256 + c] = rsh;
                    sColI[512 + c] = (cok && args.bias) ? static_cast<const int32_t *>(args.bias)[n] : 0;
                } else if constexpr (EK == EpiKind::W4A8) {
                    sColF[c] = cok ? args.scale_b[n] : 0.0f;
                    sColF[256 + c] = (cok && args.bias) ? TdTraits<TD>::load(args.bias, n) : 0.0f;
                } else if constexpr (EK == EpiKind::W4A16) {
                    sColF[256 + c] = (cok && args.bias) ? TdTraits<TD>::load(args.bias, n) : 0.0f;
                }
            }
            __syncwarp();

            float sa = 0.0f;
            int32_t zp = 0;
            if constexpr (EK == EpiKind::W4A8) {
                if (row_ok) {
                    sa = args.scale_a[mrow];
                    zp = args.zp_a[mrow];
                }
            }
            if (!TQT_TIMED(0, ptx::mbar_wait(BAR(kTmemFull + acc), pha, sAbort, args.fault, kFaultEpilogueWait))) {
                ok = false;
                break;
            }
            if constexpr (EK == EpiKind::W4A8) {
                if (!TQT_TIMED(1, ptx::mbar_wait(BAR(kRsumFull + acc), pha, sAbort, args.fault, kFaultEpilogueWait))) {
                    ok = false;
                    break;
                }
            }
            ptx::tc_fence_after();
            const uint32_t t_addr = tmem_base + acc * 256u + ((quad * 32u) << 16);
            const uint32_t nchunks = (ncols + 31u) / 32u;
            const bool has_c = args.C != nullptr, has_bias = args.bias != nullptr;
            for (uint32_t ch = 0; ch < nchunks; ++ch) {
                uint32_t r[32];
                __syncwarp();  // tcgen05.ld is warp-collective: issue it converged
                ptx::tmem_ld_32x32b_x32(t_addr + ch * 32u, r);
                ptx::tmem_wait_ld();
                if (row_ok) {
                    const uint32_t c0 = ch * 32u;
                    const uint32_t nvalid = min(32u, ncols - c0);
                    alignas(16) OutT out[32];
                    if constexpr (EK == EpiKind::S32 || EK == EpiKind::Req8) {
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
                            int32_t v = (int32_t)r[j];
                            v = v < args.cmin_i ? args.cmin_i : v;
                            v = v > args.cmax_i ? args.cmax_i : v;
                            out[j] = v;
                        } else if constexpr (EK == EpiKind::Req8) {
                            uint32_t u = r[j];
                            u += (uint32_t)sColI[512 + c];
                            out[j] = (int8_t)requant_value((int32_t)u, sColI[c], sColI[256 + c], args.rq_zp_d, args.cmin_i, args.cmax_i);
                        } else if constexpr (EK == EpiKind::W4A8) {
                            // operands were 16*q: the accumulator is an exact multiple of 16
                            int32_t a = ((int32_t)r[j]) >> 4;
                            a -= zp * sRsum[acc * 256 + c];
                            float cv = 0.0f;
                            if (has_c && j < nvalid) cv = TdTraits<TD>::load(args.C, mrow * args.ldc + n0 + c);
                            const float v = w4a8_epilogue(a, sa, sColF[c], has_c, cv, has_bias,
                                                          sColF[256 + c], args.cmin_f, args.cmax_f);
                            out[j] = cvt_out<OutT>(v);
                        } else {
                            float v = __uint_as_float(r[j]);
                            float cv = 0.0f;
                            if (has_c && j < nvalid) cv = TdTraits<TD>::load(args.C, mrow * args.ldc + n0 + c);
                            v = has_c ? __fadd_rn(v, cv) : v;
                            v = has_bias ? __fadd_rn(v, sColF[256 + c]) : v;
                            v = v < args.cmin_f ? args.cmin_f : v;
                            v = v > args.cmax_f ? args.cmax_f : v;
                            out[j] = cvt_out<OutT>(v);
                        }
                    }
                    OutT *dst = static_cast<OutT *>(args.D) + mrow * args.ldd + n0 + c0;
                    if (args.vec_store && nvalid == 32u) {
                        constexpr uint32_t nvec = 32u * sizeof(OutT) / 16u;
#pragma unroll
                        for (uint32_t v = 0; v < nvec; ++v)
                            reinterpret_cast<uint4 *>(dst)[v] = reinterpret_cast<const uint4 *>(out)[v];
                    } else {
#pragma unroll
                        for (uint32_t j = 0; j < 32; ++j)
                            if (j < nvalid) dst[j] = out[j];
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(BAR(kTmemEmpty + acc));
        }
    } else if (kConv) {
        // ===================== int4 converters (warps 6..9) =====================
        const uint32_t r = (warp - 6u) * 32u + lane;    // row of each 128-row block this thread expands
        const uint32_t swz_in = (r >> 1) & 3u, swz_out = r & 7u;
        uint32_t it = 0, xit = 0, ti = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++ti) {
            const uint32_t tn = t / tiles_m;
            const uint32_t nblk = min(2u, nblocks - tn * 2);
            const uint32_t acc = ti & 1u, pha = (ti >> 1) & 1u;
            int32_t rsum[2] = {0, 0};
            for (uint32_t kb = 0; kb < KB && ok; ++kb, ++it) {
                const uint32_t s = it % S, ph = (it / S) & 1u;
                if (!TQT_TIMED(0, ptx::mbar_wait(BAR(kFull + s), ph, sAbort, args.fault, kFaultConverterWait))) {
                    ok = false;
                    break;
                }
                const uint8_t *raw = sB + s * Cfg::kBStage;
                const uint32_t nsub = kF16 ? min(2u, a_blocks_k - kb * 2) : 1u;
                for (uint32_t h = 0; h < nsub; ++h, ++xit) {
                    const uint32_t e = xit % 2u, phe = (xit / 2u) & 1u;
                    if (!TQT_TIMED(1, ptx::mbar_wait(BAR(kConvEmpty + e), phe ^ 1u, sAbort, args.fault, kFaultConverterWait))) {
                        ok = false;
                        break;
                    }
                    uint8_t *exp = sExp + e * kExpBytes;
                    for (uint32_t j = 0; j < nblk; ++j) {
                        const uint8_t *rawrow = raw + j * Cfg::kBBlock + r * 64u;
                        uint8_t *exprow = exp + j * 16384u + r * 128u;
                        if constexpr (!kF16) {
#pragma unroll
                            for (uint32_t seg = 0; seg < 4; ++seg) {
                                const uint4 w = *reinterpret_cast<const uint4 *>(rawrow + ((seg ^ swz_in) << 4));
                                uint4 lo, hi;
                                lo.x = (w.x << 4) & 0xF0F0F0F0u; hi.x = w.x & 0xF0F0F0F0u;
                                lo.y = (w.y << 4) & 0xF0F0F0F0u; hi.y = w.y & 0xF0F0F0F0u;
                                lo.z = (w.z << 4) & 0xF0F0F0F0u; hi.z = w.z & 0xF0F0F0F0u;
                                lo.w = (w.w << 4) & 0xF0F0F0F0u; hi.w = w.w & 0xF0F0F0F0u;
                                *reinterpret_cast<uint4 *>(exprow + (((2 * seg) ^ swz_out) << 4)) = lo;
                                *reinterpret_cast<uint4 *>(exprow + (((2 * seg + 1) ^ swz_out) << 4)) = hi;
                            }
                            rsum[j] += (int32_t) reinterpret_cast<const int16_t *>(raw + j * Cfg::kBBlock + kI4NibBytes)[r];
                        } else {
                            // 64 k of this sub-step = segments 2h, 2h+1; each word holds 8 k as
                            // nibbles (k0,k2,k4,k6,k1,k3,k5,k7) so that (w >> 4t) & 0x000F000F = (k2t, k2t+1).
                            // nibble u = q + 8; 0x6400 | u is the f16 1024 + u, so q = that - 1032 exactly,
                            // and q * scale is rounded once, like the RVV kernel's f16 multiply.
                            const size_t nrow = (size_t)(tn * 2 + j) * 128u + r;
                            const bool n_ok = nrow < args.n;
                            const uint32_t kbase = kb * 128u + h * 64u;
                            const __half *srow = args.scale_blk + nrow * args.ldsb;
                            const __half2 k1032 = __float2half2_rn(1032.0f);
                            const bool word_scale = (args.bl & 7u) == 0u;   // one scale per 8-k word
#pragma unroll
                            for (uint32_t sg = 0; sg < 2; ++sg) {
                                const uint32_t seg = 2 * h + sg;
                                const uint4 w4 = *reinterpret_cast<const uint4 *>(rawrow + ((seg ^ swz_in) << 4));
                                const uint32_t ws[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                                for (uint32_t wi = 0; wi < 4; ++wi) {
                                    const uint32_t k0 = kbase + sg * 32u + wi * 8u;   // first k of this word
                                    uint32_t o[4];
                                    if (word_scale) {
                                        __half sc = __ushort_as_half((unsigned short)0);
                                        if (n_ok && k0 < args.k) sc = __ldg(srow + k0 / args.bl);
                                        const __half2 sc2 = __half2half2(sc);
#pragma unroll
                                        for (uint32_t tt = 0; tt < 4; ++tt) {
                                            const uint32_t bits = ((ws[wi] >> (4 * tt)) & 0x000F000Fu) | 0x64006400u;
                                            const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&bits), k1032), sc2);
                                            o[tt] = *reinterpret_cast<const uint32_t *>(&v);
                                        }
                                    } else {
#pragma unroll
                                        for (uint32_t tt = 0; tt < 4; ++tt) {
                                            const uint32_t kk = k0 + 2 * tt;   // bl is even: a pair never straddles blocks
                                            __half sc = __ushort_as_half((unsigned short)0);
                                            if (n_ok && kk < args.k) sc = __ldg(srow + kk / args.bl);
                                            const uint32_t bits = ((ws[wi] >> (4 * tt)) & 0x000F000Fu) | 0x64006400u;
                                            const __half2 v = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&bits), k1032), __half2half2(sc));
                                            o[tt] = *reinterpret_cast<const uint32_t *>(&v);
                                        }
                                    }
                                    const uint32_t chunk = sg * 4u + wi;
                                    *reinterpret_cast<uint4 *>(exprow + ((chunk ^ swz_out) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                                }
                            }
                        }
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(BAR(kConvFull + e));
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(BAR(kEmpty + s));
            }
            if (!ok) break;
            if constexpr (EK == EpiKind::W4A8) {
                // hand the row sums of this tile to the epilogue once accumulator `acc` is free again
                if (!TQT_TIMED(2, ptx::mbar_wait(BAR(kTmemEmpty + acc), pha ^ 1u, sAbort, args.fault, kFaultConverterWait))) {
                    ok = false;
                    break;
                }
                sRsum[acc * 256 + r] = rsum[0];
                sRsum[acc * 256 + 128 + r] = rsum[1];
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(BAR(kRsumFull + acc));
            }
        }
    }

    if (TQT_DIAG_ON(args) && lane == 0 && (warp == 0 || warp == 1 || warp == 2 || warp == 6)) {
        // slots per CTA: producer 0-3, MMA 4-7, epilogue warp 8-11, converter warp 12-15; each {wait0, wait1, wait2, total}
        long long *d = args.dbg + (size_t)blockIdx.x * 16 + (warp == 0 ? 0 : warp == 1 ? 4 : warp == 2 ? 8 : 12);
        d[0] = wcyc[0];
        d[1] = wcyc[1];
        d[2] = wcyc[2];
        d[3] = clock64() - t_role0;
    }
    // ---- teardown: everyone arrives, then the allocating warp frees tensor memory ----
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, 512);
    }
}

// ---- host side --------------------------------------------------------------------------------------
int sm_count_cached()
{
    static int cache[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cache[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev] = n;
    }
    return cache[dev];
}

template <BMode BM, EpiKind EK, Dtype TD>
static Result launch_umma(const UmmaArgs &a, cudaStream_t st)
{
    constexpr uint32_t smem = umma_smem_bytes<BM>();
    auto kern = gemm_umma_kernel<BM, EK, TD>;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
        attr_set[dev] = true;
    }
    const uint32_t tiles = ((a.m + 127) / 128) * ((((a.n + 127) / 128) + 1) / 2);
    const uint32_t grid = tiles < (uint32_t)sm_count_cached() ? tiles : (uint32_t)sm_count_cached();
    kern<<<grid, ModeCfg<BM>::kThreads, smem, st>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

static bool fill_common(UmmaArgs &a, const GemmCommon &g, size_t out_elem, size_t a_kblk, size_t b_kblk)
{
    if (g.m == 0 || g.n == 0 || g.k == 0) return false;
    if (g.m > 0x7fffff00ull || g.n > 0x7fffff00ull || g.k > 0x7fffff00ull) return false;
    a.m = (uint32_t)g.m;
    a.n = (uint32_t)g.n;
    a.k = (uint32_t)g.k;
    a.A = (const uint8_t *)g.A;
    a.B = (const uint8_t *)g.B;
    a.a_kblocks_total = (uint32_t)ceil_div(g.lda, a_kblk);
    a.b_kblocks_total = (uint32_t)ceil_div(g.ldb, b_kblk);
    a.b_block_bytes = (uint32_t)kI8BlockBytes;
    a.C = g.C;
    a.ldc = g.ldc;
    a.D = g.D;
    a.ldd = g.ldd;
    a.bias = g.bias;
    a.vec_store = ((reinterpret_cast<uintptr_t>(g.D) & 15) == 0 && ((g.ldd * out_elem) & 15) == 0) ? 1 : 0;
    a.n_replicas = (uint32_t)(g.n_replicas > 7 ? 7 : g.n_replicas);
    for (uint32_t i = 0; i < a.n_replicas; ++i) a.replica_delta[i] = g.replica_delta[i];
    a.fault = fault_word_device_ptr();
    a.dbg = timing_buffer();
    a.wait_shift = g_wait_shift.load(std::memory_order_relaxed);
    a.inject = g_inject.load(std::memory_order_relaxed);
    // bulk copies need 16-byte aligned sources; block sizes are multiples of 16
    if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.B) & 15)) return false;
    return true;
}

Result pair_gemm_i8(const UmmaArgs &a, bool requant, cudaStream_t st);
Result ts_gemm_w4a8(const UmmaArgs &a, Dtype td, bool pair, cudaStream_t st);
Result ts_gemm_w4a16(const UmmaArgs &a, Dtype td, bool pair, cudaStream_t st);

// TQT_B200_UMMA=single|pair forces one of the two tensor-core kernels (tests); default: CTA pairs
// once the problem has more than one 128-row tile, the single-CTA kernel below that.
static bool use_pair(uint32_t m, uint32_t min_m)
{
    const int v = umma_variant();
    if (v == 1) return false;
    if (v == 2) return true;
    return m > min_m;
}

// Operands that together overflow L2 (126 MB, shared with the output stream): walk the tile grid in
// bands of 8 activation-row tiles, so a band's activations stay resident while the weights stream once
// per band.  TQT_B200_BAND overrides (0 = one band), for measurements.
static uint32_t choose_band(size_t a_bytes, size_t b_bytes)
{
    static const int forced = [] {
        const char *e = std::getenv("TQT_B200_BAND");
        return e ? std::atoi(e) : -1;
    }();
    if (forced >= 0) return (uint32_t)forced;
    return a_bytes + b_bytes > (size_t)72 << 20 ? 8u : 0u;
}

Result umma_gemm_i32(const GemmCommon &g, int32_t cmin, int32_t cmax)
{
    UmmaArgs a{};
    if (!fill_common(a, g, 4, 128, 128)) return Result{kUnsupported, 0};
    a.cmin_i = cmin;
    a.cmax_i = cmax;
    a.band_m = choose_band(g.m * g.k, g.n * g.k);
    if (a.n_replicas) return Result{kUnsupported, 0};
    if (use_pair(a.m, 128)) return pair_gemm_i8(a, false, (cudaStream_t)g.stream);
    return launch_umma<BMode::I8, EpiKind::S32, Dtype::F32>(a, (cudaStream_t)g.stream);
}

Result umma_gemm_requant_i8(const GemmCommon &g, const RequantParams &p, int cmin, int cmax)
{
    UmmaArgs a{};
    if (!fill_common(a, g, 1, 128, 128)) return Result{kUnsupported, 0};
    a.cmin_i = cmin;
    a.cmax_i = cmax;
    a.rq_scale_a = p.scale_a;
    a.scale_b = p.scale_b;
    a.rq_per_tensor = p.quant_channel_b == 1;
    a.rq_scale_d = p.scale_d;
    a.rq_zp_d = p.zero_point_d;
    a.band_m = choose_band(g.m * g.k, g.n * g.k);
    if (a.n_replicas) return Result{kUnsupported, 0};
    if (use_pair(a.m, 128)) return pair_gemm_i8(a, true, (cudaStream_t)g.stream);
    return launch_umma<BMode::I8, EpiKind::Req8, Dtype::F32>(a, (cudaStream_t)g.stream);
}

Result pair_gemm_i8_rows(const UmmaArgs &a, cudaStream_t st);
Result pair_gemm_i8_dxcx(const UmmaArgs &a, Dtype td, cudaStream_t st);

// ---- int8 x int8 with row-major operands: tiled TMA loads into the CTA-pair kernel -------------------------------
Result pair_gemm_i8_tma(const UmmaArgs &a, EpiKind ek, Dtype td, size_t lda, size_t ldb, cudaStream_t st);

// Fills the operand sources for layouts (la, lb); false for combinations the tensor-core kernel does not take
// (A stored [k, m]; both packed, which the block kernels handle).
static bool tma_sources(UmmaArgs &a, Layout la, Layout lb)
{
    if (la == Layout::KMajor || (la == Layout::Packed && lb == Layout::Packed)) return false;
    a.a_src = la == Layout::Packed ? kSrcBlocks : kSrcTmaK;
    a.b_src = lb == Layout::Packed ? kSrcBlocks : lb == Layout::RowMajor ? kSrcTmaK : kSrcTmaMn;
    return true;
}

Result umma_gemm_i32_layouts(const GemmCommon &g, int32_t cmin, int32_t cmax, Layout la, Layout lb)
{
    UmmaArgs a{};
    if (!fill_common(a, g, 4, 128, 128) || a.n_replicas || !tma_sources(a, la, lb)) return Result{kUnsupported, 0};
    a.cmin_i = cmin;
    a.cmax_i = cmax;
    a.band_m = choose_band(g.m * g.k, g.n * g.k);
    return pair_gemm_i8_tma(a, EpiKind::S32, Dtype::F32, g.lda, g.ldb, (cudaStream_t)g.stream);
}

Result umma_gemm_requant_i8_layouts(const GemmCommon &g, const RequantParams &p, int cmin, int cmax, Layout la, Layout lb)
{
    UmmaArgs a{};
    if (!fill_common(a, g, 1, 128, 128) || a.n_replicas || !tma_sources(a, la, lb)) return Result{kUnsupported, 0};
    a.cmin_i = cmin;
    a.cmax_i = cmax;
    a.rq_scale_a = p.scale_a;
    a.scale_b = p.scale_b;
    a.rq_per_tensor = p.quant_channel_b == 1;
    a.rq_scale_d = p.scale_d;
    a.rq_zp_d = p.zero_point_d;
    a.band_m = choose_band(g.m * g.k, g.n * g.k);
    return pair_gemm_i8_tma(a, EpiKind::Req8, Dtype::F32, g.lda, g.ldb, (cudaStream_t)g.stream);
}

Result umma_gemm_requant_rows_i8_layouts(const GemmCommon &g, const RowRequantParams &p, int cmin, int cmax, Layout la,
                                         Layout lb)
{
    UmmaArgs a{};
    if (!fill_common(a, g, 1, 128, 128) || a.n_replicas || !tma_sources(a, la, lb)) return Result{kUnsupported, 0};
    a.cmin_i = cmin;
    a.cmax_i = cmax;
    a.rq_scale_rows = p.scale_a;
    a.rq_per_tensor = p.quant_channel_a == 1;
    a.rq_scale_a = p.scale_b;
    a.rq_scale_d = p.scale_d;
    a.rq_zp_d = p.zero_point_d;
    a.band_m = choose_band(g.m * g.k, g.n * g.k);
    return pair_gemm_i8_tma(a, EpiKind::Req8Row, Dtype::F32, g.lda, g.ldb, (cudaStream_t)g.stream);
}

// qai8dx x qsi8cx with float output on row-major operands (A [m, lda], B^T [n, ldb]): the epilogue adds up the rows of B
// for the zero-point correction that the packed blocks carry in their tails.
Result umma_gemm_dxcx_layouts(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax, Layout la, Layout lb)
{
    UmmaArgs a{};
    if (la != Layout::RowMajor || lb != Layout::RowMajor) return Result{kUnsupported, 0};
    if (!fill_common(a, g, td == Dtype::F32 ? 4 : 2, 128, 128) || a.n_replicas || !tma_sources(a, la, lb)) return Result{kUnsupported, 0};
    a.scale_a = p.scale_a;
    a.zp_a = p.zp_a;
    a.scale_b = p.scale_b;
    a.cmin_f = cmin;
    a.cmax_f = cmax;
    a.band_m = choose_band(g.m * g.k, g.n * g.k);
    return pair_gemm_i8_tma(a, EpiKind::DxCx, td, g.lda, g.ldb, (cudaStream_t)g.stream);
}

// qai8dxp x qsi8cxp with float output on packed operands (B blocks carry their row sums): the CTA-pair kernel.
Result umma_gemm_dxcx(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax)
{
    UmmaArgs a{};
    if (!fill_common(a, g, td == Dtype::F32 ? 4 : 2, 128, 128)) return Result{kUnsupported, 0};
    if (a.n_replicas) return Result{kUnsupported, 0};
    a.b_block_bytes = (uint32_t)kI8SumBlockBytes;
    a.scale_a = p.scale_a;
    a.zp_a = p.zp_a;
    a.scale_b = p.scale_b;
    a.cmin_f = cmin;
    a.cmax_f = cmax;
    a.band_m = choose_band(g.m * g.k, g.n * g.k);
    return pair_gemm_i8_dxcx(a, td, (cudaStream_t)g.stream);
}

// Mx1-bias requantising GEMM on packed operands: the CTA-pair kernel with a per-row epilogue (any m).
Result umma_gemm_requant_rows_i8(const GemmCommon &g, const RowRequantParams &p, int cmin, int cmax)
{
    UmmaArgs a{};
    if (!fill_common(a, g, 1, 128, 128)) return Result{kUnsupported, 0};
    if (a.n_replicas) return Result{kUnsupported, 0};
    a.cmin_i = cmin;
    a.cmax_i = cmax;
    a.rq_scale_rows = p.scale_a;
    a.rq_per_tensor = p.quant_channel_a == 1;
    a.rq_scale_a = p.scale_b;
    a.rq_scale_d = p.scale_d;
    a.rq_zp_d = p.zero_point_d;
    a.band_m = choose_band(g.m * g.k, g.n * g.k);
    return pair_gemm_i8_rows(a, (cudaStream_t)g.stream);
}

Result umma_gemm_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax)
{
    UmmaArgs a{};
    const size_t es = td == Dtype::F32 ? 4 : 2;
    if (!fill_common(a, g, es, 128, 128)) return Result{kUnsupported, 0};
    if (g.k > 65536) return Result{kUnsupported, 0};  // 16*q operands: keep |acc| < 2^31
    a.scale_a = p.scale_a;
    a.zp_a = p.zp_a;
    a.scale_b = p.scale_b;
    a.cmin_f = cmin;
    a.cmax_f = cmax;
    a.band_m = choose_band(g.m * g.k, g.n * g.k / 2);
    cudaStream_t st = (cudaStream_t)g.stream;
    if (umma_variant() == 3) return ts_gemm_w4a8(a, td, false, st);
    if (use_pair(a.m, 96)) return ts_gemm_w4a8(a, td, true, st);
    if (a.n_replicas) return ts_gemm_w4a8(a, td, true, st);   // only the CTA-pair tensor-memory kernels store replicas
    switch (td) {
        case Dtype::F32: return launch_umma<BMode::I4Cx, EpiKind::W4A8, Dtype::F32>(a, st);
        case Dtype::F16: return launch_umma<BMode::I4Cx, EpiKind::W4A8, Dtype::F16>(a, st);
        default: return launch_umma<BMode::I4Cx, EpiKind::W4A8, Dtype::BF16>(a, st);
    }
}

Result umma_gemm_w4a16(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td, float cmin,
                       float cmax)
{
    UmmaArgs a{};
    const size_t es = td == Dtype::F32 ? 4 : 2;
    if (!fill_common(a, g, es, 64, 128)) return Result{kUnsupported, 0};
    a.scale_blk = (const __half *)scale_b;
    a.ldsb = ldsb;
    a.bl = (uint32_t)bl;
    a.cmin_f = cmin;
    a.cmax_f = cmax;
    a.band_m = choose_band(g.m * g.k * 2, g.n * g.k / 2);
    cudaStream_t st = (cudaStream_t)g.stream;
    if (umma_variant() == 3) return ts_gemm_w4a16(a, td, false, st);
    if (use_pair(a.m, 96)) return ts_gemm_w4a16(a, td, true, st);
    if (a.n_replicas) return ts_gemm_w4a16(a, td, true, st);
    if (td == Dtype::F16) return launch_umma<BMode::I4C2, EpiKind::W4A16, Dtype::F16>(a, st);
    return launch_umma<BMode::I4C2, EpiKind::W4A16, Dtype::F32>(a, st);
}

// ---- int4 weights with row-major operands: tiled TMA loads into the CTA-pair tensor-memory kernel ----------------
Result ts_gemm_unpacked(const UmmaArgs &a, bool w4a16, Dtype td, size_t lda, size_t ldb, cudaStream_t st);

Result umma_gemm_w4a8_unpacked(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax)
{
    UmmaArgs a{};
    if (!fill_common(a, g, td == Dtype::F32 ? 4 : 2, 128, 128) || a.n_replicas || g.k > 65536) return Result{kUnsupported, 0};
    a.scale_a = p.scale_a;
    a.zp_a = p.zp_a;
    a.scale_b = p.scale_b;
    a.cmin_f = cmin;
    a.cmax_f = cmax;
    a.band_m = choose_band(g.m * g.k, g.n * g.k / 2);
    return ts_gemm_unpacked(a, false, td, g.lda, g.ldb, (cudaStream_t)g.stream);
}

Result umma_gemm_w4a16_unpacked(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td, float cmin,
                                float cmax)
{
    UmmaArgs a{};
    if (td == Dtype::BF16 || !fill_common(a, g, td == Dtype::F32 ? 4 : 2, 64, 128) || a.n_replicas) return Result{kUnsupported, 0};
    a.scale_blk = (const __half *)scale_b;
    a.ldsb = ldsb;
    a.bl = (uint32_t)bl;
    a.cmin_f = cmin;
    a.cmax_f = cmax;
    a.band_m = choose_band(g.m * g.k * 2, g.n * g.k / 2);
    return ts_gemm_unpacked(a, true, td, g.lda, g.ldb, (cudaStream_t)g.stream);
}

// ---- W4A8 with the activation quantiser fused in front ----------------------------------------------------------
Result ts_gemm_w4a8_fusedq(const UmmaArgs &a, Dtype td, const void *q_in, size_t q_lda, bool q_bf16, cudaStream_t st);

Result umma_gemm_w4a8_fusedq(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax, const void *q_in,
                             size_t q_lda, bool q_bf16)
{
    UmmaArgs a{};
    if (!fill_common(a, g, td == Dtype::F32 ? 4 : 2, 128, 128) || a.n_replicas || umma_variant() != 0) return Result{kUnsupported, 0};
    a.scale_a = p.scale_a;
    a.zp_a = p.zp_a;
    a.scale_b = p.scale_b;
    a.cmin_f = cmin;
    a.cmax_f = cmax;
    a.band_m = choose_band(g.m * g.k, g.n * g.k / 2);
    return ts_gemm_w4a8_fusedq(a, td, q_in, q_lda, q_bf16, (cudaStream_t)g.stream);
}

// ---- unquantised f16 / bf16 GEMM on the CTA-pair kernel ---------------------------------------------------------
Result pair_gemm_f16(const UmmaArgs &a, bool bf16, Dtype td, bool bias_per_row, size_t lda, size_t ldb, cudaStream_t st);

Result umma_gemm_float(const GemmCommon &g, Dtype ta, Dtype td, float cmin, float cmax, Layout la, Layout lb, bool bias_per_row)
{
    UmmaArgs a{};
    if (ta == Dtype::F32) return Result{kUnsupported, 0};
    if (!fill_common(a, g, td == Dtype::F32 ? 4 : 2, 64, 64) || a.n_replicas) return Result{kUnsupported, 0};
    a.a_src = la == Layout::Packed ? kSrcBlocks : kSrcTmaK;
    a.b_src = lb == Layout::Packed ? kSrcBlocks : lb == Layout::RowMajor ? kSrcTmaK : kSrcTmaMn;
    a.cmin_f = cmin;
    a.cmax_f = cmax;
    a.band_m = choose_band(g.m * g.k * 2, g.n * g.k * 2);
    return pair_gemm_f16(a, ta == Dtype::BF16, td, bias_per_row, g.lda, g.ldb, (cudaStream_t)g.stream);
}

}  // namespace tqt
