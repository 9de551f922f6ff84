// HBM-streaming W4A8 GEMV for decode (m <= 16; more rows run on the tensor-core kernel): no tensor
// cores, no clusters, no shared-memory staging of weights, no scratch memory.
//
// A CTA owns 8 consecutive output columns (8 rows of one 128-row block tile of B_packed) and loops
// over such groups when there are more groups than resident CTAs; its eight warps take interleaved
// K blocks.  Inside a warp lane = (row, 16-byte segment), so one warp-wide 128-bit load covers 512
// contiguous bytes of a packed block: every 32-byte sector is used whole, once.  A thread holds four
// weight loads at a time (64 registers in all), so four CTAs (32 warps) are resident per SM: on this
// part a streaming read reaches full bandwidth with many warps that each have a few loads
// outstanding, not with few warps that have many.  The next group's (or round's) loads are issued
// as soon as the registers are free, before the current group is combined and stored.
// Nibbles are expanded with two logic ops per 8 weights (operands 16*q, as in the tensor-core
// kernel) and accumulated with dp4a; the zero-point correction uses the int16 partial row sums
// stored at the tail of every packed block.  The four segments of a row are combined with warp
// shuffles and the eight warps through shared memory: integer sums, so the result is exact and
// independent of the split.  The epilogue is the GEMM's (reference:
// src/gemm/gemm_i8_i4/gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp/..._4x1vl_rvv.cpp:118-177).
//
// Programmatic dependent launch: the kernel lets its successor start at once and requests its
// weights and per-column constants before waiting for its predecessor, so back-to-back GEMVs (the
// layers of a decode step) overlap their memory phases.  Everything after that wait is on the
// critical path of the chain (a kernel's wait ends only when its predecessor has completed), so it
// is kept short: the activation words of a whole chunk are requested together, straight into
// registers (staging them in shared memory, or fetching the weights with bulk copies to make room
// for more resident kernels, both measured slower).  Activations, C and D are touched only after
// the wait.
// TQT_B200_PDL=0 switches this off.
#include <cstdlib>

#include "epilogues.cuh"
#include "ptx_sm100.cuh"

namespace tqt {

int sm_count_cached();

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
};

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
    // everything else may have been produced by the preceding kernel
    if (args.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");

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
        if (next >= sgroups) break;
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
    if constexpr (MR <= 8) {
        const uint32_t groups = (a.n + kGemvWarpRows - 1) / kGemvWarpRows;
        const int forced = gemv_forced_groups();
        const bool two = forced ? forced == 2 : (groups + 1) / 2 <= (uint32_t)sm_count_cached() * 2u;
        if (two) return launch_gemv_t<MR, 2, TD>(a, st);
    }
    return launch_gemv_t<MR, 1, TD>(a, st);
}

template <Dtype TD>
static Result launch_gemv_m(const GemvArgs &a, cudaStream_t st)
{
    if (a.m <= 1) return launch_gemv_g<1, TD>(a, st);
    if (a.m <= 2) return launch_gemv_g<2, TD>(a, st);
    if (a.m <= 4) return launch_gemv_g<4, TD>(a, st);
    if (a.m <= 8) return launch_gemv_g<8, TD>(a, st);
    return launch_gemv_g<16, TD>(a, st);
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
