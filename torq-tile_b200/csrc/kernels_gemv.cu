// HBM-streaming W4A8 GEMV for decode (m <= 8; 9..16 rows run on the tensor-core kernel): no tensor cores, no clusters, no scratch memory.
//
// One CTA per 32 output columns (32 consecutive rows of one 128-row block tile of B_packed) over
// the whole K.  Warp w owns rows 4w..4w+3; inside a warp lane = (row, kgroup): the eight kgroups
// split the K blocks.  Every thread issues the 128-bit loads of its share of the weights straight
// into registers at kernel entry (16 loads = 256 B per thread per round of 32 K blocks, 64 KiB per
// CTA), so the whole weight matrix is in flight across the GPU before any arithmetic starts and no
// single thread serialises the requests.  Nibbles are expanded with two logic ops per 8 weights
// (operands 16*q, as in the tensor-core kernel), accumulated with dp4a against activation words
// staged in shared memory, and the eight kgroups are combined with warp shuffles: integer sums, so
// the result is exact and independent of the split.  The epilogue is the GEMM's (reference:
// src/gemm/gemm_i8_i4/gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp/..._4x1vl_rvv.cpp:118-177).
//
// Programmatic dependent launch: the kernel lets its successor start at once and requests its
// weights before waiting for its predecessor, so back-to-back GEMVs (the layers of a decode step)
// overlap their memory phases; activations, C and D are touched only after the wait.
// TQT_B200_PDL=0 switches this off.
#include <cstdlib>

#include "epilogues.cuh"
#include "ptx_sm100.cuh"

namespace tqt {

long long *timing_buffer();

__device__ __forceinline__ long long gtime_ns()
{
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

constexpr uint32_t kGemvThreads = 256;
constexpr uint32_t kGemvRows = 32;      // output columns per CTA
constexpr uint32_t kGemvRoundKB = 32;   // K blocks per round: 8 kgroups x 4 blocks per thread

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
    long long *dbg;  // optional per-CTA phase timestamps (diagnostic), 16 slots per CTA
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

template <int MR, Dtype TD>
__global__ void __launch_bounds__(kGemvThreads, (MR <= 4 ? 2 : 1)) gemv_w4a8_kernel(const GemvArgs args)
{
    // activations of one round, de-swizzled: [32 K blocks][MR rows][128 B] (+16 B per block against bank conflicts)
    constexpr uint32_t kActStride = MR * 128u + 16u;
    __shared__ __align__(16) uint8_t sAct[kGemvRoundKB * kActStride];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t tile = blockIdx.x >> 2, quarter = blockIdx.x & 3u;
    const uint32_t KB = (args.k + 127) / 128;
    const uint32_t row_l = lane >> 3, kg = lane & 7u;
    const uint32_t r_blk = quarter * kGemvRows + warp * 4u + row_l;   // row inside the 128-row block
    const uint32_t swz = (r_blk >> 1) & 3u;

    long long ts[5] = {0, 0, 0, 0, 0};
    const bool dbg = args.dbg != nullptr && tid == 0;
    if (dbg) ts[0] = gtime_ns();
    if (args.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const uint8_t *wbase = args.B + (size_t)tile * args.b_kblocks_total * kI4CxBlockBytes + r_blk * 64u;
    uint4 wcur[16];
    auto load_round = [&](uint32_t base, uint4(&w)[16]) {
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t kb = base + kg + 8u * i;
            if (kb < KB) {
                const uint8_t *p = wbase + (size_t)kb * kI4CxBlockBytes;
#pragma unroll
                for (uint32_t seg = 0; seg < 4; ++seg) w[i * 4 + seg] = ldg_stream(p + ((seg ^ swz) << 4));
            } else {
#pragma unroll
                for (uint32_t seg = 0; seg < 4; ++seg) w[i * 4 + seg] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    load_round(0, wcur);
    if (dbg) ts[1] = gtime_ns();
    // weights are static; everything else may have been produced by the preceding kernel
    if (args.pdl) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (dbg) ts[2] = gtime_ns();

    int32_t acc[MR], acc2[MR];
#pragma unroll
    for (int i = 0; i < MR; ++i) acc[i] = acc2[i] = 0;
    int32_t rs16 = 0;   // 16 * sum of q over this thread's K blocks

    for (uint32_t base = 0; base < KB; base += kGemvRoundKB) {
        const uint32_t cnt = min(kGemvRoundKB, KB - base);
        if (base) __syncthreads();   // previous round's activations are no longer needed
        for (uint32_t i = tid; i < cnt * MR * 8u; i += kGemvThreads) {
            const uint32_t c = i & 7u, row = (i >> 3) % MR, kbl = (i >> 3) / MR;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < args.m)
                v = __ldg(reinterpret_cast<const uint4 *>(args.A + (size_t)(base + kbl) * kI8BlockBytes +
                                                          sw128_byte(row, c * 16u)));
            *reinterpret_cast<uint4 *>(sAct + kbl * kActStride + row * 128u + c * 16u) = v;
        }
        if (base) load_round(base, wcur);
        __syncthreads();
        if (dbg && base == 0) ts[3] = gtime_ns();
#pragma unroll
        for (uint32_t i = 0; i < 4; ++i) {
            const uint32_t s = kg + 8u * i;
            if (s < cnt) {
                const uint8_t *act = sAct + s * kActStride;
#pragma unroll
                for (uint32_t seg = 0; seg < 4; ++seg) {
                    const uint4 w = wcur[i * 4 + seg];
                    const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
                    uint32_t lo[4], hi[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        lo[j] = (ws[j] << 4) & 0xF0F0F0F0u;   // 16*q for k = 32*seg + 4j .. +3
                        hi[j] = ws[j] & 0xF0F0F0F0u;          // 16*q for k = 32*seg + 16 + 4j .. +3
                        rs16 = __dp4a((int)lo[j], 0x01010101, rs16);
                        rs16 = __dp4a((int)hi[j], 0x01010101, rs16);
                    }
#pragma unroll
                    for (int mi = 0; mi < MR; ++mi) {
                        const uint4 a0 = *reinterpret_cast<const uint4 *>(act + mi * 128u + seg * 32u);
                        const uint4 a1 = *reinterpret_cast<const uint4 *>(act + mi * 128u + seg * 32u + 16u);
                        const uint32_t al[4] = {a0.x, a0.y, a0.z, a0.w};
                        const uint32_t ah[4] = {a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc[mi] = __dp4a((int)al[j], (int)lo[j], acc[mi]);
                            acc2[mi] = __dp4a((int)ah[j], (int)hi[j], acc2[mi]);
                        }
                    }
                }
            }
        }
    }

    // combine the eight K groups of each row (lanes that differ in their low three bits)
#pragma unroll
    for (int mi = 0; mi < MR; ++mi) {
        int32_t v = acc[mi] + acc2[mi];
        v += __shfl_xor_sync(0xffffffffu, v, 1);
        v += __shfl_xor_sync(0xffffffffu, v, 2);
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        acc[mi] = v;
    }
    rs16 += __shfl_xor_sync(0xffffffffu, rs16, 1);
    rs16 += __shfl_xor_sync(0xffffffffu, rs16, 2);
    rs16 += __shfl_xor_sync(0xffffffffu, rs16, 4);
    if (dbg) {
        ts[4] = gtime_ns();
        for (int i = 0; i < 5; ++i) args.dbg[(size_t)blockIdx.x * 16 + i] = ts[i];
    }

    const uint32_t n = tile * 128u + r_blk;
    if (kg == 0 && n < args.n) {
        const int32_t rs = rs16 >> 4;
        const float sb = args.scale_b[n];
        const float bv = args.bias ? TdTraits<TD>::load(args.bias, n) : 0.0f;
#pragma unroll
        for (int mi = 0; mi < MR; ++mi) {
            if ((uint32_t)mi < args.m) {
                int32_t a = acc[mi] >> 4;   // operands were 16*q
                a -= args.zp_a[mi] * rs;
                const float cv = args.C ? TdTraits<TD>::load(args.C, (size_t)mi * args.ldc + n) : 0.0f;
                const float v = w4a8_epilogue(a, args.scale_a[mi], sb, args.C != nullptr, cv, args.bias != nullptr, bv,
                                              args.cmin, args.cmax);
                TdTraits<TD>::store(args.D, (size_t)mi * args.ldd + n, v);
            }
        }
    }
}

static bool pdl_enabled()
{
    static int cached = -1;
    if (cached < 0) {
        const char *e = std::getenv("TQT_B200_PDL");
        cached = (e && e[0] == '0') ? 0 : 1;
    }
    return cached != 0;
}

template <int MR, Dtype TD>
static Result launch_gemv_t(GemvArgs a, uint32_t ctas, cudaStream_t st)
{
    a.pdl = pdl_enabled() ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas, 1, 1);
    cfg.blockDim = dim3(kGemvThreads, 1, 1);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_w4a8_kernel<MR, TD>, a);
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

template <Dtype TD>
static Result launch_gemv_m(const GemvArgs &a, uint32_t ctas, cudaStream_t st)
{
    if (a.m <= 1) return launch_gemv_t<1, TD>(a, ctas, st);
    if (a.m <= 2) return launch_gemv_t<2, TD>(a, ctas, st);
    if (a.m <= 4) return launch_gemv_t<4, TD>(a, ctas, st);
    return launch_gemv_t<8, TD>(a, ctas, st);
}

Result gemv_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax)
{
    if (g.m == 0 || g.n == 0) return Result{kOk, 0};
    if (g.m > 8 || g.k == 0 || g.k > 65536 || g.n > 0x3fffff00ull) return Result{kUnsupported, 0};
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
    const uint32_t ctas = (uint32_t)ceil_div(g.n, kGemvRows);   // CTA c owns columns [32c, 32c + 32)
    cudaStream_t st = (cudaStream_t)g.stream;
    switch (td) {
        case Dtype::F32: return launch_gemv_m<Dtype::F32>(a, ctas, st);
        case Dtype::F16: return launch_gemv_m<Dtype::F16>(a, ctas, st);
        default: return launch_gemv_m<Dtype::BF16>(a, ctas, st);
    }
}

}  // namespace tqt
