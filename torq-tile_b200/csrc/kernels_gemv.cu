// HBM-streaming W4A8 GEMV for decode (m <= 16): no tensor cores, the whole weight matrix is put in
// flight at once.
//
// One thread-block cluster per 128 output columns (one row-tile of B_packed); the CTAs of a cluster
// split K.  Each CTA issues bulk copies (TMA, untiled) for all of its weight blocks at entry, one
// mbarrier per block, so that ~N*K/2 bytes are outstanding across the GPU before any arithmetic
// starts; it stages the few activation rows in shared memory meanwhile.  Thread (row, half) expands
// its row's nibbles with two logic ops per 8 weights (operands 16*q, as in the tensor-core kernel)
// and accumulates with dp4a against broadcast activation words.  Partial sums are combined with
// integer atomics into the cluster leader's shared memory (distributed shared memory), so the
// result is exact and independent of the split, and the leader applies the same epilogue as the
// GEMM (reference: src/gemm/gemm_i8_i4/gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp/..._4x1vl_rvv.cpp:118-177).
//
// No global scratch memory is used.
#include <cooperative_groups.h>

#include "epilogues.cuh"
#include "ptx_sm100.cuh"

namespace cg = cooperative_groups;

namespace tqt {

constexpr uint32_t kGemvThreads = 256;
constexpr uint32_t kGemvMaxSlots = 20;  // weight blocks resident per CTA (20 x 8448 B = 165 KiB)

struct GemvArgs {
    uint32_t m, n, k;
    const uint8_t *A;  // packed int8 blocks (row-tile 0 only: m <= 16)
    const uint8_t *B;  // packed qsi4cx blocks
    uint32_t a_kblocks_total, b_kblocks_total;
    const void *C;
    size_t ldc;
    void *D;
    size_t ldd;
    const void *bias;
    const float *scale_a;
    const int32_t *zp_a;
    const float *scale_b;
    float cmin, cmax;
    uint32_t kb_per_cta;  // K blocks handled by each CTA of a cluster
    uint32_t slots;       // resident weight blocks per round
    unsigned int *fault;
};

template <int MR, Dtype TD>
__global__ void __launch_bounds__(kGemvThreads) gemv_w4a8_kernel(const GemvArgs args)
{
    extern __shared__ __align__(128) uint8_t smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t crank = cluster.block_rank();
    const uint32_t csize = cluster.num_blocks();
    const uint32_t ntile = blockIdx.y;
    const uint32_t tid = threadIdx.x;

    const uint32_t KB = (args.k + 127) / 128;
    const uint32_t kb_begin = min(KB, crank * args.kb_per_cta);
    const uint32_t kb_end = min(KB, kb_begin + args.kb_per_cta);
    const uint32_t nkb = kb_end - kb_begin;
    const uint32_t slots = args.slots;

    // shared memory: [slots] weight blocks | activations [nkb][MR][128] | reduce [(MR+1)][128] int32 | barriers
    uint8_t *sW = smem;
    uint8_t *sAct = sW + slots * kI4CxBlockBytes;
    int32_t *sRed = reinterpret_cast<int32_t *>(sAct + (size_t)args.kb_per_cta * MR * 128u);
    uint64_t *bars = reinterpret_cast<uint64_t *>(sRed + (MR + 1) * 128);
    __shared__ int sAbort;

    if (tid == 0) {
        for (uint32_t i = 0; i < slots; ++i) ptx::mbar_init(ptx::smem_u32(bars + i), 1);
        sAbort = 0;
        ptx::fence_mbar_init();
    }
    for (uint32_t i = tid; i < (MR + 1) * 128; i += kGemvThreads) sRed[i] = 0;
    __syncthreads();

    // put the first round of weight blocks in flight
    const uint8_t *wsrc = args.B + ((size_t)ntile * args.b_kblocks_total + kb_begin) * kI4CxBlockBytes;
    if (tid == 0) {
        const uint32_t first = min(nkb, slots);
        for (uint32_t i = 0; i < first; ++i) {
            const uint32_t bar = ptx::smem_u32(bars + i);
            ptx::mbar_arrive_expect_tx(bar, (uint32_t)kI4CxBlockBytes);
            ptx::bulk_g2s(ptx::smem_u32(sW + i * kI4CxBlockBytes), wsrc + (size_t)i * kI4CxBlockBytes,
                          (uint32_t)kI4CxBlockBytes, bar);
        }
    }
    // stage the activation rows of this CTA's K range, de-swizzled: sAct[kb][row][128]
    for (uint32_t i = tid; i < nkb * MR * 8u; i += kGemvThreads) {
        const uint32_t c = i & 7u, row = (i >> 3) % MR, kbl = (i >> 3) / MR;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < args.m)
            v = __ldg(reinterpret_cast<const uint4 *>(args.A + (size_t)(kb_begin + kbl) * kI8BlockBytes +
                                                      sw128_byte(row, c * 16u)));
        *reinterpret_cast<uint4 *>(sAct + ((size_t)kbl * MR + row) * 128u + c * 16u) = v;
    }
    __syncthreads();
    cluster.sync();  // every CTA of the cluster is running and has zeroed its reduce buffer

    const uint32_t r = tid & 127u, half = tid >> 7;
    const uint32_t swz = (r >> 1) & 3u;
    int32_t acc[MR], acc2[MR];
#pragma unroll
    for (int i = 0; i < MR; ++i) acc[i] = acc2[i] = 0;
    int32_t rsum = 0;
    bool ok = true;
    volatile int *abort_flag = &sAbort;

    // Every thread runs the same number of rounds (the refill below uses __syncthreads); after a
    // failed wait the abort flag makes all remaining waits return at once.
    uint32_t last_base = 0;
    for (uint32_t base = 0; base < nkb; base += slots) {
        last_base = base;
        const uint32_t cnt = min(slots, nkb - base);
        const uint32_t parity = (base / slots) & 1u;
        for (uint32_t i = half; i < cnt && ok; i += 2) {
            if (!ptx::mbar_wait(ptx::smem_u32(bars + i), parity, abort_flag, args.fault, kFaultGemvWait)) {
                ok = false;
                break;
            }
            const uint8_t *blk = sW + i * kI4CxBlockBytes;
            const uint8_t *act = sAct + (size_t)(base + i) * MR * 128u;
            rsum += (int32_t) reinterpret_cast<const int16_t *>(blk + kI4NibBytes)[r];
#pragma unroll
            for (uint32_t seg = 0; seg < 4; ++seg) {
                const uint4 w = *reinterpret_cast<const uint4 *>(blk + r * 64u + ((seg ^ swz) << 4));
                const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int mi = 0; mi < MR; ++mi) {
                    // activation words for k = 32*seg .. +31 of row mi (same address for the whole warp: broadcast)
                    const uint4 a0 = *reinterpret_cast<const uint4 *>(act + mi * 128u + seg * 32u);
                    const uint4 a1 = *reinterpret_cast<const uint4 *>(act + mi * 128u + seg * 32u + 16u);
                    const uint32_t al[4] = {a0.x, a0.y, a0.z, a0.w};
                    const uint32_t ah[4] = {a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[mi] = __dp4a((int)al[j], (int)((ws[j] << 4) & 0xF0F0F0F0u), acc[mi]);
                        acc2[mi] = __dp4a((int)ah[j], (int)(ws[j] & 0xF0F0F0F0u), acc2[mi]);
                    }
                }
            }
        }
        if (base + slots < nkb) {
            // next round re-uses the slots: everyone must be done reading them
            __syncthreads();
            if (tid == 0 && !*abort_flag) {
                const uint32_t next = min(slots, nkb - (base + slots));
                for (uint32_t i = 0; i < next; ++i) {
                    const uint32_t bar = ptx::smem_u32(bars + i);
                    ptx::mbar_arrive_expect_tx(bar, (uint32_t)kI4CxBlockBytes);
                    ptx::bulk_g2s(ptx::smem_u32(sW + i * kI4CxBlockBytes),
                                  wsrc + (size_t)(base + slots + i) * kI4CxBlockBytes, (uint32_t)kI4CxBlockBytes, bar);
                }
                last_base = base + slots;
            }
            __syncthreads();
        }
    }
    __syncthreads();
    const bool aborted = *abort_flag != 0;

    // combine: integer atomics into the leader's reduce buffer (exact, order-independent)
    int32_t *leader = cluster.map_shared_rank(sRed, 0);
    if (!aborted) {
#pragma unroll
        for (int mi = 0; mi < MR; ++mi) {
            const int32_t v = acc[mi] + acc2[mi];
            if (v != 0) atomicAdd(leader + mi * 128 + r, v);
        }
        if (rsum != 0) atomicAdd(leader + MR * 128 + r, rsum);
    } else if (tid == 0) {
        // bail-out: wait (bounded) for the copies of the last round issued before leaving
        const uint32_t cnt = nkb > last_base ? min(slots, nkb - last_base) : 0u;
        const uint32_t parity = (last_base / slots) & 1u;
        for (uint32_t i = 0; i < cnt; ++i) {
            const long long t0 = clock64();
            while (!ptx::mbar_try_wait(ptx::smem_u32(bars + i), parity)) {
                if (clock64() - t0 > ptx::kWaitLimitCycles) {
                    if (args.fault) atomicCAS(args.fault, 0u, (unsigned)kFaultDrainWait);
                    break;
                }
            }
        }
    }
    cluster.sync();
    if (crank == 0 && tid < 128u && !aborted) {
        const uint32_t n = ntile * 128u + r;
        if (n < args.n) {
            const int32_t rs = sRed[MR * 128 + r];
            const float sb = args.scale_b[n];
            const float bv = args.bias ? TdTraits<TD>::load(args.bias, n) : 0.0f;
#pragma unroll
            for (int mi = 0; mi < MR; ++mi) {
                if ((uint32_t)mi < args.m) {
                    int32_t a = sRed[mi * 128 + r] >> 4;  // operands were 16*q
                    a -= args.zp_a[mi] * rs;
                    const float cv = args.C ? TdTraits<TD>::load(args.C, (size_t)mi * args.ldc + n) : 0.0f;
                    const float v = w4a8_epilogue(a, args.scale_a[mi], sb, args.C != nullptr, cv, args.bias != nullptr, bv,
                                                  args.cmin, args.cmax);
                    TdTraits<TD>::store(args.D, (size_t)mi * args.ldd + n, v);
                }
            }
        }
    }
}

template <int MR, Dtype TD>
static Result launch_gemv_t(const GemvArgs &a, uint32_t csize, uint32_t ntiles, cudaStream_t st)
{
    const size_t smem = (size_t)a.slots * kI4CxBlockBytes + (size_t)a.kb_per_cta * MR * 128u + (size_t)(MR + 1) * 128 * 4 +
                        (size_t)a.slots * 8 + 64;
    auto kern = gemv_w4a8_kernel<MR, TD>;
    cudaError_t e;
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        // once per device: allow the largest footprint any call may need
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448 - 1024);
        if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
        attr_set[dev] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize, ntiles, 1);
    cfg.blockDim = dim3(kGemvThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, a);
    if (e != cudaSuccess) return Result{kLaunchFailed, (int)e};
    return Result{kOk, 0};
}

template <Dtype TD>
static Result launch_gemv_m(const GemvArgs &a, uint32_t csize, uint32_t ntiles, cudaStream_t st)
{
    if (a.m <= 1) return launch_gemv_t<1, TD>(a, csize, ntiles, st);
    if (a.m <= 2) return launch_gemv_t<2, TD>(a, csize, ntiles, st);
    if (a.m <= 4) return launch_gemv_t<4, TD>(a, csize, ntiles, st);
    if (a.m <= 8) return launch_gemv_t<8, TD>(a, csize, ntiles, st);
    return launch_gemv_t<16, TD>(a, csize, ntiles, st);
}

Result gemv_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float cmin, float cmax)
{
    if (g.m == 0 || g.n == 0) return Result{kOk, 0};
    if (g.m > 16 || g.k == 0 || g.k > 65536 || g.n > 0x7fffff00ull) return Result{kUnsupported, 0};
    if ((reinterpret_cast<uintptr_t>(g.A) & 15) || (reinterpret_cast<uintptr_t>(g.B) & 15)) return Result{kUnsupported, 0};
    GemvArgs a{};
    a.m = (uint32_t)g.m;
    a.n = (uint32_t)g.n;
    a.k = (uint32_t)g.k;
    a.A = (const uint8_t *)g.A;
    a.B = (const uint8_t *)g.B;
    a.a_kblocks_total = (uint32_t)ceil_div(g.lda, 128);
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
    a.fault = fault_word_device_ptr();
    const uint32_t KB = (uint32_t)ceil_div(g.k, 128);
    const uint32_t ntiles = (uint32_t)ceil_div(g.n, 128);
    if (ntiles > 65535) return Result{kUnsupported, 0};
    // split K across the cluster until the grid covers the GPU (portable cluster size <= 8)
    uint32_t csize = 1;
    while (csize < 8 && ntiles * csize < 120 && csize * 2 <= KB) csize *= 2;
    a.kb_per_cta = (KB + csize - 1) / csize;
    a.slots = a.kb_per_cta < kGemvMaxSlots ? a.kb_per_cta : kGemvMaxSlots;
    {
        const uint32_t mr = a.m <= 1 ? 1 : a.m <= 2 ? 2 : a.m <= 4 ? 4 : a.m <= 8 ? 8 : 16;
        const size_t smem = (size_t)a.slots * kI4CxBlockBytes + (size_t)a.kb_per_cta * mr * 128u + (size_t)(mr + 1) * 512 +
                            (size_t)a.slots * 8 + 64;
        if (smem > 220 * 1024) return Result{kUnsupported, 0};
    }
    cudaStream_t st = (cudaStream_t)g.stream;
    switch (td) {
        case Dtype::F32: return launch_gemv_m<Dtype::F32>(a, csize, ntiles, st);
        case Dtype::F16: return launch_gemv_m<Dtype::F16>(a, csize, ntiles, st);
        default: return launch_gemv_m<Dtype::BF16>(a, csize, ntiles, st);
    }
}

}  // namespace tqt
