// Thin inline-PTX wrappers for the sm_100a features the kernels use: mbarrier, bulk async copies
// (TMA, untiled form), tensor memory and tcgen05.mma.  Every wait is bounded by a cycle budget.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace tqt {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// try_wait suspends the thread in hardware until the phase completes or this many nanoseconds have
// passed, so that waiting warps do not compete for issue slots with the warps that do the work.
constexpr uint32_t kTryWaitSuspendNs = 20000;

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns = kTryWaitSuspendNs)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Non-blocking test of a phase: cheaper than try_wait, which may suspend the thread.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity, uint32_t hint_ns = kTryWaitSuspendNs)
{
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// About one second at B200 clocks.  A wait that exceeds it records `code` in *fault, raises the
// CTA-wide abort flag and returns false; every other wait in the CTA then returns false promptly.
// The abort flag is a pair of ints in shared memory: [0] the flag, [1] a right shift applied to the limit
// (0 in normal use; a test makes a wait run out in about a millisecond with 10).
constexpr long long kWaitLimitCycles = 2000000000ll;
__device__ __forceinline__ long long wait_limit(volatile int *abort_flag) { return kWaitLimitCycles >> (abort_flag[1] & 31); }

// Bounded wait.  Every polling thread spins on try_wait, which itself suspends the thread in hardware for up to
// hint_ns nanoseconds (sleeping between polls in software was measured to cost throughput, because the pipelines
// are latency-sensitive).
// The polling loop with its time limit is one out-of-line function: inlined at every wait it made the kernels' hot
// loops several times longer, and they are sensitive to code size.  The inlined part is a single test.
template <bool CLUSTER>
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned int *fault,
                                            unsigned int code, uint32_t hint_ns)
{
    const long long t0 = clock64();
    unsigned int spins = 0;
    for (;;) {
        if (CLUSTER ? mbar_try_wait_cluster(bar, parity, hint_ns) : mbar_try_wait(bar, parity, hint_ns)) return true;
        if ((++spins & 31u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > wait_limit(abort_flag)) {
                *abort_flag = 1;
                if (fault) atomicCAS(fault, 0u, code);
                return false;
            }
        }
    }
}

template <bool CLUSTER>
__device__ __forceinline__ bool mbar_wait_impl(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                               unsigned int *fault, unsigned int code, uint32_t hint_ns)
{
    if (!CLUSTER && hint_ns == 0u) {
        if (mbar_test_wait(bar, parity)) return true;   // the common case on the critical loops: already complete
    } else if (CLUSTER ? mbar_try_wait_cluster(bar, parity, hint_ns) : mbar_try_wait(bar, parity, hint_ns)) {
        return true;
    }
    return mbar_wait_slow<CLUSTER>(bar, parity, abort_flag, fault, code, hint_ns);
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          unsigned int *fault, unsigned int code, uint32_t hint_ns = kTryWaitSuspendNs)
{
    return mbar_wait_impl<false>(bar, parity, abort_flag, fault, code, hint_ns);
}

// ---- async proxy ------------------------------------------------------------------------------------
// Makes generic-proxy shared-memory writes visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Untiled bulk copy global -> shared, completion reported as transaction bytes on an mbarrier.
// dst and src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Tiled TMA load of one 2-D box global -> shared through a tensor map (a 128-byte opaque descriptor the host encodes
// with cuTensorMapEncodeTiled and passes as a __grid_constant__ kernel parameter), completion as transaction bytes
// on an mbarrier of this CTA.  x is the coordinate along the contiguous dimension: x times the element size must be a
// multiple of 16 bytes.  Cells outside the tensor read as zero and still count towards the box's bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const void *tensor_map, int32_t x, int32_t y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     dst_smem),
                 "l"(tensor_map), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const void *tensor_map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}

// ---- tensor memory --------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on the mbarrier when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st()
{
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

// 32 lanes x 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

// ---- tcgen05.mma -------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand stored as rows of 128 bytes with the
// 128-byte swizzle, 8-row groups 1024 bytes apart (the layout a 128-byte-swizzled TMA box, or our
// pre-swizzled packed blocks, produce).  Bits: [0,14) address>>4, [16,30) leading byte offset>>4
// (unused for swizzled K-major, set to 1), [32,46) stride byte offset>>4 (1024>>4), [46,48) version 1,
// [61,64) layout type 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_desc_k_sw128(uint32_t smem_addr)
{
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

// Instruction descriptor (dense, no negate, both operands K-major):
// [4,6) D format (0 f16, 1 f32, 2 s32); [7,10) A format; [10,13) B format; bit 15 / 16: A / B operand MN-major;
// [17,23) N>>3; [24,29) M>>4.
// kind::i8 formats: 0 = u8, 1 = s8.  kind::f16 formats: 0 = f16, 1 = bf16.
// The same descriptor with explicit byte offsets: lbo between 128-byte-wide groups along the operand's M / N dimension
// (MN-major operands wider than one group), sbo between groups of 8 rows.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr, uint32_t lbo, uint32_t sbo)
{
    return (uint64_t)((smem_addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) | ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) |
           (1ull << 46) | (2ull << 61);
}

constexpr uint32_t kIdescBMajorMn = 1u << 16;   // N-side operand MN-major (its rows run along K in shared memory)
__host__ __device__ constexpr uint32_t make_idesc(uint32_t d_fmt, uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n)
{
    return (d_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem], int8 inputs, int32 accumulate, K = 32 per instruction.
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Same with the M-side operand in tensor memory (lane = row, four int8 per 32-bit column).
__device__ __forceinline__ void mma_i8_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Same with f16 inputs, f32 accumulate, K = 16 per instruction.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}


// ---- thread-block clusters and CTA pairs (cta_group::2) ---------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the variable at the same offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
// arrive on an mbarrier given by a shared::cluster address (possibly in the peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// bounded wait with cluster-scope acquire (the arrivals may come from the peer CTA)
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                                  unsigned int *fault, unsigned int code, uint32_t hint_ns = kTryWaitSuspendNs)
{
    return mbar_wait_impl<true>(bar, parity, abort_flag, fault, code, hint_ns);
}
// Hardware cluster barrier: every thread of both CTAs arrives; cannot be bounded, so it is only
// used where all paths provably reach it (kernel prologue and teardown).
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Completion of all prior MMAs of this thread arrives once on the barrier at this offset in every
// CTA of `cta_mask` (an arrive broadcast, not a data copy).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"(cta_mask)
                 : "memory");
}
// Pair MMA, issued by one thread of the leader CTA: M = 256 (128 rows per CTA), each CTA supplies
// half of the N-side operand from its own shared memory.
__device__ __forceinline__ void mma_i8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Same with the M-side operand in tensor memory (each CTA's own 128 lanes).
__device__ __forceinline__ void mma_i8_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_f16_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The four K slices of one K step of the CTA-pair SS MMA in one instruction block (only the low words of the two
// descriptors advance, by two 16-byte units per K slice of 32 bytes).
// BSTEP: distance between the N-side operand's K slices in 16-byte units: 2 for a K-major stage (32 bytes along a row),
// 256 for an MN-major one (32 rows of 128 bytes).
template <uint32_t BSTEP = 2>
__device__ __forceinline__ void mma_i8_ss_pair_group4(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                      uint32_t idesc, uint32_t accum_first)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p, pt;\n\t"
        ".reg .b32 la, lb;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %5, p;\n\t"
        "add.u32 la, %1, 2;\n\t add.u32 lb, %3, %7;\n\t mov.b64 da, {la, %2};\n\t mov.b64 db, {lb, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %5, pt;\n\t"
        "add.u32 la, %1, 4;\n\t add.u32 lb, %3, %8;\n\t mov.b64 da, {la, %2};\n\t mov.b64 db, {lb, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %5, pt;\n\t"
        "add.u32 la, %1, 6;\n\t add.u32 lb, %3, %9;\n\t mov.b64 da, {la, %2};\n\t mov.b64 db, {lb, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %5, pt;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accum_first), "n"(BSTEP), "n"(2 * BSTEP),
          "n"(3 * BSTEP)
        : "memory");
}

// The same block for 16-bit floating-point operands (kind::f16: f16 or bf16 by the instruction descriptor, f32
// accumulation, K = 16 per instruction = 32 bytes, so the descriptors step as for int8).
template <uint32_t BSTEP = 2>
__device__ __forceinline__ void mma_f16_ss_pair_group4(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                       uint32_t idesc, uint32_t accum_first)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p, pt;\n\t"
        ".reg .b32 la, lb;\n\t"
        ".reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "mov.b64 da, {%1, %2};\n\t mov.b64 db, {%3, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t"
        "add.u32 la, %1, 2;\n\t add.u32 lb, %3, %7;\n\t mov.b64 da, {la, %2};\n\t mov.b64 db, {lb, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, pt;\n\t"
        "add.u32 la, %1, 4;\n\t add.u32 lb, %3, %8;\n\t mov.b64 da, {la, %2};\n\t mov.b64 db, {lb, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, pt;\n\t"
        "add.u32 la, %1, 6;\n\t add.u32 lb, %3, %9;\n\t mov.b64 da, {la, %2};\n\t mov.b64 db, {lb, %4};\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, pt;\n\t"
        "}"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accum_first), "n"(BSTEP), "n"(2 * BSTEP),
          "n"(3 * BSTEP)
        : "memory");
}

// A group of eight TS MMAs (two K steps of four K slices) in one instruction block, to keep the issuing
// thread's instruction count per MMA at its minimum (the thread is the bottleneck of the mainloop).  MMA q = 4 h + j
// takes its M-side operand at a_tmem + 8 q, its N-side descriptor at desc + h * stage16 + 2 j (only the low word of
// the descriptor changes: the address field counts 16-byte units), accumulates unless it is the very first of a tile
// (accum_first = 0).  two_steps = 0 issues the first four only.
#define TQT_MMA_TS_GROUP8(NAME, KINDSTR)                                                                                  \
    __device__ __forceinline__ void NAME(uint32_t d_tmem, uint32_t a_tmem, uint32_t desc_lo, uint32_t desc_hi,            \
                                         uint32_t stage16, uint32_t idesc, uint32_t accum_first, uint32_t two_steps)     \
    {                                                                                                                     \
        asm volatile(                                                                                                     \
            "{\n\t"                                                                                                       \
            ".reg .pred p, pt, q;\n\t"                                                                                    \
            ".reg .b32 lo, at, lo1;\n\t"                                                                                  \
            ".reg .b64 d;\n\t"                                                                                            \
            "setp.ne.b32 p, %6, 0;\n\t"                                                                                   \
            "setp.eq.b32 pt, 0, 0;\n\t"                                                                                   \
            "setp.ne.b32 q, %7, 0;\n\t"                                                                                   \
            "mov.b64 d, {%2, %3};\n\t"                                                                                    \
            "tcgen05.mma." KINDSTR " [%0], [%1], d, %5, p;\n\t"                                                           \
            "add.u32 lo, %2, 2;\n\t add.u32 at, %1, 8;\n\t mov.b64 d, {lo, %3};\n\t"                                      \
            "tcgen05.mma." KINDSTR " [%0], [at], d, %5, pt;\n\t"                                                          \
            "add.u32 lo, %2, 4;\n\t add.u32 at, %1, 16;\n\t mov.b64 d, {lo, %3};\n\t"                                     \
            "tcgen05.mma." KINDSTR " [%0], [at], d, %5, pt;\n\t"                                                          \
            "add.u32 lo, %2, 6;\n\t add.u32 at, %1, 24;\n\t mov.b64 d, {lo, %3};\n\t"                                     \
            "tcgen05.mma." KINDSTR " [%0], [at], d, %5, pt;\n\t"                                                          \
            "add.u32 lo1, %2, %4;\n\t add.u32 at, %1, 32;\n\t mov.b64 d, {lo1, %3};\n\t"                                  \
            "@q tcgen05.mma." KINDSTR " [%0], [at], d, %5, pt;\n\t"                                                       \
            "add.u32 lo, lo1, 2;\n\t add.u32 at, %1, 40;\n\t mov.b64 d, {lo, %3};\n\t"                                    \
            "@q tcgen05.mma." KINDSTR " [%0], [at], d, %5, pt;\n\t"                                                       \
            "add.u32 lo, lo1, 4;\n\t add.u32 at, %1, 48;\n\t mov.b64 d, {lo, %3};\n\t"                                    \
            "@q tcgen05.mma." KINDSTR " [%0], [at], d, %5, pt;\n\t"                                                       \
            "add.u32 lo, lo1, 6;\n\t add.u32 at, %1, 56;\n\t mov.b64 d, {lo, %3};\n\t"                                    \
            "@q tcgen05.mma." KINDSTR " [%0], [at], d, %5, pt;\n\t"                                                       \
            "}"                                                                                                           \
            :                                                                                                             \
            : "r"(d_tmem), "r"(a_tmem), "r"(desc_lo), "r"(desc_hi), "r"(stage16), "r"(idesc), "r"(accum_first),           \
              "r"(two_steps)                                                                                              \
            : "memory");                                                                                                  \
    }
TQT_MMA_TS_GROUP8(mma_i8_ts_group8, "cta_group::1.kind::i8")
TQT_MMA_TS_GROUP8(mma_f16_ts_group8, "cta_group::1.kind::f16")
TQT_MMA_TS_GROUP8(mma_i8_ts_pair_group8, "cta_group::2.kind::i8")
TQT_MMA_TS_GROUP8(mma_f16_ts_pair_group8, "cta_group::2.kind::f16")
#undef TQT_MMA_TS_GROUP8

// 32 lanes x 32 consecutive 32-bit columns, registers -> tensor memory.
__device__ __forceinline__ void tmem_st_32x32b_x32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t nthreads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace ptx
}  // namespace tqt
