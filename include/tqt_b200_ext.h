/*
 * Extensions of the B200 library that have no function of the same name in the reference.
 */
#ifndef TQT_B200_EXT_H
#define TQT_B200_EXT_H

#include "tqt_b200_common.h"

#ifdef __cplusplus
extern "C" {
#endif

/*
 * qai8dx: dynamic per-row asymmetric int8 quantisation of activations, fused with the LHS pack.
 * In the reference this arithmetic exists only as a test/example helper
 * (quantize_a_per_row_asym, test/gemm/test_gemm_i8_i4_rvv.cpp:40-77, with quantize_i8,
 * test/common/test_common.h:232-240); run_a_pack there takes already quantised int8.  Per row:
 *   fmin = min(0, min x), fmax = max(0, max x), s = (fmax - fmin) / 255;
 *   s == 0 -> scale 1, zero point 0, q = 0;
 *   zp = clamp(nearbyintf(-128 - fmin / s), -128, 127); q = clamp(nearbyintf(x / s) + zp, -128, 127)
 * with true IEEE division and round-half-to-even, so the int8 values are bit-identical to the
 * helper's.  A is [m,k] row-major (lda in elements) of f32 / f16 / bf16; A_packed is the packed
 * LHS layout of the qai8dxp kernel types (size from their get_a_packed_size); scale_a [m] and
 * zero_point_a [m] are device arrays.
 */
void tqt_run_quant_pack_qai8dxp_f32_128x128_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_packed,
                                                   float *scale_a, int32_t *zero_point_a);
void tqt_run_quant_pack_qai8dxp_f16_128x128_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_packed,
                                                   float *scale_a, int32_t *zero_point_a);
void tqt_run_quant_pack_qai8dxp_bf16_128x128_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_packed,
                                                    float *scale_a, int32_t *zero_point_a);
/* Quantise + GEMM in one call: the activations A (a_type 0 = f32, 1 = f16, 2 = bf16; [m, lda]) are quantised into the
 * caller's A_packed / scale_a / zero_point_a buffers (sized as for tqt_run_quant_pack_qai8dxp_*) and the W4A8 GEMM of
 * the same output type runs on them: D = clamp((A_q x B) * scale_a * scale_b + C + bias).  For 16-bit activations with
 * k <= 4096 and more than 16 rows this is ONE cooperative launch (the GEMM kernel quantises its own activations, one
 * row per warp, and crosses a grid-wide barrier before its mainloop); other shapes run the two kernels back to back.
 * Results are those of the two separate calls, bit for bit.  The grid barrier uses a file-scope device array of the
 * library: do not run two of these calls at the same time on one device (calls on one stream never do).  No
 * counterpart in the reference, whose callers quantise on the host. */
void tqt_run_quant_gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A, size_t lda, int a_type, void *A_packed, float *scale_a,
    int32_t *zero_point_a, const void *B_packed, size_t ldb, const void *C, size_t ldc, void *D, size_t ldd,
    const void *bias, float clamp_min, float clamp_max, const float *scale_b);
#if !defined(TQT_B200_NO_HALF_TYPES)
void tqt_run_quant_gemm_1xnbias_clamp_f16_qai8dxp_qsi4cxp_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A, size_t lda, int a_type, void *A_packed, float *scale_a,
    int32_t *zero_point_a, const void *B_packed, size_t ldb, const void *C, size_t ldc, void *D, size_t ldd,
    const void *bias, float16_t clamp_min, float16_t clamp_max, const float *scale_b);
void tqt_run_quant_gemm_1xnbias_clamp_bf16_qai8dxp_qsi4cxp_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A, size_t lda, int a_type, void *A_packed, float *scale_a,
    int32_t *zero_point_a, const void *B_packed, size_t ldb, const void *C, size_t ldc, void *D, size_t ldd,
    const void *bias, bfloat16_t clamp_min, bfloat16_t clamp_max, const float *scale_b);
#endif
/* Quantise + GEMM for callers that cannot allocate device memory and have no workspace to pass: a plug-in inside a
 * serving process whose memory pool already owns the whole GPU (cudaMalloc fails there), or inside a loop that cannot
 * afford cudaMalloc's device-wide synchronisation.  Same arithmetic as the call above with f32 output, but the packed
 * activations, scales and zero points live in a static device array of the library (8 MiB + 64 KiB, held by every GPU
 * that loads the library until the process exits); the call allocates nothing.
 *   Limit: m <= 8192 and tqt_get_a_packed_size_gemm_1xnbias_clamp_f32_qai8dxp_qsi4cxp_128x128_sm100a(m, k) <= 8 MiB
 *   (e.g. 2048 x 4096).  Larger calls launch nothing and leave status TQT_CUDA_UNSUPPORTED.
 *   The first call on each device looks the array's address up (with that device current): make that call before any
 *   stream capture.
 *   All calls on a device share the array: calls that overlap on the GPU (different streams) race; calls on one stream
 *   do not.  The array keeps the last call's contents; nothing in it has to be cleared between calls.
 * No counterpart in the reference, whose callers own every buffer. */
void tqt_run_quant_gemm_static_1xnbias_clamp_f32_qai8dxp_qsi4cxp_128x128_sm100a(
    size_t m, size_t n, size_t k, const void *A, size_t lda, int a_type, const void *B_packed, size_t ldb, const void *C,
    size_t ldc, void *D, size_t ldd, const void *bias, float clamp_min, float clamp_max, const float *scale_b);

/* Same quantiser with a plain row-major int8 result [m,k] (ldq in elements), for the unpacked
 * (qai8dx) kernel types and for inspection. */
void tqt_run_quant_qai8dx_f32_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_q, size_t ldq,
                                     float *scale_a, int32_t *zero_point_a);
void tqt_run_quant_qai8dx_f16_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_q, size_t ldq,
                                     float *scale_a, int32_t *zero_point_a);
void tqt_run_quant_qai8dx_bf16_sm100a(size_t m, size_t k, const void *A, size_t lda, void *A_q, size_t ldq,
                                      float *scale_a, int32_t *zero_point_a);

/* Inverse of the packers, for tests and for callers that need the plain data back. */
void tqt_run_a_unpack_i8_128x128_sm100a(size_t m, size_t k, const void *A_packed, size_t lda_packed, void *A,
                                        size_t lda);
void tqt_run_bt_unpack_qsi4cxp_128x128_sm100a(size_t n, size_t k, const void *B_packed, size_t ldb_packed,
                                              void *B, size_t ldb);
void tqt_run_bt_unpack_qsi4c2p_128x128_sm100a(size_t n, size_t k, const void *B_packed, size_t ldb_packed,
                                              void *B, size_t ldb);
void tqt_run_a_unpack_f16_128x128_sm100a(size_t m, size_t k, const void *A_packed, size_t lda_packed, void *A,
                                         size_t lda);

/*
 * Column-parallel sharding of the weight matrix across the GPUs of one node.  The reference has no
 * multi-device code; its tile-portion API (any n_idx that is a multiple of n_step, params arrays
 * indexed from the call's own origin) is what makes the shards independent.  Rank r of `world`
 * owns output columns [n_begin, n_begin + n_count): contiguous ranges whose starts are multiples
 * of 128, sizes differing by at most one 128-column block.  Every rank runs the unchanged
 * single-GPU kernels on its slice of B_packed / scale_b / bias and a replica of A.
 */
void tqt_shard_plan_n(size_t n, size_t world, size_t rank, size_t *n_begin, size_t *n_count);

/* Output replicas for the calling thread's following run_gemm calls (fused GEMM -> all-gather): every
 * element a kernel stores at address x inside the buffer [local_base, local_base + local_bytes) is also
 * stored at replica_bases[i] + (x - local_base), i < count <= 7; every replica buffer must be at least
 * local_bytes long.  While replicas are set, a run_gemm whose output range [D, D + ((m-1)*ldd + n) * sizeof(TD))
 * is not inside the registered buffer is refused with TQT_CUDA_INVALID_ARGUMENT and launches nothing (its
 * replica stores would land at arbitrary addresses of other GPUs).  The setting stays until it is cleared:
 * clear it (count = 0) in the same scope that set it, also on error paths.  The replicas are copies of the same output buffer
 * mapped from other GPUs (CUDA IPC or symmetric memory): the epilogue writes each tile to all of them with
 * plain peer stores while the mainloop of the next tile runs, so no separate collective is needed.  The
 * stores are visible to the peers once the kernel has completed; ordering against the peers' readers is the
 * caller's (a barrier after the call).  count = 0 switches it off.  Honoured by the packed W4A8 and W4A16
 * kernel types on their tensor-core path; any other run_gemm reports TQT_CUDA_UNSUPPORTED while replicas
 * are set.  No counterpart in the reference, whose kernels write one buffer. */
void tqt_cuda_set_output_replicas(const void *local_base, size_t local_bytes, void *const *replica_bases, size_t count);

/* Which device kernel a run_gemm call of the given shape would launch: 0 = tcgen05 tensor-core
 * GEMM, 1 = HBM-streaming GEMV (m <= 16), 2 = generic CUDA-core kernel (unpacked operands). */
int tqt_cuda_kernel_choice_w4a8(size_t m, size_t n, size_t k);

/* Diagnostic for tests: the kernel family the process's most recent int8 x int8 launch used.  0 = none yet,
 * 1 = generic CUDA-core kernel, 2 = tcgen05 CTA-pair kernel on packed blocks, 3 = tcgen05 CTA-pair kernel with a
 * row-major operand fetched by tiled TMA loads (taken when the operand's base address and row stride are
 * multiples of 16 bytes; other row-major operands run on the generic kernel). */
int tqt_cuda_debug_last_kernel(void);

/* Test switch: force a kernel path ("auto" | "umma" | "gemv" | "simt") and a tensor-core kernel ("single" |
 * "pair" | "ts"; NULL = automatic) for all later run_gemm calls of the process, replacing what the environment
 * variables TQT_B200_PATH / TQT_B200_UMMA (read once, at the first call) gave.  A forced path that cannot take a
 * call reports TQT_CUDA_UNSUPPORTED. */
void tqt_cuda_debug_set_path(const char *path, const char *umma);

/* Test knob for the failure path.  Every wait inside the tensor-core kernels (on an mbarrier that a bulk copy,
 * an MMA or another warp completes) is bounded: a wait that runs out records a code that
 * tqt_cuda_read_device_fault() returns (0x100 producer, 0x200 / 0x300 MMA issuer, 0x400 epilogue, 0x500
 * converter, 0x700 producer draining its copies), the CTA stops issuing work, lets its copies land, frees its
 * tensor memory and returns without storing the tile; the context stays usable.  wait_shift shortens every
 * limit (about one second) by that many binary orders of magnitude; flags bit 0 makes one producer warp of the
 * packed W4A8 / W4A16 tensor-memory kernels withhold the copies and the barrier arrive of its first stage, so
 * that the waits downstream of it run out.  Process-wide, for the launches that follow; (0, 0) restores normal
 * operation.  Nothing traps, faults or spins without a limit. */
void tqt_cuda_debug_inject_wait_failure(unsigned wait_shift, unsigned flags);

/* Diagnostic: install a caller-owned device buffer of 16 int64 per CTA (148 CTAs at most) that the
 * tensor-core GEMM fills with the cycles each warp role spent waiting (producer, MMA issuer, one
 * epilogue warp, one converter warp: {wait0, wait1, wait2, total} each), and the one-row GEMV with six phase stamps per CTA.
 * NULL switches it off.  The kernels contain this instrumentation only when the library was built with -DTQT_B200_DIAG
 * (their hot loops are sensitive to code size); an ordinary build accepts the call and leaves the buffer untouched. */
void tqt_cuda_debug_set_timing_buffer(void *dev_ptr);

/* Diagnostic: launch, on the calling thread's stream, a kernel with the GEMV's launch shape (thread
 * count, loads in flight, programmatic dependent launch) that only reads `bytes` bytes from the
 * device buffer src (16-byte aligned) and computes nothing: the read ceiling the GEMV's achieved
 * bandwidth is compared with at a given size.  sink: 128 bytes of device memory, or NULL. */
void tqt_cuda_debug_stream_read(const void *src, size_t bytes, void *sink);

#if !defined(TQT_B200_NO_HALF_TYPES)
/* Return the bit pattern of a 16-bit float received by value: lets a foreign-function binding
 * verify how it passes the clamp arguments of the f16 / bf16 kernel types. */
uint16_t tqt_cuda_debug_f16_bits(float16_t v);
uint16_t tqt_cuda_debug_bf16_bits(bfloat16_t v);
#endif

#ifdef __cplusplus
}
#endif

#endif /* TQT_B200_EXT_H */
