/*
 * TORQ-Tile quantized GEMM micro-kernels for NVIDIA B200 (sm_100a): common definitions.
 *
 * The entry points declared in the tqt_b200_gemm_*.h headers keep the names, argument lists and
 * tile-portion semantics of the reference's stateless C micro-kernel API
 * (tqt_<action>_<kernel-type>_<variant>, reference README.md:67-92), with the variant suffix
 * "_128x128_sm100a" in place of "_4x1vl_rvv" / "_8x2vl_rvv".
 *
 * Conventions that differ from the CPU library because the kernels run on a GPU:
 *   - every data pointer (A, B, C, D, bias, packed buffers, and the arrays the params structs
 *     point to) is a DEVICE pointer valid on the calling thread's current CUDA device;
 *   - params structs themselves are HOST structs, read at call time;
 *   - run_* functions enqueue work on the stream chosen with tqt_cuda_set_stream() (default:
 *     the legacy default stream) and return without waiting;
 *   - the library allocates nothing and keeps no state besides that per-thread stream and the
 *     per-thread status word.
 *
 * Error convention: like the reference (src/common/tqt_common.h:61-91, void returns, params ==
 * NULL returns silently) the run_* functions return void.  Instead of aborting the process they
 * record a status readable with tqt_cuda_get_last_status().
 */
#ifndef TQT_B200_COMMON_H
#define TQT_B200_COMMON_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Scalar typedefs as in the reference (src/common/tqt_common.h:27-28).  They appear by value in
 * the clamp arguments of the f16 / bf16 kernel types, so translation units that include those
 * prototypes must be compiled by a compiler that knows the types (gcc >= 12, clang >= 15). */
#if !defined(TQT_B200_NO_HALF_TYPES)
typedef __bf16 bfloat16_t;
typedef _Float16 float16_t;
#endif

/* Tile granularity of every "_128x128_sm100a" variant: start indices passed to the offset helpers
 * and to run_* must be multiples of these (reference: m_step = 4, n_step = VLENB).  K-slab indices
 * (k_idx) must be multiples of TQT_B200_K_STEP. */
#define TQT_B200_M_STEP 128
#define TQT_B200_N_STEP 128
#define TQT_B200_K_STEP 128

enum tqt_cuda_status {
    TQT_CUDA_OK = 0,
    TQT_CUDA_INVALID_ARGUMENT = 1,  /* a precondition the reference would TQT_ASSUME failed */
    TQT_CUDA_LAUNCH_FAILED = 2,     /* the CUDA runtime refused the launch; see ..._cuda_error() */
    TQT_CUDA_UNSUPPORTED = 3        /* shape or alignment outside what this variant accepts */
};

/* Stream used by the calling thread's subsequent run_* calls (a cudaStream_t passed as void*). */
void tqt_cuda_set_stream(void *stream);
void *tqt_cuda_get_stream(void);
/* Status of the calling thread's most recent run_* call, and the cudaError_t behind a
 * TQT_CUDA_LAUNCH_FAILED.  No device synchronisation is performed. */
int tqt_cuda_get_last_status(void);
int tqt_cuda_get_last_cuda_error(void);
/* Device-side watchdog: kernels bound every wait on a barrier; a wait that runs out sets a
 * non-zero code in a per-device word that this call reads (after synchronising the stream). */
int tqt_cuda_read_device_fault(void);
/* Library version string, e.g. "torq-tile-b200 0.1 (sm_100a)". */
const char *tqt_cuda_version(void);

#ifdef __cplusplus
}
#endif

#endif /* TQT_B200_COMMON_H */
