// Internal interface between the C-ABI shim (abi.cpp, compiled by g++) and the CUDA launchers
// (*.cu, compiled by nvcc).  Plain C++ types only: no half types, no CUDA headers.
#pragma once

#include <cstddef>
#include <cstdint>

namespace tqt {

// ---- packed layouts --------------------------------------------------------------------------
// Every packed operand is an array of blocks [ceil(rows/128)][ceil(k/KB)] of fixed size.
constexpr size_t kTileRows = 128;
constexpr size_t kI8BlockK = 128;        // int8 elements per block row (128 bytes)
constexpr size_t kI8BlockBytes = 16384;  // 128 rows x 128 B, 128-byte-swizzled
constexpr size_t kI8SumBlockBytes = kI8BlockBytes + 256;  // int8 block + 128 int16 partial row sums (qsi8cxp of the dynamic-activation types)
constexpr size_t kF16BlockK = 64;        // f16 elements per block row (128 bytes)
constexpr size_t kF16BlockBytes = 16384;
constexpr size_t kI4BlockK = 128;        // int4 elements per block row (64 bytes)
constexpr size_t kI4NibBytes = 8192;     // 128 rows x 64 B
constexpr size_t kI4CxBlockBytes = kI4NibBytes + 256;  // + 128 int16 partial row sums
constexpr size_t kI4C2BlockBytes = kI4NibBytes;

inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

enum class Dtype : int { F32 = 0, F16 = 1, BF16 = 2 };

enum Status : int { kOk = 0, kInvalid = 1, kLaunchFailed = 2, kUnsupported = 3 };

// Result of a launcher: status + raw cudaError_t (0 when none).
struct Result {
    int status;
    int cuda_error;
};

// ---- pack / unpack / quantise ---------------------------------------------------------------
// elem_size 1 (int8) or 2 (f16).  transposed_src: source is [k, rows] row-major (run_b_pack).
Result launch_pack_rows(void *stream, size_t rows, size_t k, size_t ld_src, size_t ld_packed, const void *src,
                        void *dst, int elem_size, bool transposed_src);
// int8 rows into blocks of kI8SumBlockBytes, then the int16 partial row sums of every block (the zero-point
// correction term of the qai8dxp x qsi8cxp types).
Result launch_pack_rows_sums(void *stream, size_t rows, size_t k, size_t ld_src, size_t ld_packed, const void *src,
                             void *dst, bool transposed_src);
Result launch_unpack_rows(void *stream, size_t rows, size_t k, size_t ld_packed, const void *src, void *dst,
                          size_t ld_dst, int elem_size);
// int4: src [n, k/2] bytes, row stride ld_src_bytes.  c2 = qsi4c2 ordering (no row sums).
Result launch_pack_i4(void *stream, size_t n, size_t k, size_t ld_src_bytes, size_t ld_packed, const void *src,
                      void *dst, bool c2);
Result launch_unpack_i4(void *stream, size_t n, size_t k, size_t ld_packed, const void *src, void *dst,
                        size_t ld_dst_bytes, bool c2);
// qai8dx quantiser.  packed: write the swizzled block layout, else row-major with stride ldq.
Result launch_quant_qai8dx(void *stream, size_t m, size_t k, const void *A, size_t lda, Dtype ta, void *out,
                           size_t ldq, bool packed, float *scale_a, int32_t *zp_a);

// ---- GEMM ------------------------------------------------------------------------------------
struct GemmCommon {
    size_t m, n, k;
    const void *A;
    size_t lda;  // row-major A: elements; packed A: k extent the buffer was packed with
    const void *B;
    size_t ldb;  // same for B
    const void *C;
    size_t ldc;
    void *D;
    size_t ldd;
    const void *bias;
    void *stream;
    // Output replicas: every element stored at address x of D is also stored at x + replica_delta[i]
    // (peer-mapped copies of the output buffer on other GPUs).  Honoured by the tensor-memory kernels
    // of the W4A8 / W4A16 packed types; other paths report kUnsupported while replicas are set.
    size_t n_replicas;
    long long replica_delta[7];
};

enum class Path : int { Auto = 0, Umma = 1, Gemv = 2, Simt = 3 };

// D(int32) = clamp(C + A*B).  packed: both operands in the int8 block layout; else A [m,k], B [k,n].
Result launch_gemm_i32(const GemmCommon &g, bool packed, int32_t clamp_min, int32_t clamp_max, Path path);

struct RequantParams {
    float scale_a;
    const float *scale_b;  // device
    int quant_channel_b;
    float scale_d;
    int32_t zero_point_d;
};
// Static W8A8 with int8 output (packed operands).
Result launch_gemm_requant_i8(const GemmCommon &g, const RequantParams &p, int clamp_min, int clamp_max,
                              Path path);

struct W4A8Params {
    const float *scale_a;  // device [m]
    const int32_t *zp_a;   // device [m]
    const float *scale_b;  // device [n]
};
// W4A8, float output of type td (C, bias typed like D).
Result launch_gemm_w4a8(const GemmCommon &g, const W4A8Params &p, Dtype td, float clamp_min, float clamp_max,
                        Path path);

// Quantise + W4A8 GEMM with the intermediates in the library's own static device array (static_scratch.cu); g.A / g.lda
// are filled in by the callee.  kUnsupported when the call exceeds the array.
Result quant_gemm_w4a8_static(GemmCommon g, const void *A, size_t lda, Dtype ta, const float *scale_b, Dtype td,
                              float clamp_min, float clamp_max);

// W4A16 block-quant; A f16 packed, B qsi4c2 packed; td F16 or F32.
Result launch_gemm_w4a16(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td,
                         float clamp_min, float clamp_max, Path path);

// ---- sibling kernel types (generic CUDA-core path) --------------------------------------------
// How an operand is stored: Packed = the 128 x 128 block layout; RowMajor = [rows, k] with stride ld
// (rows = m for A, n for B: the reference's "t" layouts); KMajor = [k, rows] with stride ld.
enum class Layout : int { Packed = 0, RowMajor = 1, KMajor = 2 };

// 1xN-bias requantising GEMM with any operand layouts.
Result launch_gemm_requant_i8_layouts(const GemmCommon &g, const RequantParams &p, int clamp_min, int clamp_max,
                                      Layout la, Layout lb);

struct RowRequantParams {
    const float *scale_a;  // device [m] (one value when quant_channel_a == 1)
    int quant_channel_a;
    float scale_b;
    float scale_d;
    int32_t zero_point_d;
};
// Mx1-bias requantising GEMM (per-row scale of A), bias int32 [m].
Result launch_gemm_requant_rows_i8(const GemmCommon &g, const RowRequantParams &p, int clamp_min, int clamp_max,
                                   Layout la, Layout lb);

// qai8dx x qsi8cx, float output of type td (F32 or F16); C is ignored, bias typed like D.  A packed B is in
// the blocks-with-sums layout (kI8SumBlockBytes).
Result launch_gemm_dxcx(const GemmCommon &g, const W4A8Params &p, Dtype td, float clamp_min, float clamp_max,
                        Layout la, Layout lb);

// W4A8 on unpacked operands: A int8 [m, lda], B nibbles [n, ldb / 2 bytes] (low nibble = even k, value q + 8).
Result launch_gemm_w4a8_unpacked(const GemmCommon &g, const W4A8Params &p, Dtype td, float clamp_min,
                                 float clamp_max);

// W4A16 on unpacked operands: A f16 [m, lda], B nibbles [n, ldb / 2 bytes], scale_b [n, ldsb] f16.
Result launch_gemm_w4a16_unpacked(const GemmCommon &g, size_t bl, const void *scale_b, size_t ldsb, Dtype td,
                                  float clamp_min, float clamp_max);

// ---- int8 convolution wrappers: im2col ---------------------------------------------------------
// Geometry of one group of a convolution, every extent checked by the caller to fit 31 bits: index 0 = depth,
// 1 = height, 2 = width.  rows = output positions, k = kernel volume x channels per group.
struct ConvGeom {
    uint32_t in[3], out[3], ker[3], stride[3], dil[3], pad[3];
    uint32_t c_total;  // channels of the whole input tensor
    uint32_t ic_pg;    // input channels per group
    uint32_t c_off;    // first channel of this group
    uint32_t rows, k;
};
// Gather into the packed int8 block layout (rows = output positions).  channel_first: input [C, D, H, W], K order
// (ic, kd, kh, kw); else input [D, H, W, C], K order (kd, kh, kw, ic).
Result launch_im2col_pack_i8(void *stream, const ConvGeom &g, bool channel_first, const void *activation, size_t ld_packed,
                             void *packed);
// Gather into a plain matrix: [rows, k] for channel-last, [k, rows] for channel-first.
Result launch_im2col_i8(void *stream, const ConvGeom &g, bool channel_first, const void *activation, void *matrix);

// W4A8 GEMM that quantises its own activations (16-bit [m, q_lda]) into g.A, p.scale_a, p.zp_a before its mainloop: one
// cooperative launch.  kUnsupported when the shape has no fused form (the caller then launches quantiser and GEMM).
Result umma_gemm_w4a8_fusedq(const GemmCommon &g, const W4A8Params &p, Dtype td, float clamp_min, float clamp_max,
                             const void *q_in, size_t q_lda, bool q_bf16);

// Unquantised GEMM (kernels_float.cu, kernels_pair.cu): operands of type ta in layouts la / lb (A never KMajor), C, bias
// and D of type td, bias per column or per row.
Result launch_gemm_float(const GemmCommon &g, Dtype ta, Dtype td, float clamp_min, float clamp_max, Layout la, Layout lb,
                         bool bias_per_row);

// Implicit-GEMM convolutions: see kernels_simt.cu.
Result launch_igemm_cl_requant_i8(const GemmCommon &g, const ConvGeom &geom, uint32_t pos0, const void *input,
                                  const RequantParams &p, int clamp_min, int clamp_max, Layout weights);
Result launch_igemm_cf_requant_rows_i8(const GemmCommon &g, const ConvGeom &geom, uint32_t pos0, const void *input,
                                       const RowRequantParams &p, int clamp_min, int clamp_max, Layout weights);

// Reads (and clears) the device-side watchdog word of the current device after synchronising
// the stream.  0 = no fault.
int read_device_fault(void *stream);

// Diagnostic: device buffer of 16 int64 per CTA that the tensor-core GEMM fills with per-role wait cycles
// (nullptr switches it off).  Owned by the caller.
void set_timing_buffer(void *dev_ptr);

// Test knob of the tensor-core kernels' bounded waits: shift every wait limit right by wait_shift (10: about a
// millisecond) and, with bit 0 of flags, make the first producer warp of the tensor-memory kernels withhold its
// first stage, so that a wait runs out and the kernel returns with a fault code.  (0, 0) = normal operation.
void set_failure_injection(unsigned wait_shift, unsigned flags);

// Diagnostic: launch a kernel with the GEMV's launch shape that only reads `bytes` from src (16-byte aligned).
Result stream_read(const void *src, size_t bytes, void *sink, void *stream);

// Path / tensor-core kernel overrides (tests): TQT_B200_PATH = auto|umma|gemv|simt and TQT_B200_UMMA =
// single|pair|ts are read from the environment once; set_path_switches replaces both at run time (nullptr or an
// unknown word = automatic choice).  umma_variant: 0 automatic, 1 single CTA, 2 CTA pair, 3 single-CTA
// tensor-memory kernel.
Path env_path();
// Diagnostic for tests: which kernel family the most recent int8 x int8 launch of the process used (kKernel*).
enum : int { kKernelNone = 0, kKernelSimt = 1, kKernelPairBlocks = 2, kKernelPairTma = 3, kKernelTsTma = 4, kKernelTsFusedQuant = 5 };
void note_kernel(int family);
int last_kernel();
int umma_variant();
void set_path_switches(const char *path, const char *umma);

}  // namespace tqt
