// C entry points over the W4A8 helpers of the reference's own gtest suite.
//
// TEST INFRASTRUCTURE ONLY.  The reference keeps its dynamic-activation quantiser, its int4
// per-channel weight quantiser and its W4A8 fp32 oracle in an anonymous namespace inside
// test/gemm/test_gemm_i8_i4_rvv.cpp (a gtest translation unit that cannot be built without gtest
// and the RVV kernels).  The build recipe (oracle/Makefile, target "ref") cuts exactly that
// anonymous namespace out of the file where it lies in the reference checkout into the generated
// file oracle/_ref/w4a8_helpers.gen.inc (not committed, rebuilt every time), and this translation
// unit includes it unchanged.  Nothing below computes anything: it forwards to those functions and
// narrows the fp32 result through the output type exactly as the suite does
// (test/gemm/test_gemm_i8_i4_rvv.cpp:296-299), so that the restated oracle in tqt_oracle.c can be
// pinned bit for bit against code the reference itself ships.
#include <algorithm>
#include <cfloat>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <vector>

#include "src/common/tqt_common.h"
#include "test/common/data_generator.h"
#include "test/common/test_common.h"

using namespace torq_tile::test;

// The helpers call std::fabsf, which libstdc++ only declares from GCC 14 on; the C library's
// ::fabsf is the same function (the toolchain here is g++ 13).
#if defined(__GLIBCXX__) && __GNUC__ < 14
namespace std
{
using ::fabsf;
}
#endif

#include "w4a8_helpers.gen.inc"   // quantize_a_per_row_asym, quantize_b_per_channel_sym_int4, w4a8_reference_fp32

namespace
{
template <typename TD>
void run_w4a8(size_t m, size_t n, size_t k, const int8_t *A, const uint8_t *B, const float *scale_a,
              const int32_t *zp_a, const float *scale_b, const void *C, const void *bias, void *D,
              float clamp_min, float clamp_max)
{
    // the suite widens C and bias to fp32 first (test_gemm_i8_i4_rvv.cpp:271-283)
    std::vector<float> c32, b32;
    if (C) {
        c32.resize(m * n);
        for (size_t i = 0; i < m * n; ++i) c32[i] = to_float(static_cast<const TD *>(C)[i]);
    }
    if (bias) {
        b32.resize(n);
        for (size_t i = 0; i < n; ++i) b32[i] = to_float(static_cast<const TD *>(bias)[i]);
    }
    std::vector<float> d32(m * n);
    w4a8_reference_fp32(m, n, k, A, B, scale_a, zp_a, scale_b, C ? c32.data() : nullptr,
                        bias ? b32.data() : nullptr, d32.data(), clamp_min, clamp_max);
    for (size_t i = 0; i < m * n; ++i) static_cast<TD *>(D)[i] = to_target_type<TD>(d32[i]);
}
}  // namespace

extern "C" {

// test/gemm/test_gemm_i8_i4_rvv.cpp:40-77
void ref_w4a8_quantize_a_per_row_asym(const float *A, size_t m, size_t k, int8_t *A_i8, float *scale_a,
                                      int32_t *zp_a)
{
    quantize_a_per_row_asym(A, m, k, A_i8, scale_a, zp_a);
}

// test/gemm/test_gemm_i8_i4_rvv.cpp:82-118
void ref_w4a8_quantize_b_per_channel_sym_int4(const float *B, size_t n, size_t k, uint8_t *B_packed,
                                              float *scale_b)
{
    quantize_b_per_channel_sym_int4(B, n, k, B_packed, scale_b);
}

// test/gemm/test_gemm_i8_i4_rvv.cpp:122-156 followed by the cast through TD (:296-299).
// td: 0 = f32, 1 = f16, 2 = bf16; C, bias and D are TD arrays ([m,n] dense, [n], [m,n] dense).
void ref_w4a8_gemm(size_t m, size_t n, size_t k, const int8_t *A, const uint8_t *B, const float *scale_a,
                   const int32_t *zp_a, const float *scale_b, const void *C, const void *bias, void *D,
                   float clamp_min, float clamp_max, int td)
{
    if (td == 0)
        run_w4a8<float>(m, n, k, A, B, scale_a, zp_a, scale_b, C, bias, D, clamp_min, clamp_max);
    else if (td == 1)
        run_w4a8<float16_t>(m, n, k, A, B, scale_a, zp_a, scale_b, C, bias, D, clamp_min, clamp_max);
    else
        run_w4a8<bfloat16_t>(m, n, k, A, B, scale_a, zp_a, scale_b, C, bias, D, clamp_min, clamp_max);
}

// test/common/data_generator.{h,cpp}: the 16-bit generators the suite draws C and bias with.
void ref_fill_uniform_bf16(void *dst, size_t rows, size_t cols, float lo, float hi, uint32_t seed)
{
    UniformRandomGenerator<bfloat16_t> g(lo, hi, seed);
    g.fill_matrix((bfloat16_t *)dst, rows, cols);
}

}  // extern "C"
