// C entry points over the reference's own portable C++ test helpers.
//
// TEST INFRASTRUCTURE ONLY.  This translation unit contains no arithmetic of its own: it
// includes the reference's headers from the reference checkout at build time (see
// oracle/Makefile, REF=<path>) and forwards to them, so that the restated oracle in
// tqt_oracle.c can be pinned against code the reference itself ships, and so that the
// benchmark can time the reference's CPU implementation ("kind": "reference").
// The resulting library lives in oracle/_ref/ and is never linked into the product.
#include <cstddef>
#include <cstdint>
#include <cstring>

#include "src/common/tqt_common.h"
#include "src/gemm/gemm_i8_i8/tqt_utils_i8_i8.h"
#include "test/common/data_generator.h"
#include "test/common/quantize_utils.h"
#include "test/common/reference_gemm.h"
#include "test/common/test_common.h"

using namespace torq_tile::test;

extern "C" {

// test/common/reference_gemm.cpp:92-129
void ref_gemm_i32_i8(size_t m, size_t n, size_t k, const int8_t *A, size_t lda, const int8_t *B,
                     size_t ldb, int b_transposed, const int32_t *C, size_t ldc, int32_t *D,
                     size_t ldd, int32_t clamp_min, int32_t clamp_max)
{
    reference_gemm_i32_i8(m, n, k, A, lda, B, ldb,
                          b_transposed ? BLayout::kTransposed : BLayout::kRowMajor, C, ldc, D, ldd,
                          clamp_min, clamp_max);
}

// test/common/reference_gemm.cpp:132-179, f16 output
void ref_gemm_w4a16_f16(size_t m, size_t n, size_t k, size_t bl, const void *A, size_t lda,
                        const uint8_t *B, size_t ldb, const void *scale_b, size_t ldsb,
                        const void *C, size_t ldc, void *D, size_t ldd, const void *bias,
                        float clamp_min, float clamp_max)
{
    reference_gemm_quantized_weight_mixed<float16_t, float16_t>(
        m, n, k, bl, (const float16_t *)A, lda, B, ldb, (const float16_t *)scale_b, ldsb,
        (const float16_t *)C, ldc, (float16_t *)D, ldd, (const float16_t *)bias, BiasMode::k1xN,
        (float16_t)clamp_min, (float16_t)clamp_max);
}

// test/common/reference_gemm.cpp:132-179, f32 output
void ref_gemm_w4a16_f32(size_t m, size_t n, size_t k, size_t bl, const void *A, size_t lda,
                        const uint8_t *B, size_t ldb, const void *scale_b, size_t ldsb,
                        const void *C, size_t ldc, void *D, size_t ldd, const void *bias,
                        float clamp_min, float clamp_max)
{
    reference_gemm_quantized_weight_mixed<float16_t, float>(
        m, n, k, bl, (const float16_t *)A, lda, B, ldb, (const float16_t *)scale_b, ldsb,
        (const float *)C, ldc, (float *)D, ldd, (const float *)bias, BiasMode::k1xN, clamp_min,
        clamp_max);
}

// test/common/quantize_utils.h:34-70
void ref_quantize_fp16_to_int4(size_t n, size_t k, size_t bl, const void *src, uint8_t *dst,
                               void *scale, size_t ld_scale)
{
    quantize_fp16_to_int4(n, k, bl, (const float16_t *)src, dst, (float16_t *)scale, ld_scale);
}

// src/gemm/gemm_i8_i8/tqt_utils_i8_i8.h:98-132
void ref_quantize_multiplier(double v, int32_t *mult, int32_t *shift)
{
    tqt_quantize_multiplier(v, mult, shift);
}

// test/common/test_common.h:232-240
int8_t ref_quantize_i8(float val, float scale, int32_t zp)
{
    return quantize_i8(val, scale, zp);
}

// test/common/test_common.h:280-290
void ref_fuse_zp_to_bias(int32_t *fused, const int32_t *bias, const int8_t *data, int32_t zp,
                         size_t channels, size_t channel_size)
{
    fuse_zp_to_bias(fused, bias, data, zp, channels, channel_size);
}

// The compiler's own narrowing/widening of the reference's scalar typedefs
// (src/common/tqt_common.h:27-28).
uint16_t ref_f32_to_f16(float f)
{
    float16_t h = static_cast<float16_t>(f);
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}
uint16_t ref_f32_to_bf16(float f)
{
    bfloat16_t h = static_cast<bfloat16_t>(f);
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}
float ref_f16_to_f32(uint16_t u)
{
    float16_t h;
    memcpy(&h, &u, 2);
    return static_cast<float>(h);
}
float ref_bf16_to_f32(uint16_t u)
{
    bfloat16_t h;
    memcpy(&h, &u, 2);
    return static_cast<float>(h);
}

// test/common/data_generator.{h,cpp}: the reference's seeded uniform generators.
void ref_fill_uniform_f32(float *dst, size_t rows, size_t cols, float lo, float hi, uint32_t seed)
{
    UniformRandomGenerator<float> g(lo, hi, seed);
    g.fill_matrix(dst, rows, cols);
}
void ref_fill_uniform_i8(int8_t *dst, size_t rows, size_t cols, int lo, int hi, uint32_t seed)
{
    UniformRandomGenerator<int8_t> g((int8_t)lo, (int8_t)hi, seed);
    g.fill_matrix(dst, rows, cols);
}
void ref_fill_uniform_i32(int32_t *dst, size_t rows, size_t cols, int32_t lo, int32_t hi,
                          uint32_t seed)
{
    UniformRandomGenerator<int32_t> g(lo, hi, seed);
    g.fill_matrix(dst, rows, cols);
}
void ref_fill_uniform_f16(void *dst, size_t rows, size_t cols, float lo, float hi, uint32_t seed)
{
    UniformRandomGenerator<float16_t> g(lo, hi, seed);
    g.fill_matrix((float16_t *)dst, rows, cols);
}

}  // extern "C"
