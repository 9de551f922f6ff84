// C entry point over the reference's portable float GEMM (test/common/reference_gemm.cpp:11-88: reference_gemm<TA, TD>).
//
// TEST INFRASTRUCTURE ONLY.  No arithmetic of its own: forwards to the reference's template instantiations, compiled
// from the reference checkout at build time (oracle/Makefile, REF=<path>), so that tqo_gemm_float in tqt_oracle.c can be
// pinned against the reference's own code.  Built into oracle/_ref/, never linked into the product.
#include <cstddef>
#include <cstdint>

#include "src/common/tqt_common.h"
#include "test/common/reference_gemm.h"

using namespace torq_tile::test;

namespace
{
template <typename TA, typename TD>
void run(size_t m, size_t n, size_t k, const void *A, size_t lda, const void *B, size_t ldb, int b_transposed, const void *C,
         size_t ldc, void *D, size_t ldd, const void *bias, int bias_per_row, float cmin, float cmax)
{
    reference_gemm<TA, TD>(m, n, k, static_cast<const TA *>(A), lda, static_cast<const TA *>(B), ldb,
                           b_transposed ? BLayout::kTransposed : BLayout::kRowMajor, static_cast<const TD *>(C), ldc,
                           static_cast<TD *>(D), ldd, static_cast<const TD *>(bias), bias_per_row ? BiasMode::kMx1 : BiasMode::k1xN,
                           static_cast<TD>(cmin), static_cast<TD>(cmax));
}
}  // namespace

extern "C" {

// ta / td: 0 = f32, 1 = f16, 2 = bf16.  Returns 0, or -1 for a combination the reference does not instantiate.
int ref_gemm_float(int ta, int td, size_t m, size_t n, size_t k, const void *A, size_t lda, const void *B, size_t ldb,
                   int b_transposed, const void *C, size_t ldc, void *D, size_t ldd, const void *bias, int bias_per_row,
                   float cmin, float cmax)
{
#define TQT_ARGS m, n, k, A, lda, B, ldb, b_transposed, C, ldc, D, ldd, bias, bias_per_row, cmin, cmax
    if (ta == 0 && td == 0) run<float, float>(TQT_ARGS);
    else if (ta == 1 && td == 1) run<float16_t, float16_t>(TQT_ARGS);
    else if (ta == 2 && td == 2) run<bfloat16_t, bfloat16_t>(TQT_ARGS);
    else if (ta == 2 && td == 0) run<bfloat16_t, float>(TQT_ARGS);
    else if (ta == 2 && td == 1) run<bfloat16_t, float16_t>(TQT_ARGS);
    else return -1;
#undef TQT_ARGS
    return 0;
}

}  // extern "C"
