// Epilogue functors: one output element at a time.  Used directly by the CUDA-core and GEMV
// kernels; the tensor-core kernel applies the same scalar functions from dev_common.cuh to the
// 32-column strips it reads from tensor memory.
#pragma once

#include "dev_common.cuh"

namespace tqt {

// D = clamp(C + acc)  (reference: gemm_clamp_i32_i8_i8, ..._4x1vl_rvv.cpp:72-101)
struct EpiI32 {
    const int32_t *C;
    size_t ldc;
    int32_t *D;
    size_t ldd;
    int32_t cmin, cmax;
    __device__ void operator()(size_t m, size_t n, int32_t acc, int32_t /*rsum*/) const
    {
        if (C) acc = (int32_t)((uint32_t)acc + (uint32_t)C[m * ldc + n]);
        acc = acc < cmin ? cmin : acc;
        acc = acc > cmax ? cmax : acc;
        D[m * ldd + n] = acc;
    }
};

// Static W8A8 requantisation to int8 (reference: ..._qai8_qai8p_qsi8cxp_4x1vl_rvv.cpp:121-159, 193-209).
struct EpiRequant {
    const int32_t *C;
    size_t ldc;
    const int32_t *bias;
    int8_t *D;
    size_t ldd;
    float scale_a;
    const float *scale_b;
    int quant_channel_b;
    float scale_d;
    int32_t zp_d;
    int32_t cmin, cmax;
    __device__ void operator()(size_t m, size_t n, int32_t acc, int32_t /*rsum*/) const
    {
        uint32_t u = (uint32_t)acc;
        if (C) u += (uint32_t)C[m * ldc + n];
        if (bias) u += (uint32_t)bias[n];
        int32_t mult, rsh;
        requant_column(scale_a, scale_b[quant_channel_b == 1 ? 0 : n], scale_d, &mult, &rsh);
        D[m * ldd + n] = (int8_t)requant_value((int32_t)u, mult, rsh, zp_d, cmin, cmax);
    }
};

// W4A8 float output (reference: ..._qai8dxp_qsi4cxp_4x1vl_rvv.cpp:118-177).
template <Dtype TD>
struct EpiW4A8 {
    const void *C;
    size_t ldc;
    const void *bias;
    void *D;
    size_t ldd;
    const float *scale_a;
    const int32_t *zp_a;
    const float *scale_b;
    float cmin, cmax;
    __device__ void operator()(size_t m, size_t n, int32_t acc, int32_t rsum) const
    {
        acc -= zp_a[m] * rsum;
        const float c = C ? TdTraits<TD>::load(C, m * ldc + n) : 0.0f;
        const float b = bias ? TdTraits<TD>::load(bias, n) : 0.0f;
        const float r = w4a8_epilogue(acc, scale_a[m], scale_b[n], C != nullptr, c, bias != nullptr, b, cmin, cmax);
        TdTraits<TD>::store(D, m * ldd + n, r);
    }
};

// Static W8A8 requantisation with per-row parameters and an Mx1 bias (reference:
// ..._mx1bias_reqi32toi8_clamp_qai8_qsi8dx_qai8_4x1vl_rvv.cpp:84-118, 141-163; requant tail
// tqt_kernel_gemm_i8_i8_4x1vl_rvv.h:264-330).  scale_a is indexed from the call's first row.
struct EpiRequantRow {
    const int32_t *C;
    size_t ldc;
    const int32_t *bias;   // [m]
    int8_t *D;
    size_t ldd;
    const float *scale_a;  // [m], or one value when quant_channel_a == 1
    int quant_channel_a;
    float scale_b;
    float scale_d;
    int32_t zp_d;
    int32_t cmin, cmax;
    __device__ void operator()(size_t m, size_t n, int32_t acc, int32_t /*rsum*/) const
    {
        uint32_t u = (uint32_t)acc;
        if (C) u += (uint32_t)C[m * ldc + n];
        if (bias) u += (uint32_t)bias[m];
        int32_t mult, rsh;
        requant_column(scale_a[quant_channel_a == 1 ? 0 : m], scale_b, scale_d, &mult, &rsh);
        D[m * ldd + n] = (int8_t)requant_value((int32_t)u, mult, rsh, zp_d, cmin, cmax);
    }
};

// Dynamic-activation W8A8 with float output, qai8dx x qsi8cx (reference:
// tqt_kernel_gemm_qai8dx_qsi8cx_4x1vl_rvv.h: the zero point is applied inside the MAC as (a - zp_a)
// :95-139, which equals acc - zp_a * rowsum(b) in wrapping int32; r = (float)acc * (scale_b * scale_a)
// :167-176; C is ignored; f32: + bias, clamp in f32; f16: narrow first, then add the bias and clamp in
// f16 :262-278).
template <Dtype TD>
struct EpiDxCx {
    const void *bias;
    void *D;
    size_t ldd;
    const float *scale_a;
    const int32_t *zp_a;
    const float *scale_b;
    float cmin, cmax;
    __device__ void operator()(size_t m, size_t n, int32_t acc, int32_t rsum) const
    {
        acc = (int32_t)((uint32_t)acc - (uint32_t)zp_a[m] * (uint32_t)rsum);
        const float s = __fmul_rn(scale_b[n], scale_a[m]);
        float r = __fmul_rn(__int2float_rn(acc), s);
        if (TD == Dtype::F32) {
            if (bias) r = __fadd_rn(r, static_cast<const float *>(bias)[n]);
            r = r < cmin ? cmin : r;
            r = r > cmax ? cmax : r;
            static_cast<float *>(D)[m * ldd + n] = r;
        } else {
            // an f16 sum of two f16 values: exact in f32 or far below half an ulp, so one rounding either way
            float h = __half2float(__float2half_rn(r));
            if (bias) h = __half2float(__float2half_rn(__fadd_rn(h, __half2float(static_cast<const __half *>(bias)[n]))));
            h = h < cmin ? cmin : h;
            h = h > cmax ? cmax : h;
            static_cast<__half *>(D)[m * ldd + n] = __float2half_rn(h);
        }
    }
};

}  // namespace tqt
