// Device-side helpers shared by every kernel: packed-layout index arithmetic, the scalar epilogue
// arithmetic (kept in one place so that the tensor-core, GEMV and CUDA-core kernels produce the
// same bits), and the watchdog word.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "tqt_internal.h"

namespace tqt {

// Device address (on the current device) of the watchdog word that a kernel sets when one of its
// bounded waits runs out; read and cleared by read_device_fault().  The word is a __device__
// variable of the library, not an allocation.  Returns nullptr if the address cannot be obtained.
unsigned int *fault_word_device_ptr();

enum FaultCode : unsigned int {
    kFaultNone = 0,
    kFaultProducerWait = 0x100,   // TMA producer waited for a free stage
    kFaultMmaWaitFull = 0x200,    // MMA issuer waited for operands
    kFaultMmaWaitTmem = 0x300,    // MMA issuer waited for an accumulator buffer
    kFaultEpilogueWait = 0x400,   // epilogue waited for an accumulator
    kFaultConverterWait = 0x500,  // int4 converter waited for data or a free buffer
    kFaultGemvWait = 0x600,       // GEMV waited for its bulk copies
    kFaultDrainWait = 0x700,      // producer waited for its own copies while bailing out
    kFaultGridBarrier = 0x800     // a CTA waited at the grid-wide barrier of the fused quantiser
};

// ---- packed-layout index arithmetic -------------------------------------------------------------
// Byte offset of element (r, kk) inside a 128 x 128 B swizzled block; es = element size in bytes.
__host__ __device__ inline uint32_t sw128_byte(uint32_t r, uint32_t byte_in_row)
{
    return r * 128u + ((((byte_in_row >> 4) ^ (r & 7u)) << 4) | (byte_in_row & 15u));
}

// qsi4cx block: byte offset and nibble half of element (r, kk), kk in [0,128).
__host__ __device__ inline uint32_t i4cx_byte(uint32_t r, uint32_t kk, uint32_t *hi)
{
    const uint32_t s = kk >> 5, t = kk & 31u;
    *hi = t >> 4;
    const uint32_t j = (t & 15u) >> 2, b = t & 3u;
    return r * 64u + (((s ^ ((r >> 1) & 3u)) << 4) | (j << 2) | b);
}

// qsi4c2 block: byte offset and nibble half of element (r, kk).
__host__ __device__ inline uint32_t i4c2_byte(uint32_t r, uint32_t kk, uint32_t *hi)
{
    const uint32_t s = kk >> 5, t = kk & 31u;
    const uint32_t j = t >> 3, i = t & 7u;
    const uint32_t p = (i >> 1) + 4u * (i & 1u);
    *hi = p & 1u;
    return r * 64u + (((s ^ ((r >> 1) & 3u)) << 4) | (j << 2) | (p >> 1));
}

// ---- scalar conversions --------------------------------------------------------------------------
template <Dtype T>
struct TdTraits;
template <>
struct TdTraits<Dtype::F32> {
    using type = float;
    __device__ static float load(const void *p, size_t i) { return static_cast<const float *>(p)[i]; }
    __device__ static void store(void *p, size_t i, float v) { static_cast<float *>(p)[i] = v; }
};
template <>
struct TdTraits<Dtype::F16> {
    using type = __half;
    __device__ static float load(const void *p, size_t i) { return __half2float(static_cast<const __half *>(p)[i]); }
    __device__ static void store(void *p, size_t i, float v) { static_cast<__half *>(p)[i] = __float2half_rn(v); }
};
template <>
struct TdTraits<Dtype::BF16> {
    using type = __nv_bfloat16;
    __device__ static float load(const void *p, size_t i)
    {
        return __bfloat162float(static_cast<const __nv_bfloat16 *>(p)[i]);
    }
    __device__ static void store(void *p, size_t i, float v)
    {
        static_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    }
};

// ---- W4A8 float epilogue ---------------------------------------------------------------------------
// r = ((float)acc * scale_a) * scale_b, then + C, then + bias, clamp; each step a separately
// rounded f32 operation (the RVV reference uses separate vfmul / vfadd / vfmax / vfmin).
__device__ inline float w4a8_epilogue(int32_t acc, float sa, float sb, bool has_c, float c, bool has_bias,
                                      float bias, float cmin, float cmax)
{
    float r = __fmul_rn(__fmul_rn(__int2float_rn(acc), sa), sb);
    if (has_c) r = __fadd_rn(r, c);
    if (has_bias) r = __fadd_rn(r, bias);
    // max / min as the RVV kernel's vfmax / vfmin (identical to the compare-and-select form for non-NaN r)
    r = fmaxf(r, cmin);
    r = fminf(r, cmax);
    return r;
}

// ---- requantisation --------------------------------------------------------------------------------
// Bit-exact device version of the reference's tqt_quantize_multiplier
// (src/gemm/gemm_i8_i8/tqt_utils_i8_i8.h:16-132): top 30 fraction bits plus the implicit one,
// +1 only when the discarded 22 bits exceed half, 2^31 renormalised, shift < -31 flushed.
__device__ inline void quantize_multiplier_dev(double v, int32_t *mult, int32_t *shift)
{
    if (v == 0.) {
        *mult = 0;
        *shift = 0;
        return;
    }
    const unsigned long long u = (unsigned long long)__double_as_longlong(v);
    long long q;
    int32_t sh;
    const unsigned int e = (unsigned int)((u >> 52) & 0x7ffull);
    if (e == 0x7ffu) {
        sh = 0x7fffffff;
        if (u & 0x000fffffffc00000ull)
            q = 0;
        else
            q = (u >> 63) ? (long long)0x8000000000000000ull : 0x7fffffffffffffffll;
    } else {
        sh = (int32_t)(e - 1023u) + 1;
        q = 0x40000000ll + (long long)((u & 0x000fffffffc00000ull) >> 22);
        if ((unsigned int)(u & 0x003fffffull) > 0x00200000u) q += 1;
        if (u >> 63) q = -q;
    }
    if (q == (1ll << 31)) {
        q /= 2;
        ++sh;
    }
    if (sh < -31) {
        sh = 0;
        q = 0;
    }
    *mult = (int32_t)q;
    *shift = sh;
}

// mult / right-shift of one output column: real = (double)sa * (double)sb / (double)sd.
__device__ inline void requant_column(float sa, float sb, float sd, int32_t *mult, int32_t *rshift)
{
    const double real = __ddiv_rn(__dmul_rn((double)sa, (double)sb), (double)sd);
    int32_t s;
    quantize_multiplier_dev(real, mult, &s);
    *rshift = (-s - 1) & 31;
}

// high32(acc*mult) >> rshift, + zp (wrapping), saturate to int16 then int8, clamp.
__device__ inline int32_t requant_value(int32_t acc, int32_t mult, int32_t rshift, int32_t zp, int32_t cmin,
                                        int32_t cmax)
{
    int32_t t = __mulhi(acc, mult);
    t >>= rshift;
    t = (int32_t)((uint32_t)t + (uint32_t)zp);
    t = max(-32768, min(32767, t));
    t = max(-128, min(127, t));
    t = max(cmin, min(cmax, t));
    return t;
}

}  // namespace tqt
