// One row of the qai8dx activation quantiser done by one warp (16-bit inputs whose row fits in the warp's registers:
// k <= 4096, k a multiple of 16, 16-byte aligned rows): shared by the stand-alone quantise(+pack) kernel and by the GEMM
// kernel that quantises its own activations before its mainloop.
#pragma once

#include <type_traits>

#include "dev_common.cuh"

namespace tqt {

__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}

// Warp-per-row variant for 16-bit inputs whose rows fit in registers (k <= 4096, k a multiple of 16,
// 16-byte aligned rows): no block-wide synchronisation, 16 loads of 16 bytes in flight per lane, every
// row read exactly once.  The per-element division x / s is done as Markstein's correction of
// x * RN(1/s) (q0 = x*y; e = x - q0*s exactly, by fma; q = q0 + e*y): with y the correctly rounded
// reciprocal this is the correctly rounded quotient, i.e. bit-identical to the IEEE division the
// reference performs (test/common/test_common.h:232-240), at three operations per element.
//
// SPLIT > 1 shares a row between SPLIT consecutive warps of the CTA (warp `sub` of the row takes the 32-chunk groups
// sub, sub + SPLIT, ...): the warps exchange their minimum / maximum through `s_red` (2 floats per warp of the CTA) and
// meet at the named barrier `bar_id`, which only the row's warps use.  Few rows then still fill the SMs with warps.
template <Dtype TA, bool PACKED, uint32_t SPLIT = 1>
__device__ __forceinline__ void quant_row_warp(size_t row, size_t k, const void *__restrict__ A, size_t lda, uint8_t *__restrict__ out,
                                               size_t ldq, size_t kblocks_total, float *__restrict__ scale_a,
                                               int32_t *__restrict__ zp_a, uint32_t lane, uint32_t sub = 0, float *s_red = nullptr,
                                               uint32_t bar_id = 0)
{
    static_assert(TA != Dtype::F32, "16-bit inputs only");
    static_assert(SPLIT == 1 || SPLIT == 2 || SPLIT == 4, "warps per row");
    constexpr uint32_t NI = 8 / SPLIT;
    const uint32_t nchunks = (uint32_t)(k / 16);   // 16-element chunks of the row; chunk c belongs to lane c % 32
    const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(A) + row * lda);
    const uint32_t lane0 = lane + 32u * sub;       // first chunk of this lane; the following ones are 32 * SPLIT apart
    uint4 raw[NI][2];
#pragma unroll
    for (uint32_t i = 0; i < NI; ++i) {
        const uint32_t c = lane0 + 32u * SPLIT * i;
        if (c < nchunks) {
            raw[i][0] = __ldg(src + 2 * c);
            raw[i][1] = __ldg(src + 2 * c + 1);
        } else {
            raw[i][0] = raw[i][1] = make_uint4(0, 0, 0, 0);
        }
    }
    auto widen = [](uint32_t w, float &lo, float &hi) {
        if (TA == Dtype::F16) {
            const __half2 h = *reinterpret_cast<const __half2 *>(&w);
            lo = __low2float(h);
            hi = __high2float(h);
        } else {
            lo = __uint_as_float(w << 16);
            hi = __uint_as_float(w & 0xffff0000u);
        }
    };
    // row minimum / maximum with packed 16-bit min/max (a NaN operand is ignored, as the reference's
    // comparisons ignore it); lanes without data keep the neutral start values
    using V2 = typename std::conditional<TA == Dtype::F16, __half2, __nv_bfloat162>::type;
    auto as_v2 = [](uint32_t w) {
        V2 v;
        memcpy(&v, &w, 4);
        return v;
    };
    V2 mn2 = as_v2(raw[0][0].x), mx2 = mn2;
    bool any = lane0 < nchunks;
#pragma unroll
    for (uint32_t i = 0; i < NI; ++i) {
        if (lane0 + 32u * SPLIT * i < nchunks) {
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t w[4] = {raw[i][h].x, raw[i][h].y, raw[i][h].z, raw[i][h].w};
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    mn2 = __hmin2(mn2, as_v2(w[j]));
                    mx2 = __hmax2(mx2, as_v2(w[j]));
                }
            }
        }
    }
    float vmin = 3.402823466e+38f, vmax = -3.402823466e+38f;
    if (any) {
        uint32_t wmn, wmx;
        memcpy(&wmn, &mn2, 4);
        memcpy(&wmx, &mx2, 4);
        float a0, a1, b0, b1;
        widen(wmn, a0, a1);
        widen(wmx, b0, b1);
        vmin = fminf(a0, a1);
        vmax = fmaxf(b0, b1);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
        vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    }
    if constexpr (SPLIT > 1) {
        // s_red points at the row's first slot: [SPLIT][2]
        if (lane == 0) {
            s_red[sub * 2] = vmin;
            s_red[sub * 2 + 1] = vmax;
        }
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(SPLIT * 32u) : "memory");
#pragma unroll
        for (uint32_t w = 0; w < SPLIT; ++w) {
            vmin = fminf(vmin, s_red[w * 2]);
            vmax = fmaxf(vmax, s_red[w * 2 + 1]);
        }
    }
    vmax = vmax > 0.0f ? vmax : 0.0f;
    vmin = vmin < 0.0f ? vmin : 0.0f;
    const float s = __fdiv_rn(__fsub_rn(vmax, vmin), 255.0f);
    int zp = 0;
    if (s != 0.0f) {
        zp = (int)rintf(__fsub_rn(-128.0f, __fdiv_rn(vmin, s)));
        zp = zp < -128 ? -128 : (zp > 127 ? 127 : zp);
    }
    if (lane == 0 && sub == 0) {
        scale_a[row] = s != 0.0f ? s : 1.0f;
        zp_a[row] = zp;
    }
    const float y = s != 0.0f ? __frcp_rn(s) : 0.0f;
    // The reciprocal route needs 1/s and the intermediate products to stay normal: rows whose scale is extreme
    // (a bf16 row has the f32 exponent range; below about 2.9e-39 the reciprocal overflows) divide instead.
    // Uniform per row, so per warp.
    const bool plain_div = !(s > 7.8886091e-31f && s < 1.2676506e30f);   // outside [2^-100, 2^100]
    const unsigned long long y2 = pack_f32x2(y, y), ns2 = pack_f32x2(-s, -s), magic2 = pack_f32x2(12582912.0f, 12582912.0f);
    const int zc = zp - 0x4B400000;   // bits of 1.5 * 2^23
    const size_t tile = row >> 7;
    const uint32_t r = (uint32_t)(row & 127);
    const uint32_t out_chunks = PACKED ? (uint32_t)((k + 127) / 128) * 8u : nchunks;   // packed rows are zero-padded to the block width
#pragma unroll
    for (uint32_t i = 0; i < NI; ++i) {
        const uint32_t c = lane0 + 32u * SPLIT * i;
        if (c >= out_chunks) continue;
        uint32_t packed[4] = {0, 0, 0, 0};
        if (c < nchunks && s != 0.0f) {
#pragma unroll
            for (uint32_t h = 0; h < 2; ++h) {
                const uint32_t w[4] = {raw[i][h].x, raw[i][h].y, raw[i][h].z, raw[i][h].w};
                int v[8];
                if (plain_div) {
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        float x2[2];
                        widen(w[j], x2[0], x2[1]);
                        v[j * 2] = __float2int_rn(__fdiv_rn(x2[0], s)) + zp;
                        v[j * 2 + 1] = __float2int_rn(__fdiv_rn(x2[1], s)) + zp;
                    }
                } else {
                    // two elements per instruction (packed f32x2 arithmetic, each lane IEEE round-to-nearest): q0 = x * y,
                    // e = fma(-q0, s, x), q = fma(e, y, q0); then q + 1.5 * 2^23 leaves rint(q) in the low mantissa bits
                    // (|q| <= 255: the scale is the row's range over 255), so the conversion is an integer subtraction
                    // folded into the zero point instead of a quarter-rate float-to-int instruction
#pragma unroll
                    for (uint32_t j = 0; j < 4; ++j) {
                        float x0, x1;
                        widen(w[j], x0, x1);
                        const unsigned long long X = pack_f32x2(x0, x1);
                        unsigned long long q0, e, q, t;
                        asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(q0) : "l"(X), "l"(y2));
                        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(e) : "l"(q0), "l"(ns2), "l"(X));
                        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(e), "l"(y2), "l"(q0));
                        asm("add.rn.f32x2 %0, %1, %2;" : "=l"(t) : "l"(q), "l"(magic2));
                        v[j * 2] = (int)(uint32_t)t + zc;
                        v[j * 2 + 1] = (int)(uint32_t)(t >> 32) + zc;
                    }
                }
                // saturate to int8 and pack four values per word: element 0 in the lowest byte
#pragma unroll
                for (uint32_t g = 0; g < 2; ++g) {
                    uint32_t hi16, word;
                    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi16) : "r"(v[g * 4 + 3]), "r"(v[g * 4 + 2]), "r"(0));
                    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(word) : "r"(v[g * 4 + 1]), "r"(v[g * 4 + 0]), "r"(hi16));
                    packed[h * 2 + g] = word;
                }
            }
        }
        const uint4 q4 = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        if (PACKED) {
            uint8_t *base = out + (tile * kblocks_total + (c >> 3)) * kI8BlockBytes;
            *reinterpret_cast<uint4 *>(base + sw128_byte(r, (c & 7u) * 16u)) = q4;
        } else {
            *reinterpret_cast<uint4 *>(out + row * ldq + (size_t)c * 16u) = q4;
        }
    }
}

}  // namespace tqt
