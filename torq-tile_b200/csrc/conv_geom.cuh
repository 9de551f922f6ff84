// Index arithmetic of the im2col view of a convolution input, shared by the im2col kernels and the implicit-GEMM
// operand accessor.  Reference: src/common/tqt_conv.h:52-196 (K order (ic, kd, kh, kw) for channel-first inputs,
// (kd, kh, kw, ic) for channel-last ones; padding positions read as 0).
#pragma once

#include "dev_common.cuh"

namespace tqt {

// Where a column index of the im2col matrix points inside the kernel window.
template <bool CF>
struct KCursor {
    uint32_t kd, kh, kw, ic;

    __device__ __forceinline__ void seek(const ConvGeom &g, uint32_t k)
    {
        uint32_t kpos;
        if (CF) {
            const uint32_t kvol = g.ker[0] * g.ker[1] * g.ker[2];
            ic = k / kvol;
            kpos = k - ic * kvol;
        } else {
            kpos = k / g.ic_pg;
            ic = k - kpos * g.ic_pg;
        }
        const uint32_t q = kpos / g.ker[2];
        kw = kpos - q * g.ker[2];
        kd = q / g.ker[1];
        kh = q - kd * g.ker[1];
    }

    __device__ __forceinline__ void next(const ConvGeom &g)
    {
        if (CF) {
            if (++kw == g.ker[2]) { kw = 0; if (++kh == g.ker[1]) { kh = 0; if (++kd == g.ker[0]) { kd = 0; ++ic; } } }
        } else {
            if (++ic == g.ic_pg) { ic = 0; if (++kw == g.ker[2]) { kw = 0; if (++kh == g.ker[1]) { kh = 0; ++kd; } } }
        }
    }

    // Offset of the input element this column reads for output position (od, oh, ow); false inside the padding.
    __device__ __forceinline__ bool source(const ConvGeom &g, uint32_t od, uint32_t oh, uint32_t ow, size_t &off) const
    {
        const int id = (int)(od * g.stride[0] + kd * g.dil[0]) - (int)g.pad[0];
        const int ih = (int)(oh * g.stride[1] + kh * g.dil[1]) - (int)g.pad[1];
        const int iw = (int)(ow * g.stride[2] + kw * g.dil[2]) - (int)g.pad[2];
        if (id < 0 || id >= (int)g.in[0] || ih < 0 || ih >= (int)g.in[1] || iw < 0 || iw >= (int)g.in[2]) return false;
        const size_t sp = ((size_t)id * g.in[1] + (size_t)ih) * g.in[2] + (size_t)iw;
        off = CF ? (size_t)(g.c_off + ic) * ((size_t)g.in[0] * g.in[1] * g.in[2]) + sp
                 : sp * g.c_total + g.c_off + ic;
        return true;
    }
};

__device__ __forceinline__ void split_position(const ConvGeom &g, uint32_t pos, uint32_t &od, uint32_t &oh, uint32_t &ow)
{
    const uint32_t q = pos / g.out[2];
    ow = pos - q * g.out[2];
    od = q / g.out[1];
    oh = q - od * g.out[1];
}

}  // namespace tqt
