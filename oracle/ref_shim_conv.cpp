// C entry point over the reference's im2col templates (src/common/tqt_conv.h:52-196, plain C++).
//
// TEST INFRASTRUCTURE ONLY.  No arithmetic of its own: includes the reference's header from the
// reference checkout at build time (oracle/Makefile, REF=<path>) and forwards to it, so that
// tqo_im2col_i8 in tqt_oracle.c can be pinned against the reference's own code.  Built into
// oracle/_ref/, never linked into the product.
#include <cstddef>
#include <cstdint>
#include <cstring>

#include "src/common/tqt_conv.h"

extern "C" {

// geom: the 21 size_t members of tqt_conv_params in declaration order.
void ref_im2col_i8(int channel_first, size_t group_idx, const int8_t *act, int8_t *out,
                   const size_t *geom)
{
    static_assert(sizeof(tqt_conv_params) == 21 * sizeof(size_t), "tqt_conv_params layout");
    tqt_conv_params p;
    std::memcpy(&p, geom, sizeof(p));
    if (channel_first)
        tqt_im2col_cf<int8_t>(group_idx, act, out, &p);
    else
        tqt_im2col_cl<int8_t>(group_idx, act, out, &p);
}

}  // extern "C"
