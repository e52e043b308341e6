// Instantiations of the loader-warp fp16 kernel (unaligned matrices and the virtual im2col operands of Conv2d/DeConv2d).
#include "gemm_host.h"

namespace d8k {

template <bool A_MN, bool B_MN>
static GemmLaunchFn pick(int bn) {
    if (bn == 128) return launch_cfg<GemmCfg<false, A_MN, B_MN, 128, 6, true>>;
    if (bn == 64) return launch_cfg<GemmCfg<false, A_MN, B_MN, 64, 6, true>>;
    return nullptr;
}

GemmLaunchFn lookup_f16_gather(bool a_mn, bool b_mn, int bn) {
    if (!a_mn && !b_mn) return pick<false, false>(bn);
    if (!a_mn && b_mn) return pick<false, true>(bn);
    if (a_mn && !b_mn) return pick<true, false>(bn);
    return pick<true, true>(bn);
}

}  // namespace d8k
