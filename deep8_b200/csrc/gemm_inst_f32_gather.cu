// Instantiations of the fp32 (3xTF32) kernel: loader warps split every operand value into tf32 hi and lo parts.
#include "gemm_host.h"

namespace d8k {

template <bool A_MN, bool B_MN>
static GemmLaunchFn pick(int bn) {
    if (bn == 128) return launch_cfg<GemmCfg<true, A_MN, B_MN, 128, 3, true>>;
    if (bn == 64) return launch_cfg<GemmCfg<true, A_MN, B_MN, 64, 4, true>>;
    return nullptr;
}

GemmLaunchFn lookup_f32_gather(bool a_mn, bool b_mn, int bn) {
    if (!a_mn && !b_mn) return pick<false, false>(bn);
    if (!a_mn && b_mn) return pick<false, true>(bn);
    if (a_mn && !b_mn) return pick<true, false>(bn);
    return pick<true, true>(bn);
}

}  // namespace d8k
