// Instantiations of the fp32 (3xTF32) kernel fed by TMA: the raw fp32 tiles serve as the tf32 hi images (the tensor core
// ignores the low 13 mantissa bits) and converter warps write the lo images beside them.
#include "gemm_host.h"

namespace d8k {

template <bool A_MN, bool B_MN>
static GemmLaunchFn pick(int bn) {
    if (bn == 64) return launch_cfg<GemmCfg<true, A_MN, B_MN, 64, 4, false>>;
    return nullptr;
}

GemmLaunchFn lookup_f32_tma(bool a_mn, bool b_mn, int bn) {
    if (!a_mn && !b_mn) return pick<false, false>(bn);
    if (!a_mn && b_mn) return pick<false, true>(bn);
    if (a_mn && !b_mn) return pick<true, false>(bn);
    return pick<true, true>(bn);
}

}  // namespace d8k
