// Instantiations of the fp32 (3xTF32) kernel fed by TMA: the raw fp32 tiles serve as the tf32 hi images (the tensor core
// ignores the low 13 mantissa bits) and converter warps write the lo images beside them.
#include "gemm_host.h"

namespace d8k {

template <bool A_MN, bool B_MN>
static GemmLaunchFn pick(int bn, bool a_in_tmem) {
    if (bn != 64) return nullptr;
    // six 32 KB stages with A's hi/lo images in tensor memory, or four 48 KB stages with everything in shared memory
    if (a_in_tmem) return launch_cfg<GemmCfg<true, A_MN, B_MN, 64, 6, false, true>>;
    return launch_cfg<GemmCfg<true, A_MN, B_MN, 64, 4, false>>;
}

GemmLaunchFn lookup_f32_tma(bool a_mn, bool b_mn, int bn, bool a_in_tmem) {
    if (!a_mn && !b_mn) return pick<false, false>(bn, a_in_tmem);
    if (!a_mn && b_mn) return pick<false, true>(bn, a_in_tmem);
    if (a_mn && !b_mn) return pick<true, false>(bn, a_in_tmem);
    return pick<true, true>(bn, a_in_tmem);
}

}  // namespace d8k
