// Instantiations of the fp32 (3xTF32) kernel fed by TMA: the raw fp32 tiles serve as the tf32 hi images (the tensor core
// ignores the low 13 mantissa bits) and converter warps write the lo images beside them.
#include "gemm_host.h"

namespace d8k {

template <bool A_MN, bool B_MN>
static GemmLaunchFn pick(int bn, bool a_in_tmem) {
    if (bn != 64) return nullptr;
    // four 32 KB stages with A's hi/lo images in tensor memory (2 x 128 accumulator columns + 4 x 64 of A fill the 512),
    // or four 48 KB stages with everything in shared memory
    if (a_in_tmem) return launch_cfg<GemmCfg<true, A_MN, B_MN, 64, 4, false, true>>;
    return launch_cfg<GemmCfg<true, A_MN, B_MN, 64, 4, false>>;
}

// four 16 KB stages of B hi/lo, three 44 KB patch slots, A's hi/lo images in tensor memory
GemmLaunchFn lookup_f32_halo(bool b_mn) {
    if (b_mn) return launch_cfg<GemmCfg<true, false, true, 64, 4, false, true, true>>;
    return launch_cfg<GemmCfg<true, false, false, 64, 4, false, true, true>>;
}

// two CTAs per SM, each with one accumulator buffer and one converter group.  mode 1: A's hi and lo images in tensor
// memory, two 32 KB stages; mode 2: only the lo image there (the raw tile is the hi image), three stages
template <int MODE, int STAGES>
static GemmLaunchFn pick_dual(bool a_mn, bool b_mn) {
    if (!a_mn && !b_mn) return launch_cfg<GemmCfg<true, false, false, 64, STAGES, false, true, false, MODE>>;
    if (!a_mn && b_mn) return launch_cfg<GemmCfg<true, false, true, 64, STAGES, false, true, false, MODE>>;
    if (a_mn && !b_mn) return launch_cfg<GemmCfg<true, true, false, 64, STAGES, false, true, false, MODE>>;
    return launch_cfg<GemmCfg<true, true, true, 64, STAGES, false, true, false, MODE>>;
}
GemmLaunchFn lookup_f32_dual(bool a_mn, bool b_mn, int mode) {
    if (mode == 4) return pick_dual<4, 4>(a_mn, b_mn);  // one CTA per SM with twin TMA and MMA threads (GemmCfg::TWIN)
    if (mode == 5) return pick_dual<5, 4>(a_mn, b_mn);  // the same for grouped launches (GemmCfg::GROUPED)
    return mode == 2 ? pick_dual<2, 3>(a_mn, b_mn) : pick_dual<1, 2>(a_mn, b_mn);
}

GemmLaunchFn lookup_f32_tma(bool a_mn, bool b_mn, int bn, bool a_in_tmem) {
    if (!a_mn && !b_mn) return pick<false, false>(bn, a_in_tmem);
    if (!a_mn && b_mn) return pick<false, true>(bn, a_in_tmem);
    if (a_mn && !b_mn) return pick<true, false>(bn, a_in_tmem);
    return pick<true, true>(bn, a_in_tmem);
}

}  // namespace d8k
