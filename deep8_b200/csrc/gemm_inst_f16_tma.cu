// Instantiations of the TMA-fed fp16 kernel: 128 x {128, 256} tiles, every operand-major combination.
#include "gemm_host.h"

namespace d8k {

template <bool A_MN, bool B_MN>
static GemmLaunchFn pick(int bn) {
    if (bn == 256) return launch_cfg<GemmCfg<false, A_MN, B_MN, 256, 4, false>>;
    if (bn == 128) return launch_cfg<GemmCfg<false, A_MN, B_MN, 128, 6, false>>;
    return nullptr;
}

// the same tiles with twin TMA-issuing and MMA-issuing threads (GemmCfg::TWIN)
template <bool A_MN, bool B_MN>
static GemmLaunchFn pick_twin(int bn) {
    if (bn == 256) return launch_cfg<GemmCfg<false, A_MN, B_MN, 256, 4, false, false, false, 4>>;
    if (bn == 128) return launch_cfg<GemmCfg<false, A_MN, B_MN, 128, 6, false, false, false, 4>>;
    return nullptr;
}

GemmLaunchFn lookup_f16_twin(bool a_mn, bool b_mn, int bn) {
    if (!a_mn && !b_mn) return pick_twin<false, false>(bn);
    if (!a_mn && b_mn) return pick_twin<false, true>(bn);
    if (a_mn && !b_mn) return pick_twin<true, false>(bn);
    return pick_twin<true, true>(bn);
}

// twin threads, grouped launches (GemmCfg::GROUPED)
template <bool A_MN, bool B_MN>
static GemmLaunchFn pick_grouped(int bn) {
    if (bn == 256) return launch_cfg<GemmCfg<false, A_MN, B_MN, 256, 4, false, false, false, 5>>;
    if (bn == 128) return launch_cfg<GemmCfg<false, A_MN, B_MN, 128, 6, false, false, false, 5>>;
    return nullptr;
}

GemmLaunchFn lookup_f16_grouped(bool a_mn, bool b_mn, int bn) {
    if (!a_mn && !b_mn) return pick_grouped<false, false>(bn);
    if (!a_mn && b_mn) return pick_grouped<false, true>(bn);
    if (a_mn && !b_mn) return pick_grouped<true, false>(bn);
    return pick_grouped<true, true>(bn);
}

GemmLaunchFn lookup_f16_tma(bool a_mn, bool b_mn, int bn) {
    if (!a_mn && !b_mn) return pick<false, false>(bn);
    if (!a_mn && b_mn) return pick<false, true>(bn);
    if (a_mn && !b_mn) return pick<true, false>(bn);
    return pick<true, true>(bn);
}

}  // namespace d8k
