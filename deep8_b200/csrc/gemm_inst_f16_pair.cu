// Instantiations of the paired-CTA (cta_group::2) TMA-fed fp16 kernel: 256 x 256 tiles per pair, three stages of two k-blocks.
#include "gemm2_kernel.cuh"
#include "gemm_host.h"

namespace d8k {

GemmLaunchFn lookup_f16_pair(bool a_mn, bool b_mn) {
    if (!a_mn && !b_mn) return launch_pair_cfg<Gemm2Cfg<false, false, 3, 2>>;
    if (!a_mn && b_mn) return launch_pair_cfg<Gemm2Cfg<false, true, 3, 2>>;
    if (a_mn && !b_mn) return launch_pair_cfg<Gemm2Cfg<true, false, 3, 2>>;
    return launch_pair_cfg<Gemm2Cfg<true, true, 3, 2>>;
}

}  // namespace d8k
