// gemm_bs_kernel instantiations: value epilogues of the dense / batched FP8 GEMM (BF16 with stochastic rounding,
// E4M3 with per-32 UE8M0 scales and optional clamp).
#include "gemm_launch.cuh"

namespace dg {

int dispatch_gemm_epi(const GemmLaunch& l) {
    DG_GEMM_CASE(1, 128, false, false, kEpiStochastic, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 256, false, false, kEpiStochastic, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 128, false, false, kEpiStochastic, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 256, false, false, kEpiStochastic, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 128, false, false, kEpiFp8Cast, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 256, false, false, kEpiFp8Cast, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 128, false, false, kEpiFp8Cast, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 256, false, false, kEpiFp8Cast, kKindMxf8f6f4)
    return kLaunchNoKernel;
}

}  // namespace dg
