// gemm_bs_kernel instantiations: the two fused Mega MoE epilogues of the kernel-per-phase forward.
#include "gemm_launch.cuh"

namespace dg {

int dispatch_gemm_moe(const GemmLaunch& l) {
    DG_GEMM_CASE(2, 256, true, false, 1, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 128, true, false, 1, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 256, true, false, 1, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 128, true, false, 1, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 256, true, false, 2, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 128, true, false, 2, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 256, true, false, 2, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 128, true, false, 2, kKindMxf8f6f4)
    return kLaunchNoKernel;
}

}  // namespace dg
