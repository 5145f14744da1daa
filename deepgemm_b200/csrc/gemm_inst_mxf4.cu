// gemm_bs_kernel instantiations: kind::mxf4 (both operands packed E2M1, 1 x 32 UE8M0 scales, K-major).
#include "gemm_launch.cuh"

namespace dg {

int dispatch_gemm_mxf4(const GemmLaunch& l) {
    DG_GEMM_CASE(1, 128, false, false, 0, kKindMxf4)
    DG_GEMM_CASE(1, 256, false, false, 0, kKindMxf4)
    DG_GEMM_CASE(2, 128, false, false, 0, kKindMxf4)
    DG_GEMM_CASE(2, 256, false, false, 0, kKindMxf4)
    DG_GEMM_CASE(1, 128, false, true, 0, kKindMxf4)
    DG_GEMM_CASE(1, 256, false, true, 0, kKindMxf4)
    DG_GEMM_CASE(2, 128, false, true, 0, kKindMxf4)
    DG_GEMM_CASE(2, 256, false, true, 0, kKindMxf4)
    DG_GEMM_CASE(1, 64, true, false, 0, kKindMxf4)
    DG_GEMM_CASE(1, 128, true, false, 0, kKindMxf4)
    DG_GEMM_CASE(2, 64, true, false, 0, kKindMxf4)
    DG_GEMM_CASE(2, 128, true, false, 0, kKindMxf4)
    DG_GEMM_CASE(2, 256, true, false, 0, kKindMxf4)
    DG_GEMM_CASE(1, 256, true, false, 0, kKindMxf4)
    return kLaunchNoKernel;
}

}  // namespace dg
