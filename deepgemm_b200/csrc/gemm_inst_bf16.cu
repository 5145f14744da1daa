// gemm_bs_kernel instantiations: kind::f16 (BF16 operands, no scale factors), store / accumulate and
// stochastic-rounding epilogues.
#include "gemm_launch.cuh"

namespace dg {

int dispatch_gemm_bf16(const GemmLaunch& l) {
    DG_GEMM_CASE(1, 128, false, false, 0, kKindBf16)
    DG_GEMM_CASE(1, 256, false, false, 0, kKindBf16)
    DG_GEMM_CASE(2, 128, false, false, 0, kKindBf16)
    DG_GEMM_CASE(2, 256, false, false, 0, kKindBf16)
    DG_GEMM_CASE(1, 128, false, true, 0, kKindBf16)
    DG_GEMM_CASE(1, 256, false, true, 0, kKindBf16)
    DG_GEMM_CASE(2, 128, false, true, 0, kKindBf16)
    DG_GEMM_CASE(2, 256, false, true, 0, kKindBf16)
    DG_GEMM_CASE(1, 64, true, false, 0, kKindBf16)
    DG_GEMM_CASE(1, 128, true, false, 0, kKindBf16)
    DG_GEMM_CASE(1, 256, true, false, 0, kKindBf16)
    DG_GEMM_CASE(2, 64, true, false, 0, kKindBf16)
    DG_GEMM_CASE(2, 128, true, false, 0, kKindBf16)
    DG_GEMM_CASE(2, 256, true, false, 0, kKindBf16)
    DG_GEMM_CASE(1, 128, false, false, kEpiStochastic, kKindBf16)
    DG_GEMM_CASE(1, 256, false, false, kEpiStochastic, kKindBf16)
    DG_GEMM_CASE(2, 128, false, false, kEpiStochastic, kKindBf16)
    DG_GEMM_CASE(2, 256, false, false, kEpiStochastic, kKindBf16)
    return kLaunchNoKernel;
}

}  // namespace dg
