// gemm_bs_kernel instantiations: kind::mxf8f6f4 (FP8 x FP8, FP8 x FP4) with the store / accumulate epilogue.
#include "gemm_launch.cuh"

namespace dg {

int dispatch_gemm_plain(const GemmLaunch& l) {
    // tokens on the UMMA M axis (dense, K-grouped, batched): BF16 and FP32 output
    DG_GEMM_CASE(1, 128, false, false, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 256, false, false, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 128, false, false, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 256, false, false, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 128, false, true, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 256, false, true, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 128, false, true, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 256, false, true, 0, kKindMxf8f6f4)
    // weights on the UMMA M axis (M-grouped layouts)
    DG_GEMM_CASE(1, 64, true, false, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 128, true, false, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 64, true, false, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 128, true, false, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(2, 256, true, false, 0, kKindMxf8f6f4)
    DG_GEMM_CASE(1, 256, true, false, 0, kKindMxf8f6f4)
    // 240-token tiles: two accumulator stages plus the scale columns fit the 512 columns of tensor memory without
    // sharing any, so a tile's first UMMA need not wait for the tile before it to be drained
    DG_GEMM_CASE(2, 240, true, false, 0, kKindMxf8f6f4)
    return kLaunchNoKernel;
}

}  // namespace dg
