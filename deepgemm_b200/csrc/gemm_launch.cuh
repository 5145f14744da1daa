// Launch glue between the host side (lib.cu: checks, tile choice, tensor maps) and the instantiations of
// gemm_bs_kernel, which are spread over several translation units so that they compile in parallel:
//   gemm_inst_plain.cu  kind::mxf8f6f4, store / accumulate epilogue
//   gemm_inst_moe.cu    kind::mxf8f6f4, the two fused Mega MoE epilogues
//   gemm_inst_mxf4.cu   kind::mxf4 (both operands packed E2M1)
//   gemm_inst_bf16.cu   kind::f16 (BF16 operands without scale factors)
//   gemm_inst_epi.cu    the value epilogues (stochastic rounding, FP8 cast with clamp)
#pragma once

#include <cstring>

#include "gemm_bs.cuh"

namespace dg {

struct GemmLaunch {
    GemmParams p;
    cudaStream_t stream;
    uint32_t units;   // CTAs (cta_group 1) or CTA pairs (cta_group 2)
    int pdl;          // launch with programmatic stream serialisation
    // which instantiation
    int ctas, bn, epi;
    bool swap, f32;
    int kind;         // kKindMxf8f6f4, kKindMxf4, kKindBf16
};

enum : int { kLaunchNoKernel = -1 };

// Each returns cudaSuccess, a CUDA error, or kLaunchNoKernel when the translation unit holds no such instantiation.
int dispatch_gemm_plain(const GemmLaunch& l);
int dispatch_gemm_moe(const GemmLaunch& l);
int dispatch_gemm_mxf4(const GemmLaunch& l);
int dispatch_gemm_bf16(const GemmLaunch& l);
int dispatch_gemm_epi(const GemmLaunch& l);

template <class Cfg>
int launch_gemm(const GemmLaunch& l) {
    // The attribute is per device; set it on every call (cheap) so that multi-device processes work.
    cudaError_t err = cudaFuncSetAttribute(gemm_bs_kernel<Cfg>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(Cfg::kSmemBytes));
    if (err != cudaSuccess) return static_cast<int>(err);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(l.units * Cfg::kCtas, 1, 1);
    cfg.blockDim = dim3(Cfg::kThreads, 1, 1);
    cfg.dynamicSmemBytes = Cfg::kSmemBytes;
    cfg.stream = l.stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = Cfg::kCtas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (l.pdl) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_bs_kernel<Cfg>, l.p));
}

#define DG_GEMM_CASE(CT, BNV, SW, F32, EPI, KIND)                                                              \
    if (l.ctas == CT && l.bn == BNV && l.swap == SW && l.f32 == F32 && l.epi == EPI && l.kind == int(KIND))    \
        return launch_gemm<GemmConfig<CT, BNV, SW, F32, EPI, int(KIND)>>(l);

}  // namespace dg
