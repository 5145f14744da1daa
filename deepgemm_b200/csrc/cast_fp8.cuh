// BF16 -> E4M3 with one UE8M0 (power-of-two) scale per 1 x gran_k group, in one pass over the data.
//
// Same arithmetic as per_token_cast_to_fp8(use_ue8m0=True) (deep_gemm/utils/math.py:13-49): amax of the group
// clamped to 1e-4, scale = the power of two at or above amax / 448, value * (1 / scale) rounded to nearest even
// E4M3.  The scales come out in one of three forms, so that no second kernel has to repack them: FP32 [rows, groups]
// (what the reference helper returns), UE8M0 bytes packed four per int32 [rows, ceil(groups / 4)] (the helper's
// use_packed_ue8m0 form; also the token-major layout of the Mega MoE input buffer), or the same words MN-major
// (element (row, kw) at kw * sf_ld + row), which is the layout the GEMM kernels read through TMA
// (csrc/jit_kernels/impls/smxx_layout.hpp:108-131).
//
// HBM bound: 2 bytes read and 1 + 1/gran_k bytes written per element.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cstdint>

namespace dg {

enum CastSfMode : uint32_t { kCastSfFloat = 0, kCastSfPackedRowMajor = 1, kCastSfPackedMnMajor = 2 };

struct CastParams {
    const __nv_bfloat16* x;
    int64_t ldx;          // elements between rows of x
    uint32_t rows, cols;  // cols % 8 == 0
    uint32_t gran_k;      // 32 or 128
    uint8_t* q;
    int64_t ldq;          // bytes between rows of q
    void* sf;
    uint32_t sf_mode;
    int64_t sf_ld;        // row-major modes: elements between rows; MN-major: words between packed-K columns
};

constexpr uint32_t kCastThreads = 256;
constexpr uint32_t kCastUnroll = 4;   // 16-byte loads in flight per lane

// One warp per row at a time; a lane owns 8 consecutive elements of each of kCastUnroll 256-element spans.
__global__ void __launch_bounds__(kCastThreads) cast_bf16_to_fp8_ue8m0_kernel(const CastParams p) {
    asm volatile("griddepcontrol.wait;" ::: "memory");                // x may come from the kernel before this one
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the consumer waits for this kernel's end itself
    const uint32_t lane = threadIdx.x % 32;
    const uint32_t warp = (blockIdx.x * kCastThreads + threadIdx.x) / 32, num_warps = gridDim.x * kCastThreads / 32;
    const uint32_t lanes_per_group = p.gran_k / 8;                    // 4 or 16
    const uint32_t groups = (p.cols + p.gran_k - 1) / p.gran_k, words = (groups + 3) / 4;
    const uint32_t span = 32 * 8 * kCastUnroll;                       // elements per warp iteration
    for (uint32_t row = warp; row < p.rows; row += num_warps) {
        const __nv_bfloat16* xr = p.x + static_cast<int64_t>(row) * p.ldx;
        uint8_t* qr = p.q + static_cast<int64_t>(row) * p.ldq;
        for (uint32_t c0 = 0; c0 < groups * p.gran_k; c0 += span) {
            uint4 raw[kCastUnroll];
            uint32_t exps[kCastUnroll];
#pragma unroll
            for (uint32_t u = 0; u < kCastUnroll; ++u) {
                const uint32_t c = c0 + (u * 32 + lane) * 8;
                raw[u] = c < p.cols ? *reinterpret_cast<const uint4*>(xr + c) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (uint32_t u = 0; u < kCastUnroll; ++u) {
                const uint32_t c = c0 + (u * 32 + lane) * 8;
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
                float v[8];
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(h[i]);
                    v[2 * i] = f.x, v[2 * i + 1] = f.y;
                    amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
                }
                for (uint32_t off = 1; off < lanes_per_group; off <<= 1)
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                // Exponent of the power of two at or above amax / 448 (448 = 1.75 * 2^8: the add carries into the
                // exponent iff the mantissa exceeds that of 1.75), floored at 2^-22 = the scale of amax 1e-4
                uint32_t e = (__float_as_uint(amax) + 0x1FFFFFu) >> 23;
                e = min(max(e, 113u) - 8u, 254u);
                const float inv = __uint_as_float((254u - e) << 23);
                if (c >= p.cols) e = 127;   // a group that covers no data: scale 1.0, as the reference pads
                exps[u] = e;
                if (c < p.cols) {
                    uint32_t w[2];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
                            make_float2(v[4 * i] * inv, v[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                        const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
                            make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
                        w[i] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
                    }
                    *reinterpret_cast<uint2*>(qr + c) = make_uint2(w[0], w[1]);
                }
            }
            // Scales.  Group of a lane's span u: (c0 + (u * 32 + lane) * 8) / gran_k.
            if (p.sf_mode == kCastSfFloat) {
#pragma unroll
                for (uint32_t u = 0; u < kCastUnroll; ++u) {
                    const uint32_t g = (c0 + (u * 32 + lane) * 8) / p.gran_k;
                    if (lane % lanes_per_group == 0 && g < groups)
                        reinterpret_cast<float*>(p.sf)[static_cast<int64_t>(row) * p.sf_ld + g] =
                            __uint_as_float(exps[u] << 23);
                }
            } else {
                // Four consecutive groups make a word.  Per-32 groups: 16 lanes of one span; per-128 groups: both
                // halves of two neighbouring spans.
#pragma unroll
                for (uint32_t u = 0; u < kCastUnroll; ++u) {
                    uint32_t word, kw;
                    bool writer;
                    if (p.gran_k == 32) {
                        const uint32_t base = lane & ~15u;
                        word = __shfl_sync(0xffffffffu, exps[u], base) |
                               (__shfl_sync(0xffffffffu, exps[u], base + 4) << 8) |
                               (__shfl_sync(0xffffffffu, exps[u], base + 8) << 16) |
                               (__shfl_sync(0xffffffffu, exps[u], base + 12) << 24);
                        kw = (c0 + (u * 32 + lane) * 8) / 128;
                        writer = lane % 16 == 0;
                    } else {
                        const uint32_t lo = exps[u & ~1u], hi = exps[u | 1u];
                        word = __shfl_sync(0xffffffffu, lo, 0) | (__shfl_sync(0xffffffffu, lo, 16) << 8) |
                               (__shfl_sync(0xffffffffu, hi, 0) << 16) | (__shfl_sync(0xffffffffu, hi, 16) << 24);
                        kw = (c0 + (u & ~1u) * 32 * 8) / 512;
                        writer = lane == 0 && (u & 1u) == 0;
                    }
                    if (writer && kw < words) {
                        int32_t* out = reinterpret_cast<int32_t*>(p.sf);
                        if (p.sf_mode == kCastSfPackedRowMajor) out[static_cast<int64_t>(row) * p.sf_ld + kw] = static_cast<int32_t>(word);
                        else                                    out[static_cast<int64_t>(kw) * p.sf_ld + row] = static_cast<int32_t>(word);
                    }
                }
            }
        }
    }
}

}  // namespace dg
