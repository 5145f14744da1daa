// Scale-factor layout kernels: FP32 power-of-two scales -> packed UE8M0 words in the
// MN-major, 16-byte-aligned layout the GEMM's scale-factor tensor maps read.
// HBM-bound byte shuffling: one 32 x 32-word tile per block, transposed through shared
// memory so that both the (K-contiguous) reads and the (MN-contiguous) writes coalesce.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace dg {

struct SfPackParams {
    const float* sf;
    int32_t* out;
    int32_t mn, sf_k, packed_k, aligned_mn, gran_mn;
    int64_t stride_b, stride_mn, stride_k;
    const int32_t* psum_layout;
    int32_t num_psum_groups, psum_alignment;
};

__device__ __forceinline__ uint32_t ue8m0_byte(float v) { return (__float_as_uint(v) >> 23) & 0xFFu; }

// grid: (ceil(mn / 32), ceil(packed_k / 32), batches); block: 32 x 8
__global__ void __launch_bounds__(256) sf_pack_ue8m0_kernel(const SfPackParams p) {
    __shared__ uint32_t tile[32][33];
    __shared__ uint32_t row_valid[32];
    grid_dependency_wait();      // the scales may come from the kernel before this one in the stream
    grid_launch_dependents();    // the GEMM that follows may start its set-up; it waits for this kernel's end itself
    const int lane = threadIdx.x, wy = threadIdx.y;
    const int m0 = blockIdx.x * 32, kw0 = blockIdx.y * 32, b = blockIdx.z;

    if (wy == 0) {
        uint32_t valid = 1;
        if (p.psum_layout != nullptr) {
            // Row m is live iff it lies in some group's [aligned start, end)
            const int m = m0 + lane;
            valid = 0;
            int prev_end = 0;
            for (int g = 0; g < p.num_psum_groups; ++g) {
                const int end = p.psum_layout[g];
                const int start = (prev_end + p.psum_alignment - 1) / p.psum_alignment * p.psum_alignment;
                if (m >= start && m < end) valid = 1;
                prev_end = end;
            }
        }
        row_valid[lane] = valid;
    }
    __syncthreads();

    const float* src = p.sf + b * p.stride_b;
    // Phase 1: thread (lane = packed word, wy + 8 i = row) packs four consecutive K scales
    const int kw = kw0 + lane;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = wy + i * 8;
        const int m = m0 + r;
        uint32_t word = 0;
        if (m < p.mn && kw < p.packed_k && row_valid[r]) {
            const float* row = src + (m / p.gran_mn) * p.stride_mn;   // gran_mn > 1: block scales shared by rows
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int k = kw * 4 + j;
                if (k < p.sf_k) word |= ue8m0_byte(row[k * p.stride_k]) << (8 * j);
            }
        }
        tile[lane][r] = word;
    }
    __syncthreads();
    // Phase 2: thread (lane = row, wy + 8 i = packed word) writes MN-contiguous
    int32_t* dst = p.out + static_cast<int64_t>(b) * p.packed_k * p.aligned_mn;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int w = wy + i * 8;
        const int m = m0 + lane;
        if (m < p.mn && kw0 + w < p.packed_k)
            dst[static_cast<int64_t>(kw0 + w) * p.aligned_mn + m] = static_cast<int32_t>(tile[w][lane]);
    }
}

struct SfPackKGroupedParams {
    const float* sf;
    int32_t* out;
    const int32_t* grouped_layout;
    int32_t num_groups, mn, sf_k_rows, packed_rows, gran_k, k_alignment, use_psum;
};

// One thread per output word (packed row, mn).  grid: (ceil(mn / 256), packed_rows); block: 256
__global__ void __launch_bounds__(256) sf_pack_ue8m0_k_grouped_kernel(const SfPackKGroupedParams p) {
    __shared__ int s_src_row, s_rows_left;
    grid_dependency_wait();
    grid_launch_dependents();
    if (threadIdx.x == 0) {
        // Find the group owning packed row blockIdx.y
        int packed = 0, src = 0, prev_end = 0;
        int found_src = -1, left = 0;
        for (int g = 0; g < p.num_groups; ++g) {
            int k;
            if (p.use_psum) {
                const int end = p.grouped_layout[g];
                const int start = (prev_end + p.k_alignment - 1) / p.k_alignment * p.k_alignment;
                k = (end - start + p.k_alignment - 1) / p.k_alignment * p.k_alignment;
                prev_end = end;
            } else {
                k = p.grouped_layout[g];
            }
            const int sf_rows = k / p.gran_k;
            const int pk = (sf_rows + 3) / 4;
            const int y = static_cast<int>(blockIdx.y);
            if (y >= packed && y < packed + pk) {
                found_src = src + (y - packed) * 4;
                left = sf_rows - (y - packed) * 4;
                break;
            }
            packed += pk, src += sf_rows;
        }
        s_src_row = found_src, s_rows_left = left;
    }
    __syncthreads();
    const int m = blockIdx.x * 256 + threadIdx.x;
    if (m >= p.mn) return;
    uint32_t word = 0;
    if (s_src_row >= 0) {
        const int n = s_rows_left < 4 ? s_rows_left : 4;
        for (int j = 0; j < n; ++j)
            word |= ue8m0_byte(p.sf[static_cast<int64_t>(s_src_row + j) * p.mn + m]) << (8 * j);
    }
    p.out[static_cast<int64_t>(blockIdx.y) * p.mn + m] = static_cast<int32_t>(word);
}

}  // namespace dg
