// Mega MoE forward: buffer layout and the CUDA-core kernels around the two grouped GEMMs
// (expert counting and index scatter, count exchange + cross-rank barrier, token pull into the
// expert-sorted pool, top-k reduction).  Peer memory is reached through plain loads / stores on
// the symmetric buffer's per-rank base addresses (NVLink), never through multicast loads.
//
// Takes the role of the dispatch / combine halves of the reference's sm100_fp8_fp4_mega_moe_impl
// (deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:360-729, 1588-1743) and of its
// NVLink barrier (deep_gemm/include/deep_gemm/comm/barrier.cuh:53-92), with bounded waits.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "gemm_bs.cuh"   // ptx helpers, moe_sf_row

namespace dg {

constexpr uint32_t kMoeMaxRanks = 16;
constexpr uint32_t kMoePoolAlign = 128;   // rows: every expert's pool segment starts on this boundary
// Token rows per tile of the single-kernel forward (a multiple of 16, at most 256).  With 256 the two accumulators and
// the scale columns need 16 more than the 512 columns of tensor memory, so neighbouring tiles share 16 columns and a
// tile's first UMMA waits until the tile before it has been drained from them; 240 (the reference's choice,
// csrc/jit_kernels/heuristics/mega_moe.hpp:88-141) avoids the sharing but cuts 1024 rows into five tiles instead of
// four: measured 3 % slower on 32 experts x ~1024 rows (1.32 vs 1.28 ms), the shared columns cost the UMMA issuer
// under 3 % of its time.
constexpr uint32_t kMoeTileRows = 256;

// The first kMoeCtrlBytes of every buffer hold the control block: words whose meaning and place do not depend on the
// configuration (num_experts, tokens, hidden ...), so that a buffer may be reused for another configuration between
// calls (SymmBuffer(base=...)): barrier flags and their epoch, the grid barrier, the per-expert send counters.
// Everything after it is rewritten by each call before it is read.
constexpr uint32_t kMoeCtrlBytes = 16384;
struct MoeCtrl {   // u32 word indices inside the control block
    static constexpr uint32_t kSignals = 0;      // [2][kMoeMaxRanks]: barrier flags written by peers
    static constexpr uint32_t kCall = 32;        // calls made so far (epoch of the barrier flags)
    static constexpr uint32_t kTotalRows = 33;   // pool rows in use, aligned
    static constexpr uint32_t kGridCount = 34;   // grid barrier: arrivals of the current generation (back to 0 when it opens)
    static constexpr uint32_t kGridGen = 35;     // grid barrier: generation, bumped by the last arriver
    static constexpr uint32_t kLayoutReady = 36, kNumTiles = 37, kCombineReady = 38;
    static constexpr uint32_t kSendCount = 64;   // [experts]: rows this rank sends to each expert (zero between calls)
};
constexpr uint32_t kMoeMaxExperts = kMoeCtrlBytes / 4 - MoeCtrl::kSendCount;

// Byte offsets inside one rank's symmetric buffer (identical on every rank).
struct MoeLayout {
    uint32_t ranks, experts, experts_local, t_max, topk, hidden, inter;
    uint32_t shared;         // shared experts (0: none); they act as one expert of intermediate size shared * inter
    uint32_t planes;         // combine planes: topk, plus one for the shared experts' result
    uint32_t pool_rows;      // capacity of the expert-sorted pool (multiple of 256)
    uint32_t sf_rows;        // row pitch of l1_sf / l2_sf: pool_rows, or more where the single kernel's tiles need it (each
                             // tile owns 256 scale rows of its own, in tcgen05.cp order relative to the tile's first row)
    uint64_t off_ctrl;       // control block, always 0
    uint64_t off_recv_count; // u32 [ranks][experts_local]: rows each source rank sends to each local expert
    uint64_t off_src_idx;    // u32 [experts_local][ranks][t_max]: token * topk + slot, written by the source rank
    uint64_t off_x, off_x_sf, off_topk_idx, off_topk_w;   // inputs the caller fills
    uint64_t off_l1_acts, off_l1_sf, off_pool_w, off_pool_meta, off_l2_acts, off_l2_sf;
    uint64_t off_combine;    // bf16 [planes][t_max][hidden]: planes 0 .. topk-1 written by the experts' ranks, plane topk
                             // by this rank's shared experts
    // Shared experts (every token of this rank, no dispatch): x's scales once more, MN-major and in tcgen05.cp row
    // order (filled by the caller like x_sf); the gated activation of all tokens; (rank, token, plane) per row
    uint64_t off_shared_sf, off_shared_l2_acts, off_shared_l2_sf, off_shared_meta;
    uint64_t off_work;       // local scratch, see MoeWork
    uint64_t total_bytes;
};

// Local tables at off_work (u32 words), all rewritten by every call
struct MoeWork {
    __host__ __device__ static uint32_t psum_end() { return 0; }   // [experts_local]: end of each expert's pool rows
    __host__ __device__ static uint32_t seg_off(uint32_t el) { return el; }
    // [experts_local * ranks]: first pool row of each (expert, source) segment
    __host__ __device__ static uint32_t seg_prefix(uint32_t el, uint32_t ranks) { return seg_off(el) + el * ranks; }
    // [experts_local * ranks + 1]: rows before each segment, unaligned (the pull kernel's work list)
    __host__ __device__ static uint32_t words(uint32_t el, uint32_t ranks) { return seg_prefix(el, ranks) + el * ranks + 1; }
};

// Work-area tables used only by the fused kernel (after the tables of MoeWork)
struct MoeFusedWork {
    __host__ __device__ static uint32_t max_tiles(const MoeLayout& L) { return L.pool_rows / kMoeTileRows + L.experts_local + 1; }
    __host__ __device__ static uint32_t tile_table(const MoeLayout& L) { return MoeWork::words(L.experts_local, L.ranks); }
    // per tile: row0, rows (UMMA N, a multiple of 16), expert, rows that carry a token, first scale row (tile * 256)
    __host__ __device__ static uint32_t pulled(const MoeLayout& L) { return tile_table(L) + max_tiles(L) * 8; }   // [max_tiles]
    __host__ __device__ static uint32_t l1_done(const MoeLayout& L) { return pulled(L) + max_tiles(L); }          // [max_tiles]
    // per expert: first pool row, first tile
    __host__ __device__ static uint32_t expert_tab(const MoeLayout& L) { return l1_done(L) + max_tiles(L); }      // [2 * experts_local]
    __host__ __device__ static uint32_t words(const MoeLayout& L) { return expert_tab(L) + 2 * L.experts_local; }
};

inline uint64_t moe_align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

// pool_cap: rows the expert-sorted pool must hold; 0 = the worst case (every token of every rank picks this rank's
// experts with all the slots it can).  A smaller pool makes a call whose rows do not fit fail with kStatusPoolOverflow.
inline MoeLayout make_moe_layout(uint32_t ranks, uint32_t experts, uint32_t t_max, uint32_t topk, uint32_t hidden,
                                 uint32_t inter, uint32_t pool_cap = 0, uint32_t shared = 0) {
    MoeLayout L{};
    L.ranks = ranks, L.experts = experts, L.experts_local = experts / ranks, L.t_max = t_max, L.topk = topk;
    L.hidden = hidden, L.inter = inter, L.shared = shared, L.planes = topk + (shared != 0 ? 1u : 0u);
    const uint64_t active_topk = topk < L.experts_local ? topk : L.experts_local;
    const uint64_t slack = static_cast<uint64_t>(L.experts_local) * kMoePoolAlign;   // every expert's rows start on a boundary
    uint64_t rows = static_cast<uint64_t>(t_max) * ranks * active_topk;
    if (pool_cap != 0 && pool_cap < rows) rows = pool_cap;
    L.pool_rows = static_cast<uint32_t>(moe_align_up(rows + slack, 256));
    const uint32_t tile_sf_rows = (L.pool_rows / kMoeTileRows + L.experts_local + 1) * 256;
    L.sf_rows = tile_sf_rows > L.pool_rows ? tile_sf_rows : L.pool_rows;
    uint64_t off = 0;
    auto take = [&](uint64_t bytes) {
        const uint64_t o = off;
        off = moe_align_up(off + bytes, 1024);
        return o;
    };
    L.off_ctrl = take(kMoeCtrlBytes);
    L.off_recv_count = take(static_cast<uint64_t>(ranks) * L.experts_local * 4);
    L.off_src_idx = take(static_cast<uint64_t>(L.experts_local) * ranks * t_max * 4);
    L.off_x = take(static_cast<uint64_t>(t_max) * hidden);
    L.off_x_sf = take(static_cast<uint64_t>(t_max) * (hidden / 128) * 4);
    L.off_topk_idx = take(static_cast<uint64_t>(t_max) * topk * 8);
    L.off_topk_w = take(static_cast<uint64_t>(t_max) * topk * 4);
    L.off_l1_acts = take(static_cast<uint64_t>(L.pool_rows) * hidden);
    L.off_l1_sf = take(static_cast<uint64_t>(L.sf_rows) * (hidden / 128) * 4);
    L.off_pool_w = take(static_cast<uint64_t>(L.pool_rows) * 4);
    L.off_pool_meta = take(static_cast<uint64_t>(L.pool_rows) * 12);
    L.off_l2_acts = take(static_cast<uint64_t>(L.pool_rows) * inter);
    L.off_l2_sf = take(static_cast<uint64_t>(L.sf_rows) * (inter / 128) * 4);
    L.off_combine = take(static_cast<uint64_t>(L.planes) * t_max * hidden * 2);
    if (shared != 0) {
        const uint64_t t_al = moe_align_up(t_max, 128), inter_s = static_cast<uint64_t>(shared) * inter;
        L.off_shared_sf = take(t_al * (hidden / 128) * 4);
        L.off_shared_l2_acts = take(t_al * inter_s);
        L.off_shared_l2_sf = take(t_al * (inter_s / 128) * 4);
        L.off_shared_meta = take(t_al * 12);
    }
    L.off_work = take(static_cast<uint64_t>(MoeFusedWork::words(L)) * 4);
    L.total_bytes = off;
    return L;
}

struct MoeArgs {
    MoeLayout L;
    uint8_t* base[kMoeMaxRanks];   // base address of every rank's buffer as mapped into this process
    uint32_t rank, num_tokens, timeout_ms;
    uint32_t* status;              // status block shared with the GEMM kernels
    int32_t* stats;                // cumulative_local_expert_recv_stats [experts_local] or null
};

enum : uint32_t { kStatusPeerTimeout = 2, kStatusPoolOverflow = 3 };

DG_DEVICE void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
DG_DEVICE uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Signal every peer with `value` in slot `which`, then wait (bounded) until every peer has signalled
// at least `value`.  Called by threads 0..ranks-1 of one CTA; returns false on timeout.
DG_DEVICE bool moe_cross_rank_barrier(const MoeArgs& a, uint32_t which, uint32_t value, uint32_t peer) {
    __threadfence_system();
    uint32_t* remote = reinterpret_cast<uint32_t*>(a.base[peer]) + MoeCtrl::kSignals + which * kMoeMaxRanks + a.rank;
    st_release_sys(remote, value);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(a.base[a.rank]) + MoeCtrl::kSignals + which * kMoeMaxRanks + peer;
    const uint64_t t0 = global_timer_ns();
    const uint64_t budget = static_cast<uint64_t>(a.timeout_ms) * 1000000ull;
    while (static_cast<int32_t>(ld_acquire_sys(mine) - value) < 0) {
        __nanosleep(200);
        if (global_timer_ns() - t0 > budget) {
            if (atomicCAS(a.status, 0u, kStatusPeerTimeout) == 0u) {
                a.status[1] = 100 + which, a.status[2] = peer, a.status[3] = value;
                __threadfence_system();
            }
            return false;
        }
    }
    return true;
}

// ---- step 1: count (token, slot) pairs per expert and tell the expert's rank which pairs to pull.
// grid: ceil(num_tokens * topk / 256), block 256
DG_DEVICE void moe_scatter_pair(const MoeArgs& a, uint32_t i) {
    const long long e = reinterpret_cast<const long long*>(a.base[a.rank] + a.L.off_topk_idx)[i];
    if (e < 0 || e >= static_cast<long long>(a.L.experts)) return;
    uint32_t* ctrl = reinterpret_cast<uint32_t*>(a.base[a.rank]);
    const uint32_t j = atomicAdd(ctrl + MoeCtrl::kSendCount + static_cast<uint32_t>(e), 1u);
    // one rank sends an expert at most t_max rows (one per token); a token that names an expert twice must not
    // write past this rank's part of the peer's table: the surplus pair is dropped (the count is capped to match)
    if (j >= a.L.t_max) return;
    const uint32_t dest = static_cast<uint32_t>(e) / a.L.experts_local, el = static_cast<uint32_t>(e) % a.L.experts_local;
    uint32_t* idx = reinterpret_cast<uint32_t*>(a.base[dest] + a.L.off_src_idx);
    idx[(static_cast<uint64_t>(el) * a.L.ranks + a.rank) * a.L.t_max + j] = i;
}
__global__ void __launch_bounds__(256) moe_scatter_kernel(const MoeArgs a) {
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i < a.num_tokens * a.L.topk) moe_scatter_pair(a, i);
}

// ---- step 2: publish the counts, cross-rank barrier, then lay out the pool.  Run by ALL threads of one CTA
// (`nthreads` of them).  With `fused` != nullptr it also writes the fused kernel's tile table, clears its
// progress counters and finally publishes `layout_ready`.  Returns false if the barrier timed out.
struct MoeFusedHooks {
    uint32_t tile_table, pulled, l1_done, expert_tab;   // word offsets in the work area
};
// `scratch`: kMoeScanWords words of shared memory for the layout scan (nullptr: scan in global memory).
constexpr uint32_t kMoeScanCap = 512, kMoeScanWords = 4 * kMoeScanCap + 1;
DG_DEVICE bool moe_exchange_body(const MoeArgs& a, uint32_t tid, uint32_t nthreads, const MoeFusedHooks* fused,
                                 uint32_t* scratch) {
    const MoeLayout& L = a.L;
    uint32_t* work = reinterpret_cast<uint32_t*>(a.base[a.rank] + L.off_work);
    uint32_t* ctrl = reinterpret_cast<uint32_t*>(a.base[a.rank]);
    __shared__ uint32_t s_call, s_ok, s_tiles, s_rows;
    if (tid == 0) {
        s_call = ++ctrl[MoeCtrl::kCall];
        s_ok = 1;
    }
    for (uint32_t e = tid; e < L.experts; e += nthreads) {
        const uint32_t cnt = min(ctrl[MoeCtrl::kSendCount + e], L.t_max);
        ctrl[MoeCtrl::kSendCount + e] = 0;   // ready for the next call
        const uint32_t dest = e / L.experts_local, el = e % L.experts_local;
        reinterpret_cast<uint32_t*>(a.base[dest] + L.off_recv_count)[a.rank * L.experts_local + el] = cnt;
    }
    __syncthreads();
    if (tid < L.ranks)
        if (!moe_cross_rank_barrier(a, 0, 2 * s_call - 1, tid)) s_ok = 0;
    __syncthreads();
    if (!s_ok) return false;
    // Pool layout: expert el owns rows [align(prev_end), end); inside, sources in rank order.
    const uint32_t* recv = reinterpret_cast<const uint32_t*>(a.base[a.rank] + L.off_recv_count);
    int32_t* meta = reinterpret_cast<int32_t*>(a.base[a.rank] + L.off_pool_meta);
    // The counts come to shared memory in parallel, one thread scans them there (a scan over global memory costs
    // a round trip per segment: 256 of them at 32 experts x 8 ranks), all threads write the tables out.
    const uint32_t segs = L.experts_local * L.ranks;
    uint32_t* s_cnt = scratch;                 // [segs]   rows per (expert, source) segment
    uint32_t* s_off = scratch + kMoeScanCap;   // [segs]   first pool row of the segment
    uint32_t* s_pre = scratch + 2 * kMoeScanCap;   // [segs + 1] rows before the segment, unaligned
    uint32_t* s_end = scratch + 3 * kMoeScanCap + 1;   // [experts_local] end of the expert's rows
    const bool staged = scratch != nullptr && segs <= kMoeScanCap;
    if (staged) {
        for (uint32_t i = tid; i < segs; i += nthreads) s_cnt[i] = recv[(i % L.ranks) * L.experts_local + i / L.ranks];
        __syncthreads();
    }
    if (tid == 0) {
        uint32_t prev_end = 0, flat = 0, tiles = 0;
        bool overflow = false;
        for (uint32_t el = 0; el < L.experts_local; ++el) {
            const uint32_t start = (prev_end + kMoePoolAlign - 1) / kMoePoolAlign * kMoePoolAlign;
            uint32_t row = start;
            for (uint32_t src = 0; src < L.ranks; ++src) {
                const uint32_t i = el * L.ranks + src;
                const uint32_t cnt = staged ? s_cnt[i] : recv[src * L.experts_local + el];
                if (staged) {
                    s_off[i] = row, s_pre[i] = flat;
                } else {
                    work[MoeWork::seg_off(L.experts_local) + i] = row;
                    work[MoeWork::seg_prefix(L.experts_local, L.ranks) + i] = flat;
                }
                row += cnt, flat += cnt;
            }
            if (staged) {
                s_end[el] = row;
                s_cnt[el] = row - start;   // the expert's row count, for the statistics (entry el is consumed by now)
            } else {
                work[MoeWork::psum_end() + el] = row;
                if (a.stats != nullptr) a.stats[el] += static_cast<int32_t>(row - start);
            }
            if (row > L.pool_rows) {
                // more rows arrived than the pool was sized for (a capacity below the worst case was asked for)
                overflow = true;
                break;
            }
            if (fused != nullptr) {
                // tiles of kMoeTileRows tokens over the expert's rows; the last one rounded up to the UMMA's N step
                const uint32_t total = row - start;
                work[fused->expert_tab + 2 * el] = start, work[fused->expert_tab + 2 * el + 1] = tiles;
                for (uint32_t off = 0; off < total; off += kMoeTileRows, ++tiles) {
                    uint32_t* t = work + fused->tile_table + tiles * 8;
                    const uint32_t valid = min(kMoeTileRows, total - off);
                    t[0] = start + off, t[1] = (valid + 15u) & ~15u, t[2] = el, t[3] = valid, t[4] = tiles * 256;
                }
            }
            prev_end = row;
        }
        if (overflow) {
            // Nothing may be written past the pool: the call is reported and goes on as a call without rows (no
            // pulls, no tiles), so that the barriers the peers wait at are still reached; y is not meaningful.
            if (atomicCAS(a.status, 0u, static_cast<uint32_t>(kStatusPoolOverflow)) == 0u) {
                a.status[1] = 110, a.status[2] = a.rank, a.status[3] = flat, a.status[4] = L.pool_rows;
                __threadfence_system();
            }
            prev_end = flat = tiles = 0;
            for (uint32_t el = 0; el < L.experts_local; ++el) {
                if (staged) s_end[el] = 0, s_cnt[el] = 0;
                else        work[MoeWork::psum_end() + el] = 0;
            }
        }
        if (staged) s_pre[segs] = flat;
        else        work[MoeWork::seg_prefix(L.experts_local, L.ranks) + segs] = flat;
        s_rows = (prev_end + kMoePoolAlign - 1) / kMoePoolAlign * kMoePoolAlign;
        ctrl[MoeCtrl::kTotalRows] = s_rows;
        s_tiles = tiles;
        if (fused != nullptr) ctrl[MoeCtrl::kNumTiles] = tiles;
    }
    __syncthreads();
    if (staged) {
        for (uint32_t i = tid; i < segs; i += nthreads) {
            work[MoeWork::seg_off(L.experts_local) + i] = s_off[i];
            work[MoeWork::seg_prefix(L.experts_local, L.ranks) + i] = s_pre[i];
        }
        if (tid == 0) work[MoeWork::seg_prefix(L.experts_local, L.ranks) + segs] = s_pre[segs];
        for (uint32_t el = tid; el < L.experts_local; el += nthreads) {
            work[MoeWork::psum_end() + el] = s_end[el];
            // one thread per expert: a serial read-modify-write per expert costs a memory round trip each
            if (a.stats != nullptr) a.stats[el] += static_cast<int32_t>(s_cnt[el]);
        }
        __threadfence();
    }
    __syncthreads();
    // Rows between an expert's end and the next boundary carry no token: mark them
    for (uint32_t el = 0; el < L.experts_local; ++el) {
        const uint32_t end = staged ? s_end[el] : work[MoeWork::psum_end() + el];
        const uint32_t stop = (end + kMoePoolAlign - 1) / kMoePoolAlign * kMoePoolAlign;
        for (uint32_t r = end + tid; r < stop; r += nthreads) meta[r * 3] = -1;
    }
    if (fused != nullptr) {
        for (uint32_t i = tid; i < s_tiles; i += nthreads) work[fused->pulled + i] = 0, work[fused->l1_done + i] = 0;
        __threadfence();
        __syncthreads();
        if (tid == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ctrl + MoeCtrl::kLayoutReady), "r"(s_call) : "memory");
    }
    return true;
}

__global__ void __launch_bounds__(256) moe_exchange_kernel(const MoeArgs a) {
    __shared__ uint32_t s_scan[kMoeScanWords];
    moe_exchange_body(a, threadIdx.x, 256, nullptr, s_scan);
}

// ---- step 3: pull every routed token (row, packed scales, route weight) into the pool.  One warp per row:
// flat rows first, first + stride, ...  The single kernel passes `pulled` (finished rows per tile) and `expert_tab`
// (first pool row and first tile per expert): its scale rows are laid out per tile.
DG_DEVICE void moe_pull_rows(const MoeArgs& a, const uint32_t* s_prefix, uint32_t first, uint32_t stride, uint32_t lane,
                             uint32_t* pulled, const uint32_t* expert_tab = nullptr) {
    const MoeLayout& L = a.L;
    const uint32_t* work = reinterpret_cast<const uint32_t*>(a.base[a.rank] + L.off_work);
    const uint32_t segments = L.experts_local * L.ranks;
    const uint32_t total = s_prefix[segments];
    const uint32_t* src_idx = reinterpret_cast<const uint32_t*>(a.base[a.rank] + L.off_src_idx);
    uint8_t* l1 = a.base[a.rank] + L.off_l1_acts;
    uint32_t* l1_sf = reinterpret_cast<uint32_t*>(a.base[a.rank] + L.off_l1_sf);
    float* pool_w = reinterpret_cast<float*>(a.base[a.rank] + L.off_pool_w);
    int32_t* meta = reinterpret_cast<int32_t*>(a.base[a.rank] + L.off_pool_meta);
    const uint32_t sf_words = L.hidden / 128;
    for (uint32_t r = first; r < total; r += stride) {
        // segment holding flat row r: last i with prefix[i] <= r
        uint32_t lo = 0, hi = segments;
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) / 2;
            if (s_prefix[mid] <= r) lo = mid; else hi = mid;
        }
        const uint32_t el = lo / L.ranks, src = lo % L.ranks, j = r - s_prefix[lo];
        const uint32_t pair = src_idx[(static_cast<uint64_t>(el) * L.ranks + src) * L.t_max + j];
        const uint32_t token = pair / L.topk, slot = pair % L.topk;
        const uint32_t dst = work[MoeWork::seg_off(L.experts_local) + lo] + j;
        const uint8_t* peer = a.base[src];
        const uint4* from = reinterpret_cast<const uint4*>(peer + L.off_x + static_cast<uint64_t>(token) * L.hidden);
        uint4* to = reinterpret_cast<uint4*>(l1 + static_cast<uint64_t>(dst) * L.hidden);
        // 8 independent 16-byte loads in flight per lane before the stores (peer loads have NVLink latency)
        const uint32_t vecs = L.hidden / 16;
        for (uint32_t c0 = 0; c0 < vecs; c0 += 256) {
            uint4 tmp[8];
#pragma unroll
            for (uint32_t u = 0; u < 8; ++u) {
                const uint32_t c = c0 + u * 32 + lane;
                if (c < vecs) tmp[u] = from[c];
            }
#pragma unroll
            for (uint32_t u = 0; u < 8; ++u) {
                const uint32_t c = c0 + u * 32 + lane;
                if (c < vecs) to[c] = tmp[u];
            }
        }
        const uint32_t* sf_from = reinterpret_cast<const uint32_t*>(peer + L.off_x_sf) + static_cast<uint64_t>(token) * sf_words;
        // scale words go straight into the per-128-row order tcgen05.cp reads (no transposition in the GEMM):
        // relative to the pool (kernel-per-phase path) or to the row's tile (single kernel)
        uint32_t sf_dst = moe_sf_row(dst), sf_ld = L.pool_rows, tile = 0;
        if (expert_tab != nullptr) {
            const uint32_t pos = dst - expert_tab[2 * el];
            tile = expert_tab[2 * el + 1] + pos / kMoeTileRows;
            sf_dst = tile * 256 + moe_sf_row(pos % kMoeTileRows), sf_ld = L.sf_rows;
        }
        for (uint32_t c = lane; c < sf_words; c += 32) l1_sf[static_cast<uint64_t>(c) * sf_ld + sf_dst] = sf_from[c];
        if (lane == 0) {
            pool_w[dst] = reinterpret_cast<const float*>(peer + L.off_topk_w)[pair];
            meta[dst * 3 + 0] = static_cast<int32_t>(src);
            meta[dst * 3 + 1] = static_cast<int32_t>(token);
            meta[dst * 3 + 2] = static_cast<int32_t>(slot);
        }
        if (pulled != nullptr) {
            // the row is read by TMA (async proxy) in another CTA once the block's count is complete
            asm volatile("fence.proxy.async;" ::: "memory");
            __threadfence();
            __syncwarp();
            if (lane == 0) atomicAdd(pulled + tile, 1u);
        }
    }
}

__global__ void __launch_bounds__(256) moe_pull_kernel(const MoeArgs a) {
    const MoeLayout& L = a.L;
    const uint32_t* work = reinterpret_cast<const uint32_t*>(a.base[a.rank] + L.off_work);
    extern __shared__ uint32_t s_prefix[];   // [segments + 1]
    const uint32_t segments = L.experts_local * L.ranks;
    for (uint32_t i = threadIdx.x; i <= segments; i += 256)
        s_prefix[i] = work[MoeWork::seg_prefix(L.experts_local, L.ranks) + i];
    __syncthreads();
    moe_pull_rows(a, s_prefix, blockIdx.x * 8 + threadIdx.x / 32, gridDim.x * 8, threadIdx.x & 31, nullptr);
}

// ---- shared experts: every row of the token buffer is its own pool row, bound for plane `topk` of this rank
__global__ void __launch_bounds__(256) moe_shared_meta_kernel(const MoeArgs a) {
    const uint32_t t = blockIdx.x * 256 + threadIdx.x;
    const uint32_t t_al = (a.L.t_max + 127) / 128 * 128;
    if (t >= t_al) return;
    int32_t* meta = reinterpret_cast<int32_t*>(a.base[a.rank] + a.L.off_shared_meta) + t * 3;
    meta[0] = t < a.num_tokens ? static_cast<int32_t>(a.rank) : -1;
    meta[1] = static_cast<int32_t>(t), meta[2] = static_cast<int32_t>(a.L.topk);
}

// ---- cross-rank barrier on its own (after the experts' ranks have pushed their results).  One CTA.
__global__ void __launch_bounds__(32) moe_barrier_kernel(const MoeArgs a) {
    const uint32_t* ctrl = reinterpret_cast<const uint32_t*>(a.base[a.rank]);
    if (threadIdx.x < a.L.ranks) moe_cross_rank_barrier(a, 1, 2 * ctrl[MoeCtrl::kCall], threadIdx.x);
}

// ---- last step: y[t] = bf16(sum over the token's valid slots, in slot order, of its combine rows).
// `nthreads` threads of one CTA own 8 consecutive columns each per pass.
// Columns [c, c + 8) and, if second, [c2, c2 + 8) of token t: every slot load of both column groups is issued before
// any is used, so a thread keeps up to 16 16-byte loads in flight (the fused kernel has few threads per SM).
template <bool kTwo>
DG_DEVICE void moe_reduce_cols(const MoeArgs& a, __nv_bfloat16* y, int64_t ldy, uint32_t t, uint32_t c, uint32_t c2) {
    const MoeLayout& L = a.L;
    const long long* idx = reinterpret_cast<const long long*>(a.base[a.rank] + L.off_topk_idx) + static_cast<uint64_t>(t) * L.topk;
    const uint8_t* col = a.base[a.rank] + L.off_combine + (static_cast<uint64_t>(t) * L.hidden + c) * 2;
    const int64_t delta = (static_cast<int64_t>(c2) - static_cast<int64_t>(c)) * 2;
    const uint64_t plane = static_cast<uint64_t>(L.t_max) * L.hidden * 2;
    float acc0[8] = {0, 0, 0, 0, 0, 0, 0, 0}, acc1[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (L.shared != 0) {   // the shared experts' row goes first, then the routed slots in slot order
        const uint4 v0 = *reinterpret_cast<const uint4*>(col + L.topk * plane);
        const uint4 v1 = kTwo ? *reinterpret_cast<const uint4*>(col + L.topk * plane + delta) : make_uint4(0, 0, 0, 0);
        const __nv_bfloat162* b0 = reinterpret_cast<const __nv_bfloat162*>(&v0);
        const __nv_bfloat162* b1 = reinterpret_cast<const __nv_bfloat162*>(&v1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f0 = __bfloat1622float2(b0[i]), f1 = __bfloat1622float2(b1[i]);
            acc0[2 * i] = f0.x, acc0[2 * i + 1] = f0.y, acc1[2 * i] = f1.x, acc1[2 * i + 1] = f1.y;
        }
    }
    for (uint32_t s0 = 0; s0 < L.topk; s0 += 8) {
        uint4 v0[8], v1[8];
        uint32_t mask = 0;
#pragma unroll
        for (uint32_t u = 0; u < 8; ++u) {
            const uint32_t s = s0 + u;
            v0[u] = make_uint4(0, 0, 0, 0), v1[u] = make_uint4(0, 0, 0, 0);
            if (s < L.topk) {
                const long long e = idx[s];
                if (e >= 0 && e < static_cast<long long>(L.experts)) {
                    mask |= 1u << u;
                    v0[u] = *reinterpret_cast<const uint4*>(col + s * plane);
                    if (kTwo) v1[u] = *reinterpret_cast<const uint4*>(col + s * plane + delta);
                }
            }
        }
        // masked slots hold +0.0 and leave the sums unchanged, so the order of the valid ones is the slot order
#pragma unroll
        for (uint32_t u = 0; u < 8; ++u) {
            const __nv_bfloat162* b0 = reinterpret_cast<const __nv_bfloat162*>(&v0[u]);
            const __nv_bfloat162* b1 = reinterpret_cast<const __nv_bfloat162*>(&v1[u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f0 = __bfloat1622float2(b0[i]);
                acc0[2 * i] += f0.x, acc0[2 * i + 1] += f0.y;
                if (kTwo) {
                    const float2 f1 = __bfloat1622float2(b1[i]);
                    acc1[2 * i] += f1.x, acc1[2 * i + 1] += f1.y;
                }
            }
        }
        (void)mask;
    }
    uint4 out;
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc0[2 * i], acc0[2 * i + 1]);
    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(y) + (static_cast<uint64_t>(t) * ldy + c) * 2) = out;
    if (kTwo) {
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc1[2 * i], acc1[2 * i + 1]);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(y) + (static_cast<uint64_t>(t) * ldy + c2) * 2) = out;
    }
}
DG_DEVICE void moe_reduce_token(const MoeArgs& a, __nv_bfloat16* y, int64_t ldy, uint32_t t, uint32_t tid, uint32_t nthreads) {
    for (uint32_t c = tid * 8; c < a.L.hidden; c += nthreads * 8) moe_reduce_cols<false>(a, y, ldy, t, c, c);
}

// grid: num_tokens, block: 128
__global__ void __launch_bounds__(128) moe_reduce_kernel(const MoeArgs a, __nv_bfloat16* y, int64_t ldy) {
    moe_reduce_token(a, y, ldy, blockIdx.x, threadIdx.x, 128);
}

}  // namespace dg
