// Mega MoE forward as ONE persistent kernel: dispatch (count, index scatter, count exchange, token pull over
// NVLink peer loads), the two expert GEMMs (tcgen05 block-scaled UMMA, 2-CTA pairs, 256-token tiles) with the
// SwiGLU / requantisation and combine-push epilogues, and the top-k reduction.
//
// Dataflow inside the launch: pull warps fill the expert-sorted pool in pool order and count rows per token
// tile; the TMA producer starts a first-GEMM tile as soon as its rows are there; second-GEMM tiles of token
// tile j - lag are interleaved after the first-GEMM tiles of tile j and wait (rarely) on a per-tile counter
// that the first GEMM's epilogue bumps; the combine push therefore spreads over the whole kernel.  Two
// grid-wide barriers (after the scatter, before the reduction) and two cross-rank barriers per call.
// Every wait is bounded and reports through the status block.
//
// Takes the role of sm100_fp8_fp4_mega_moe_impl
// (deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_mega_moe.cuh:64-94) and its scheduler
// (deep_gemm/include/deep_gemm/scheduler/mega_moe.cuh:372-476).
#pragma once

#include "mega_moe.cuh"

namespace dg {

constexpr uint32_t kFusedThreads = 544;   // 17 warps: 0 weight copies, 1 UMMA, 2 + 8..11 pull, 3 scale copies, 12 token copies,
                                          // 4..7 and 13..16 the two epilogue groups

struct MoeFusedParams {
    CUtensorMap tm_w[2], tm_wsf[2], tm_act[2], tm_actsf[2];   // [0]: first GEMM (W13, pool tokens), [1]: second (W2, activations)
    CUtensorMap tm_act_small[2][2];   // [gemm][0: 32, 1: 64 token rows per CTA]: ragged tiles fetch fewer rows
    MoeArgs a;
    MoeEpilogueParams e;
    __nv_bfloat16* y;
    int64_t ldy;
    uint32_t num_ctas;
    unsigned long long* trace;   // optional per-CTA time stamps (builds with DG_TRACE only)
    uint32_t lag;   // token tiles between a tile's first-GEMM slots and its second-GEMM slots in the schedule
    uint32_t w_fp8; // expert weights are E4M3 bytes instead of packed E2M1 codes
};

struct FusedCfg {
    static constexpr uint32_t BN = kMoeTileRows, R_STAGE = 128 * 128, C_STAGE = BN / 2 * 128, SFR_STAGE = 512, SFC_STAGE = 1024;
    static constexpr uint32_t STAGE_BYTES = R_STAGE + C_STAGE + SFR_STAGE + SFC_STAGE;
    static constexpr uint32_t PITCH = 272;
    static constexpr uint32_t TABLE_OFF = 2 * 32 * PITCH;
    static constexpr uint32_t PREFIX_OFF = TABLE_OFF + 2 * 256 * 8;   // (expert, source) segment prefix, <= 512 words
    static constexpr uint32_t kMaxSegments = 511;
    static constexpr uint32_t CD_BYTES = (PREFIX_OFF + 512 * 4 + 1023) / 1024 * 1024;
    static constexpr uint32_t kStages = (232448 - 1024 - CD_BYTES - 1024) / STAGE_BYTES;
    static constexpr uint32_t kSmemBytes = 1024 + kStages * STAGE_BYTES + CD_BYTES + 1024;
    // Two accumulators of BN columns, then 4 + 8 scale columns; where that exceeds tensor memory the accumulators share
    // kOverlap columns (stage 0's last, stage 1's first)
    static constexpr uint32_t kOverlap = 2 * BN + 12 > 512 ? 16 : 0;
    static constexpr uint32_t kAccStride = BN - kOverlap, kSfrCol = 2 * BN - kOverlap, kSfcCol = kSfrCol + 4;
    static constexpr uint32_t kTmemCols = 512;
};
static_assert(FusedCfg::kStages >= 4 && FusedCfg::kStages <= 10, "stage count");
static_assert(FusedCfg::kSfcCol + 8 <= FusedCfg::kTmemCols && FusedCfg::C_STAGE % 1024 == 0 && FusedCfg::BN % 16 == 0, "tile");

struct FusedTile {
    uint32_t kind;   // 0: first GEMM, 1: second GEMM
    uint32_t tile, row0, rows, group, n_blk, valid, sf_base;
};

// Bounded spin on a device-scope counter; false on timeout / abort.
DG_DEVICE bool fused_wait_counter(const uint32_t* counter, uint32_t target, volatile uint32_t* abort_flag,
                                  const MoeArgs& a, uint32_t site, uint32_t info) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    if (static_cast<int32_t>(v - target) >= 0) return true;
    const uint64_t t0 = global_timer_ns();
    const uint64_t budget = static_cast<uint64_t>(a.timeout_ms) * 1000000ull;
    while (true) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (static_cast<int32_t>(v - target) >= 0) return true;
        __nanosleep(100);
        if (*abort_flag) return false;
        if (global_timer_ns() - t0 > budget) {
            if (atomicCAS(a.status, 0u, static_cast<uint32_t>(kStatusTimeout)) == 0u) {
                a.status[1] = site, a.status[2] = blockIdx.x, a.status[3] = info, a.status[4] = v, a.status[5] = target;
                __threadfence_system();
            }
            *abort_flag = 1;
            return false;
        }
    }
}


// Schedule slot -> tile.  The order is that of rounds of (n1 + n2) slots, round j holding the first GEMM's n1 tiles of
// token tile j and the second GEMM's n2 tiles of token tile j - lag, with the slots that have no tile left out: the
// first `lag` rounds hold first-GEMM tiles only, the last `lag` second-GEMM tiles only.  (With the empty slots left
// in, the units' shares of the last rounds differed by several tiles and the first CTA finished 40-70 us before the
// last.)  num_tiles * (n1 + n2) slots in all; a second-GEMM tile always comes after the first-GEMM tiles it reads.
DG_DEVICE bool fused_slot_to_tile(const uint32_t* table, uint32_t num_tiles, uint32_t n1, uint32_t n2, uint32_t lag,
                                  uint32_t slot, FusedTile& t) {
    const uint32_t head = min(lag, num_tiles);          // token tiles whose two GEMMs are not interleaved with others'
    const uint32_t head_slots = head * n1, mid_slots = (num_tiles - head) * (n1 + n2);
    if (slot < head_slots) {
        t.kind = 0, t.tile = slot / n1, t.n_blk = slot % n1;
    } else if (slot - head_slots < mid_slots) {
        const uint32_t s = slot - head_slots, round = head + s / (n1 + n2), r = s % (n1 + n2);
        if (r < n1) t.kind = 0, t.tile = round, t.n_blk = r;
        else        t.kind = 1, t.tile = round - lag, t.n_blk = r - n1;
    } else {
        const uint32_t s = slot - head_slots - mid_slots;
        if (s >= head * n2) return false;
        t.kind = 1, t.tile = num_tiles - head + s / n2, t.n_blk = s % n2;
    }
    const uint32_t* e = table + t.tile * 8;
    t.row0 = e[0], t.rows = e[1], t.group = e[2], t.valid = e[3], t.sf_base = e[4];
    return true;
}

// Grid-wide barrier (all CTAs co-resident: at most one per SM).  Whole CTA calls it.  Self-contained: the last of
// the `num_ctas` arrivers puts the arrival count back to zero and bumps the generation word the others wait on, so
// the barrier does not depend on how many CTAs earlier launches had or on how many barriers they passed.  (A launch
// that gives up on a wait leaves the count behind: the buffer's control block must then be cleared, see
// SymmBuffer.reset.)
DG_DEVICE bool fused_grid_barrier(uint32_t* ctrl, uint32_t num_ctas, volatile uint32_t* abort_flag, const MoeArgs& a,
                                  uint32_t site) {
    __shared__ uint32_t s_ok;
    // The CTA's threads meet first; then ONE system-scope fence by the arriving thread orders everything the CTA wrote
    // (its stores to peer buffers too) before the arrival: a fence by each of the 544 threads cost several
    // microseconds per barrier.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        uint32_t* count = ctrl + MoeCtrl::kGridCount;
        uint32_t* gen = ctrl + MoeCtrl::kGridGen;
        uint32_t my_gen;   // read before arriving: the generation cannot move until this CTA has arrived
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(my_gen) : "l"(gen) : "memory");
        const uint32_t prev = atomicAdd(count, 1u);
        if (prev + 1 == num_ctas) {
            atomicExch(count, 0u);
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(gen), "r"(my_gen + 1) : "memory");
            s_ok = 1u;
        } else {
            s_ok = fused_wait_counter(gen, my_gen + 1, abort_flag, a, site, prev) ? 1u : 0u;
        }
    }
    __syncthreads();
    return s_ok != 0;
}

// Top-k reduction of this CTA's share of the tokens with the combine rows staged through shared
// memory by bulk copies: one item = one token x one piece of kReducePiece columns x all of its valid slots (up to 8
// rows of 6 KB), kReduceStages items in flight per CTA, so the memory-level parallelism does not depend on the
// number of threads.  Thread 0 issues, all threads sum (slot order, FP32) and store BF16.  The kernel's operand
// stages are free by now (all roles have left their loops and the grid barrier has passed).
#ifndef DG_REDUCE_PIECE
#define DG_REDUCE_PIECE (FusedCfg::BN == 256 ? 3072 : 2560)
#define DG_REDUCE_STAGES 4
#endif
constexpr uint32_t kReducePiece = DG_REDUCE_PIECE, kReduceStages = DG_REDUCE_STAGES, kReduceSlotBytes = kReducePiece * 2;
static_assert(kReducePiece <= kFusedThreads * 8 && kReducePiece % 8 == 0, "one 8-column group per thread");
static_assert(kReduceStages * 8 * kReduceSlotBytes <= FusedCfg::kStages * (FusedCfg::R_STAGE + FusedCfg::C_STAGE), "reduce stages");
static_assert((kReduceStages - 1) * 9 * kReduceSlotBytes <= FusedCfg::kStages * (FusedCfg::R_STAGE + FusedCfg::C_STAGE), "reduce stages, nine rows");

DG_DEVICE void fused_reduce_bulk(const MoeFusedParams& p, uint8_t* smem_gen, uint32_t smem_base,
                                 volatile uint32_t* abort_flag, const GemmParams& wp) {
    // A contiguous run of tokens per CTA: at any moment the CTAs read rows far apart from one another
    const uint32_t per_cta = (p.a.num_tokens + p.num_ctas - 1) / p.num_ctas;
    const uint32_t first_token = min(blockIdx.x * per_cta, p.a.num_tokens);
    const uint32_t my_tokens = min(per_cta, p.a.num_tokens - first_token);
    __shared__ __align__(8) uint64_t s_full[kReduceStages];
    __shared__ uint32_t s_mask[kReduceStages];
    const MoeLayout& L = p.a.L;
    // rows per item: the routed slots plus, with shared experts, their plane; nine rows leave room for three stages
    const uint32_t np = L.planes, nst = np <= 8 ? kReduceStages : kReduceStages - 1;
    const uint32_t pieces = (L.hidden + kReducePiece - 1) / kReducePiece;
    const uint32_t num_items = my_tokens * pieces;
    const uint8_t* combine = p.a.base[p.a.rank] + L.off_combine;
    const long long* topk_idx = reinterpret_cast<const long long*>(p.a.base[p.a.rank] + L.off_topk_idx);
    const uint64_t plane = static_cast<uint64_t>(L.t_max) * L.hidden * 2;
    if (threadIdx.x == 0) {
        for (uint32_t i = 0; i < kReduceStages; ++i) mbar_init(&s_full[i], 1);
        fence_mbar_init();
    }
    // Valid-slot masks of this CTA's tokens, computed by all threads up front: the issuing thread must not sit on
    // global loads between items (it is on every item's critical path).
    auto token_mask = [&](uint32_t i) {
        const long long* idx = topk_idx + static_cast<uint64_t>(first_token + i) * L.topk;
        uint32_t mask = 0;
        for (uint32_t u = 0; u < L.topk; ++u) {
            const long long e = idx[u];
            if (e >= 0 && e < static_cast<long long>(L.experts)) mask |= 1u << u;
        }
        if (L.shared != 0) mask |= 1u << L.topk;   // the shared experts' plane holds a row for every token
        return mask;
    };
    constexpr uint32_t kMaskCap = FusedCfg::CD_BYTES / 4;
    uint32_t* s_token_mask = reinterpret_cast<uint32_t*>(smem_gen + FusedCfg::kStages * (FusedCfg::R_STAGE + FusedCfg::C_STAGE));
    for (uint32_t i = threadIdx.x; i < min(my_tokens, kMaskCap); i += kFusedThreads) s_token_mask[i] = token_mask(i);
    __syncthreads();

    // Lane 0 of warp u issues slot u's copy (eight issuing threads: one thread issuing all eight copies of an item
    // spends longer on that than the copies take); thread 0 also posts the expected byte count.
    auto issue = [&](uint32_t it) {   // threads 0, 32, ..., 32 * (np - 1)
        const uint32_t s = it % nst, i = it / pieces, u = threadIdx.x / 32;
        const uint32_t t = first_token + i, c0 = (it % pieces) * kReducePiece;
        const uint32_t bytes = min(kReducePiece, L.hidden - c0) * 2;
        const uint32_t mask = i < kMaskCap ? s_token_mask[i] : token_mask(i);
        if (threadIdx.x == 0) {
            s_mask[s] = mask;
            mbar_arrive_expect_tx(&s_full[s], __popc(mask) * bytes);
        }
        if (mask >> u & 1) {
            const uint8_t* src = combine + (static_cast<uint64_t>(t) * L.hidden + c0) * 2;
            bulk_load(smem_base + (s * np + u) * kReduceSlotBytes, src + u * plane, bytes, smem_u32(&s_full[s]));
        }
    };
    const bool issuer = threadIdx.x % 32 == 0 && threadIdx.x / 32 < np;

    if (issuer)
        for (uint32_t it = 0; it + 1 < nst && it < num_items; ++it) issue(it);
    for (uint32_t it = 0; it < num_items; ++it) {
        const uint32_t s = it % nst;
        if (issuer && it + nst - 1 < num_items) issue(it + nst - 1);
        const bool ok = wait_barrier(&s_full[s], (it / nst) & 1, abort_flag, 0, wp, 207, it, 0, s);
        if (ok) {
            const uint32_t t = first_token + it / pieces, c0 = (it % pieces) * kReducePiece;
            const uint32_t width = min(kReducePiece, L.hidden - c0), c = threadIdx.x * 8;
            if (c < width) {
                const uint32_t mask = s_mask[s] & ((1u << L.topk) - 1u);   // routed slots; the shared plane is added first
                const uint8_t* src = smem_gen + s * np * kReduceSlotBytes + c * 2;
                float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (L.shared != 0) {   // the shared experts' row first, then the routed slots in slot order
                    const uint4 v = *reinterpret_cast<const uint4*>(src + L.topk * kReduceSlotBytes);
                    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float2 f = __bfloat1622float2(b[i]);
                        acc[2 * i] = f.x, acc[2 * i + 1] = f.y;
                    }
                }
#pragma unroll
                for (uint32_t u = 0; u < 8; ++u) {
                    if (mask >> u & 1) {
                        const uint4 v = *reinterpret_cast<const uint4*>(src + u * kReduceSlotBytes);
                        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 f = __bfloat1622float2(b[i]);
                            acc[2 * i] += f.x, acc[2 * i + 1] += f.y;
                        }
                    }
                }
                uint4 out;
                __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
                for (int i = 0; i < 4; ++i) o[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
                *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.y) + (static_cast<uint64_t>(t) * p.ldy + c0 + c) * 2) = out;
            }
        }
        if (!__syncthreads_and(ok ? 1 : 0)) break;   // the stage may be refilled; every thread leaves together on a failed wait
    }
}

#ifdef DG_TRACE
// Cycles spent in a wait, summed per warp into trace slots 5..7 (timing studies only)
#define DG_FUSED_TIMED(slot_, stmt_) do { const long long t0_ = clock64(); stmt_; wait_cycles[(slot_) - 5] += clock64() - t0_; } while (0)
#define DG_FUSED_FLUSH() do { if (p.trace != nullptr && lane == 0) { for (int i_ = 0; i_ < 3; ++i_) p.trace[(blockIdx.x * 20 + warp) * 8 + 5 + i_] = wait_cycles[i_]; \
    if (warp == 4) for (int i_ = 0; i_ < 8; ++i_) p.trace[(blockIdx.x * 20 + 18) * 8 + i_] = epi_cycles[i_]; } } while (0)
#define DG_EPI_TIMED(slot_, stmt_) do { const long long t0_ = clock64(); stmt_; epi_cycles[slot_] += clock64() - t0_; } while (0)
#define DG_FUSED_STAMP(slot_) do { if (p.trace != nullptr && lane == 0) { p.trace[(blockIdx.x * 20 + warp) * 8 + (slot_)] = global_timer_ns(); if (warp == 0) p.trace[(blockIdx.x * 20 + 19) * 8 + (slot_)] = clock64(); } } while (0)
// Finer stamps of thread 0 of every CTA (row 17): 0 scatter done, 1 grid barrier 1 passed, 2 exchange done (CTA 0),
// 3 layout seen, 4 grid barrier 2 passed, 5 cross-rank barrier 2 passed (CTA 0)
#define DG_FUSED_STAMP0(slot_) do { if (p.trace != nullptr && threadIdx.x == 0) p.trace[(blockIdx.x * 20 + 17) * 8 + (slot_)] = global_timer_ns(); } while (0)
#else
#define DG_FUSED_STAMP0(slot_) do { } while (0)
#define DG_FUSED_STAMP(slot_) do { } while (0)
#define DG_FUSED_TIMED(slot_, stmt_) do { stmt_; } while (0)
#define DG_FUSED_FLUSH() do { } while (0)
#define DG_EPI_TIMED(slot_, stmt_) do { stmt_; } while (0)
#endif

__global__ void __launch_bounds__(kFusedThreads, 1) mega_moe_fused_kernel(const __grid_constant__ MoeFusedParams p) {
    using Cfg = FusedCfg;
    constexpr uint32_t kStages = Cfg::kStages, BN = Cfg::BN;
    const MoeLayout& L = p.a.L;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t smem_r = smem_base;
    const uint32_t smem_c = smem_r + kStages * Cfg::R_STAGE;
    const uint32_t smem_cd = smem_c + kStages * Cfg::C_STAGE;
    const uint32_t smem_sfr = smem_cd + Cfg::CD_BYTES;
    const uint32_t smem_sfc = smem_sfr + kStages * Cfg::SFR_STAGE;
    GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(smem_gen + (smem_sfc + kStages * Cfg::SFC_STAGE - smem_base));
    uint32_t* s_prefix = reinterpret_cast<uint32_t*>(smem_gen + (smem_cd - smem_base) + Cfg::PREFIX_OFF);   // [segments + 1]

    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t cta_rank = cluster_ctarank();
    const bool is_leader = cta_rank == 0;
    const uint32_t unit = blockIdx.x / 2, num_units = p.num_ctas / 2;
    volatile uint32_t* abort_flag = &bars->abort;
    __shared__ __align__(8) uint64_t s_epi_bar[2][2];   // per epilogue group: staging buffer written / read
    const uint32_t peer_abort = map_to_cta(smem_u32(&bars->abort), cta_rank ^ 1);
    uint32_t* work = reinterpret_cast<uint32_t*>(p.a.base[p.a.rank] + L.off_work);
    uint32_t* ctrl = reinterpret_cast<uint32_t*>(p.a.base[p.a.rank]);
    GemmParams wp;   // only the fields wait_barrier reports through
    wp.timeout_ms = p.a.timeout_ms, wp.status = p.a.status;

    // ---------------------------------------------------------------- set-up
    if (warp == 0 && lane == 0) {
        for (uint32_t i = 0; i < 2; ++i) {
            prefetch_tmap(&p.tm_w[i]), prefetch_tmap(&p.tm_wsf[i]), prefetch_tmap(&p.tm_act[i]), prefetch_tmap(&p.tm_actsf[i]);
        }
        for (uint32_t i = 0; i < kStages; ++i) {
            mbar_init(&bars->full[i], 6);    // both CTAs' weight, token and scale producers; every copy of the stage lands here
            mbar_init(&bars->empty[i], 1);   // UMMA commit
        }
        for (uint32_t i = 0; i < 2; ++i) {
            mbar_init(&bars->tmem_full[i], 1);
            mbar_init(&bars->tmem_empty[i], 2 * 4);
            mbar_init(&bars->overlap[i], 2 * 4);
            mbar_init(&s_epi_bar[i][0], 4), mbar_init(&s_epi_bar[i][1], 4);
        }
        bars->abort = 0;
        fence_mbar_init();
    }
    cluster_sync();
    if (warp == 1) {
        tmem_alloc<2>(&bars->tmem_base, Cfg::kTmemCols);
        tmem_relinquish<2>();
    }
    tc_fence_before();
    cluster_sync();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    DG_FUSED_STAMP(0);
    // ---------------------------------------------------------------- dispatch, step 1: count and scatter indices
    const uint32_t call_old = *reinterpret_cast<volatile uint32_t*>(ctrl + MoeCtrl::kCall);   // CTA 0 bumps it after barrier 1
    const uint32_t call_new = call_old + 1;
    for (uint32_t i = blockIdx.x * kFusedThreads + threadIdx.x; i < p.a.num_tokens * L.topk; i += p.num_ctas * kFusedThreads)
        moe_scatter_pair(p.a, i);
    DG_FUSED_STAMP0(0);
    bool ok = fused_grid_barrier(ctrl, p.num_ctas, abort_flag, p.a, 201);
    DG_FUSED_STAMP0(1);
    // step 2 (CTA 0): publish counts, cross-rank barrier, pool layout, tile table, counters, layout_ready
    if (ok && blockIdx.x == 0) {
        MoeFusedHooks hooks;
        hooks.tile_table = MoeFusedWork::tile_table(L), hooks.pulled = MoeFusedWork::pulled(L);
        hooks.l1_done = MoeFusedWork::l1_done(L), hooks.expert_tab = MoeFusedWork::expert_tab(L);
        // the operand stages are idle until the roles start: their first words serve the layout scan
        moe_exchange_body(p.a, threadIdx.x, kFusedThreads, &hooks, reinterpret_cast<uint32_t*>(smem_gen));
        DG_FUSED_STAMP0(2);
    }
    if (ok) {
        if (threadIdx.x == 0)
            ok = fused_wait_counter(ctrl + MoeCtrl::kLayoutReady, call_new, abort_flag, p.a, 202, call_new);
        // every thread needs the outcome and the layout
        __shared__ uint32_t s_layout_ok;
        if (threadIdx.x == 0) s_layout_ok = ok ? 1u : 0u;
        __syncthreads();
        ok = s_layout_ok != 0;
        DG_FUSED_STAMP0(3);
    }
    const uint32_t num_tiles = ok ? ctrl[MoeCtrl::kNumTiles] : 0;
    const uint32_t* table = work + MoeFusedWork::tile_table(L);
    uint32_t* pulled = work + MoeFusedWork::pulled(L);
    uint32_t* l1_done = work + MoeFusedWork::l1_done(L);
    const uint32_t n1 = 2 * L.inter / 256, n2 = L.hidden / 256;
    const uint32_t num_slots = ok ? num_tiles * (n1 + n2) : 0;
    const uint32_t segments = L.experts_local * L.ranks;
    if (ok) {
        for (uint32_t i = threadIdx.x; i <= segments; i += kFusedThreads)
            s_prefix[i] = work[MoeWork::seg_prefix(L.experts_local, L.ranks) + i];
    }
    __syncthreads();

    DG_FUSED_STAMP(1);
    uint32_t stage = 0, phase = 0;
    auto advance = [&]() {
        stage = stage + 1 == kStages ? 0 : stage + 1;
        phase ^= (stage == 0);
    };
    uint32_t acc_iter = 0;
    FusedTile tc;
    long long wait_cycles[3] = {0, 0, 0};
    long long epi_cycles[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    (void)wait_cycles, (void)epi_cycles;

    if (warp == 0 || warp == 3 || warp == 12) {
        // ============================================================ TMA producers: warp 0 weight tiles, warp 12 token tiles,
        // warp 3 scale factors (one thread needs 150-200 cycles per copy it issues; a K block has four)
        const bool sf_role = warp == 3, w_role = warp == 0;
        const uint32_t full_bar0 = map_to_cta(smem_u32(&bars->full[0]), 0);
        for (uint32_t slot = unit; slot < num_slots && ok; slot += num_units) {
            if (!fused_slot_to_tile(table, num_tiles, n1, n2, p.lag, slot, tc)) continue;
            // Data dependencies: pool rows pulled (first GEMM) / activations written (second GEMM)
            if (tc.kind == 0) {
                DG_FUSED_TIMED(5, ok = fused_wait_counter(pulled + tc.tile, tc.valid, abort_flag, p.a, 203, tc.tile));
            } else {
                DG_FUSED_TIMED(7, ok = fused_wait_counter(l1_done + tc.tile, n1 * 8, abort_flag, p.a, 204, tc.tile));
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");   // the rows were written through the generic proxy
            const uint32_t k = tc.kind;
            const uint32_t pk = (k == 0 ? L.hidden : L.inter) / 128;          // packed scale words per row
            const uint32_t r_mn = tc.n_blk * 256 + cta_rank * 128;   // row inside the expert; the expert is the map's third coordinate
            const uint32_t sfr_mn = tc.n_blk * 256 + cta_rank * 128, sfr_k = tc.group * pk;
            const uint32_t c_mn = tc.row0 + cta_rank * (tc.rows / 2);
            const uint32_t sfc_mn = tc.sf_base;   // the tile's own 256 scale rows
            const uint32_t num_kb = pk;
            const uint32_t per_cta = tc.rows / 2;
            const CUtensorMap* tm_act = per_cta <= 32 ? &p.tm_act_small[k][0] : per_cta <= 64 ? &p.tm_act_small[k][1] : &p.tm_act[k];
            const uint32_t tx_bytes = (per_cta <= 32 ? 32u : per_cta <= 64 ? 64u : BN / 2) * 128u;
            for (uint32_t kb = 0; kb < num_kb; ++kb, advance()) {
                DG_FUSED_TIMED(6, ok = wait_barrier(&bars->empty[stage], phase ^ 1, abort_flag, peer_abort, wp, kSiteProducerEmpty, acc_iter, kb, stage));
                if (!ok) break;
                if (elect_one()) {
                    const uint32_t full_bar = full_bar0 + stage * 8;
                    if (sf_role) {
                        mbar_arrive_expect_tx_cluster(full_bar, Cfg::SFR_STAGE + Cfg::SFC_STAGE);
                        tma_load_2d<true>(smem_sfr + stage * Cfg::SFR_STAGE, &p.tm_wsf[k], full_bar, sfr_mn, sfr_k + kb);
                        tma_load_2d<true>(smem_sfc + stage * Cfg::SFC_STAGE, &p.tm_actsf[k], full_bar, sfc_mn, kb);
                    } else if (w_role) {
                        mbar_arrive_expect_tx_cluster(full_bar, p.w_fp8 ? Cfg::R_STAGE : Cfg::R_STAGE / 2);   // FP4 weights count packed bytes
                        tma_load_3d<true>(smem_r + stage * Cfg::R_STAGE, &p.tm_w[k], full_bar, kb * 128, r_mn, tc.group);
                    } else {
                        mbar_arrive_expect_tx_cluster(full_bar, tx_bytes);
                        tma_load_3d<true>(smem_c + stage * Cfg::C_STAGE, tm_act, full_bar, kb * 128, c_mn, 0);
                    }
                }
                __syncwarp();
            }
            ++acc_iter;
        }
    } else if (warp == 1) {
        // ============================================================ UMMA issuer (leader CTA)
        if (is_leader) {
            const uint32_t idesc_base = make_idesc_mxf8f6f4(p.w_fp8 ? kFmtE4M3 : kFmtE2M1, kFmtE4M3, false, false, 256, BN);
            const uint64_t sf_desc_hi = make_smem_desc(0, 0, 128, kSwizzleNone);
            const uint32_t op_hi = static_cast<uint32_t>(make_smem_desc(0, 0, 1024, kSwizzle128B) >> 32);
            const uint32_t r_lo0 = static_cast<uint32_t>(make_smem_desc(smem_r, 0, 1024, kSwizzle128B));
            const uint32_t c_lo0 = static_cast<uint32_t>(make_smem_desc(smem_c, 0, 1024, kSwizzle128B));
            const uint32_t sfr_tmem = tmem_base + Cfg::kSfrCol, sfc_tmem = tmem_base + Cfg::kSfcCol;
            for (uint32_t slot = unit; slot < num_slots && ok; slot += num_units) {
                if (!fused_slot_to_tile(table, num_tiles, n1, n2, p.lag, slot, tc)) continue;
                const uint32_t acc = acc_iter & 1, acc_phase = (acc_iter >> 1) & 1;
                DG_FUSED_TIMED(5, ok = wait_barrier(&bars->tmem_empty[acc], acc_phase ^ 1, abort_flag, peer_abort, wp, kSiteMmaTmemEmpty, acc_iter, 0, acc));
                if (Cfg::kOverlap > 0 && ok && acc_iter > 0) {
                    // the tile before this one has been read out of the columns the two accumulators share
                    const uint32_t prev = acc_iter - 1;
                    DG_FUSED_TIMED(7, ok = wait_barrier(&bars->overlap[prev & 1], (prev >> 1) & 1, abort_flag, peer_abort, wp, kSiteMmaOverlap, acc_iter, 0, acc));
                }
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * Cfg::kAccStride;
                const uint32_t idesc_tile = idesc_with_n(idesc_base, tc.rows);
                const uint32_t num_kb = (tc.kind == 0 ? L.hidden : L.inter) / 128;
                for (uint32_t kb = 0; kb < num_kb; ++kb, advance()) {
                    DG_FUSED_TIMED(6, ok = wait_barrier(&bars->full[stage], phase, abort_flag, peer_abort, wp, kSiteMmaFull, acc_iter, kb, stage));
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one()) {
                        utccp_32x128b_warpx4<2>(sfr_tmem, sf_desc_hi | ((smem_sfr + stage * Cfg::SFR_STAGE) >> 4));
                        utccp_32x128b_warpx4<2>(sfc_tmem, sf_desc_hi | ((smem_sfc + stage * Cfg::SFC_STAGE) >> 4));
                        utccp_32x128b_warpx4<2>(sfc_tmem + 4, sf_desc_hi | ((smem_sfc + stage * Cfg::SFC_STAGE + 512) >> 4));
                        const uint32_t r_lo = r_lo0 + stage * (Cfg::R_STAGE >> 4), c_lo = c_lo0 + stage * (Cfg::C_STAGE >> 4);
#pragma unroll
                        for (uint32_t ks = 0; ks < 4; ++ks) {
                            const uint64_t r_desc = (static_cast<uint64_t>(op_hi) << 32) | (r_lo + ks * 2);
                            const uint64_t c_desc = (static_cast<uint64_t>(op_hi) << 32) | (c_lo + ks * 2);
                            umma_mxf8f6f4<2>(d_tmem, r_desc, c_desc, idesc_tile | (ks << 4) | (ks << 29), sfr_tmem, sfc_tmem,
                                             (kb | ks) != 0);
                        }
                        umma_commit<2>(&bars->empty[stage]);
                        if (kb + 1 == num_kb) umma_commit<2>(&bars->tmem_full[acc]);
                    }
                    __syncwarp();
                }
                ++acc_iter;
            }
        }
    } else if ((warp >= 4 && warp < 8) || warp >= 13) {
        // ============================================================ epilogue: two groups of four warps (4..7 and
        // 13..16; TMEM lane quadrant = warp % 4).  Group g drains the tiles that land in accumulator stage g, so a
        // group has two tile periods for one tile; with one group the UMMA issuer waited for the epilogue 17 % of
        // the time.  Each group owns one staging buffer, one per-token table and two barriers (buffer written /
        // buffer read).
        const uint32_t group = warp >= 13 ? 1u : 0u, q = warp % 4;
        const uint32_t tmem_empty_bar = map_to_cta(smem_u32(&bars->tmem_empty[0]), 0);
        const uint32_t overlap_bar = map_to_cta(smem_u32(&bars->overlap[0]), 0);
        uint64_t* bar_written = &s_epi_bar[group][0];
        uint64_t* bar_read = &s_epi_bar[group][1];
        uint8_t* stage_gen = smem_gen + (smem_cd - smem_base) + group * 32 * Cfg::PITCH;
        uint64_t* ttab = reinterpret_cast<uint64_t*>(smem_gen + (smem_cd - smem_base) + Cfg::TABLE_OFF) + group * 256;
        uint32_t chunks_done = 0;

        for (uint32_t slot = unit; slot < num_slots && ok; slot += num_units) {
            if (!fused_slot_to_tile(table, num_tiles, n1, n2, p.lag, slot, tc)) continue;
            const uint32_t acc = acc_iter & 1, acc_phase = (acc_iter >> 1) & 1;
            ++acc_iter;
            if (acc != group) continue;
            // Per-token data of the tile, fetched while its UMMAs run.  The reading threads themselves must have
            // seen the counters that say the pool rows (and, for the second GEMM, the routing metadata) are there.
            if (tc.kind == 0) {
                DG_FUSED_TIMED(7, ok = fused_wait_counter(pulled + tc.tile, tc.valid, abort_flag, p.a, 207, tc.tile));
            } else {
                DG_FUSED_TIMED(7, ok = fused_wait_counter(l1_done + tc.tile, n1 * 8, abort_flag, p.a, 208, tc.tile));
            }
            if (!ok) break;
            // The table's previous readers (this group's previous tile) are done: every warp of the group passed
            // that tile's last `bar_read` arrival before coming here, and the first chunk below waits for it.
            if (chunks_done > 0)
                DG_FUSED_TIMED(6, ok = wait_barrier(bar_read, (chunks_done - 1) & 1, abort_flag, peer_abort, wp, kSiteEpilogueSync, acc_iter, 0, 2));
            if (!ok) break;
            DG_EPI_TIMED(0,
            for (uint32_t tok = q * 32 + lane; tok < tc.rows; tok += 128) {
                const uint32_t row = tc.row0 + tok;
                if (tc.kind == 0) {
                    reinterpret_cast<float*>(ttab)[tok] = p.e.pool_w[row];
                } else {
                    const int32_t src_rank = p.e.pool_meta[row * 3];
                    uint64_t dst = 0;
                    if (src_rank >= 0) {
                        const uint64_t token = static_cast<uint32_t>(p.e.pool_meta[row * 3 + 1]);
                        const uint64_t sl = static_cast<uint32_t>(p.e.pool_meta[row * 3 + 2]);
                        dst = reinterpret_cast<uint64_t>(p.e.peer_base[src_rank]) + p.e.off_combine +
                              (sl * p.e.t_max + token) * p.e.hidden * 2;
                    }
                    ttab[tok] = dst;
                }
            }
            __syncwarp(););
            DG_FUSED_TIMED(5, ok = wait_barrier(&bars->tmem_full[acc], acc_phase, abort_flag, peer_abort, wp, kSiteEpilogueTmemFull, acc_iter, 0, acc));
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + acc * Cfg::kAccStride + ((q * 32) << 16);
            const uint32_t n0 = tc.n_blk * 256 + cta_rank * 128;
            const uint32_t num_chunks = (tc.rows + 31) / 32;
            const bool reverse = Cfg::kOverlap > 0 && acc == 0;   // stage 0 shares its last columns, stage 1 its first: drain those first
#pragma unroll 1
            for (uint32_t i = 0; i < num_chunks && ok; ++i) {
                const uint32_t ch = reverse ? num_chunks - 1 - i : i;
                uint32_t v[32];
                DG_EPI_TIMED(1, tmem_ld_32x32b_x32(t_acc + ch * 32, v); tmem_ld_wait(););
                if (i == 0 || i + 1 == num_chunks) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (Cfg::kOverlap > 0 && i == 0) mbar_arrive_cluster(overlap_bar + acc * 8);
                        if (i + 1 == num_chunks) mbar_arrive_cluster(tmem_empty_bar + acc * 8);
                    }
                }
                // the staging buffer's previous chunk has been read by all four warps (the tile's first chunk
                // already waited above)
                if (i > 0)
                    DG_FUSED_TIMED(6, ok = wait_barrier(bar_read, (chunks_done - 1) & 1, abort_flag, peer_abort, wp, kSiteEpilogueSync, acc_iter, ch, 2));
                if (!ok) break;
                DG_EPI_TIMED(2,
                _Pragma("unroll")
                for (uint32_t t = 0; t < 32; ++t)
                    *reinterpret_cast<__nv_bfloat16*>(stage_gen + t * Cfg::PITCH + (q * 32 + lane) * 2) =
                        __float2bfloat16_rn(__uint_as_float(v[t]));
                __syncwarp(););
                if (lane == 0) mbar_arrive(bar_written);
                DG_FUSED_TIMED(6, ok = wait_barrier(bar_written, chunks_done & 1, abort_flag, peer_abort, wp, kSiteEpilogueSync, acc_iter, ch, 3));
                if (!ok) break;
                const uint32_t chunk_rows = min(32u, tc.rows - ch * 32);
                if (tc.kind == 0)
                    DG_EPI_TIMED(3, moe_l1_chunk(p.e, stage_gen, Cfg::PITCH, reinterpret_cast<const float*>(ttab), q, lane, ch, chunk_rows, tc.row0, n0, tc.sf_base); __syncwarp(););
                else
                    DG_EPI_TIMED(4, moe_l2_chunk(stage_gen, Cfg::PITCH, ttab, q * 32 + lane, ch, chunk_rows, n0, p.e.post_down ? p.e.pool_w + tc.row0 : nullptr); __syncwarp(););
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_read);
                ++chunks_done;
            }
            if (!ok) break;
            if (tc.kind == 0) {
                // The tile's activations are read by TMA in other CTAs once all of its n-tiles have reported
                DG_EPI_TIMED(5,
                asm volatile("fence.proxy.async;" ::: "memory");
                __threadfence();
                __syncwarp();
                if (lane == 0) atomicAdd(l1_done + tc.tile, 1u););
            }
        }
        __threadfence_system();   // pushes to the source ranks are out before the final barriers
    } else if (ok) {
        // ============================================================ pull warps (2, 8..11): fill the pool in pool order
        const uint32_t pw = warp == 2 ? 0 : warp - 7;   // 0..4
        moe_pull_rows(p.a, s_prefix, blockIdx.x * 5 + pw, p.num_ctas * 5, lane, pulled, work + MoeFusedWork::expert_tab(L));
    }

    DG_FUSED_FLUSH();
    DG_FUSED_STAMP(2);
    // ---------------------------------------------------------------- combine: everyone has pushed, then reduce
    bool ok2 = fused_grid_barrier(ctrl, p.num_ctas, abort_flag, p.a, 205);
    DG_FUSED_STAMP0(4);
    if (ok2 && blockIdx.x == 0) {
        __shared__ uint32_t s_bar_ok;
        if (threadIdx.x == 0) s_bar_ok = 1;
        __syncthreads();
        if (threadIdx.x < L.ranks)
            if (!moe_cross_rank_barrier(p.a, 1, 2 * call_new, threadIdx.x)) s_bar_ok = 0;
        __syncthreads();
        DG_FUSED_STAMP0(5);
        if (threadIdx.x == 0 && s_bar_ok)
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ctrl + MoeCtrl::kCombineReady), "r"(call_new) : "memory");
    }
    if (ok2) {
        __shared__ uint32_t s_comb_ok;
        if (threadIdx.x == 0)
            s_comb_ok = fused_wait_counter(ctrl + MoeCtrl::kCombineReady, call_new, abort_flag, p.a, 206, call_new) ? 1u : 0u;
        __syncthreads();
        DG_FUSED_STAMP(3);
        if (s_comb_ok) {
            const uint32_t my_tokens = p.a.num_tokens > blockIdx.x ? (p.a.num_tokens - blockIdx.x + p.num_ctas - 1) / p.num_ctas : 0;
            if (L.topk <= 8) {
                fused_reduce_bulk(p, smem_gen, smem_base, abort_flag, wp);
            } else {
                // this CTA's tokens (blockIdx.x, + num_ctas, ...) as one flat list of 8-column items
                const uint32_t chunks = L.hidden / 8;
                for (uint32_t item = threadIdx.x; item < my_tokens * chunks; item += kFusedThreads) {
                    const uint32_t t = blockIdx.x + (item / chunks) * p.num_ctas, c = (item % chunks) * 8;
                    moe_reduce_cols<false>(p.a, p.y, p.ldy, t, c, c);
                }
            }
        }
    }

    DG_FUSED_STAMP(4);
    // ---------------------------------------------------------------- tear-down
    if (*abort_flag) {
        for (int i = 0; i < 20; ++i) __nanosleep(10000);
    }
    __syncwarp();
    tc_fence_before();
    cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<2>(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace dg
