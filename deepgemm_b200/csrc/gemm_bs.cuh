// Block-scaled FP8 / FP8xFP4 GEMM for sm_100a: one persistent, warp-specialised kernel.
//
//   D[m, n] = alpha * sum_k (A[m, k] * 2^ea[m, k / gran_a]) * (B[n, k] * 2^eb[n, k / gran_b])  (+ C)
//
// Replaces the reference's sm100_fp8_fp4_gemm_1d1d_impl
// (deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_gemm_1d1d.cuh:24-46) for all of its
// M-/K-grouped schedules.  The design is written in terms of the two UMMA operands:
//
//   R ("row" operand, UMMA A): 128 rows per CTA; rows become TMEM lanes.
//   C ("col" operand, UMMA B): BN rows per tile (split in halves across a CTA pair);
//                              rows become TMEM columns.
//
// kSwap = false: R = GEMM A (tokens), C = GEMM B (weights): the accumulator is a D tile.
// kSwap = true : R = GEMM B (weights), C = GEMM A (tokens): the accumulator is D^T, which
//                lets a CTA pair share one (possibly short) token block of any expert.
//
// Warp roles (288 threads):  0 TMA producer of the R tiles | 1 UMMA issuer (+TMEM owner) | 2 scale-factor
// transposer | 3 TMA producer of the scale factors | 4..7 epilogue (warp % 4 == TMEM lane quadrant) |
// 8 TMA producer of the C tiles | 9 second scale-factor transposer (kind::mxf4 only: 320 threads).
//
// Three UMMA kinds: kind::f16 for BF16 operands without scale factors (64 K elements per stage, UMMA K = 16), kind::mxf8f6f4 (E4M3 and unpacked E2M1 operands, 128 K elements per stage, UMMA K = 32) and, when
// both operands are packed E2M1, kind::mxf4 (256 K elements per stage in the same 128 bytes per row, UMMA K = 64,
// two scale words per row and stage: the 9 PFLOP/s path; sm100_fp8_fp4_gemm_1d1d.cuh:51-54 of the reference).
//
// Every wait is bounded: on expiry the waiting thread records where it gave up in the
// status block, raises the CTA's (and its pair's) abort flag, all roles leave their
// loops, outstanding copies are given time to land, TMEM is freed and the kernel returns.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace dg {

enum GemmType : uint32_t {
    kGemmNormal = 0,
    kGemmMContiguous = 1,   // grouped_layout: int32[M], expert id per row (-1 = padding)
    kGemmMMasked = 2,       // grouped_layout: int32[G], valid rows per group
    kGemmMPsum = 3,         // grouped_layout: int32[G], cumulative unaligned row ends
    kGemmKGrouped = 4,      // grouped_layout: int32[G], padded K per group
    kGemmKGroupedPsum = 5,  // grouped_layout: int32[G], cumulative unaligned K ends
    kGemmBatched = 6,       // num_groups independent m x n x k problems (no layout tensor)
};

// Epilogue kinds (GemmConfig::kEpi)
enum EpilogueKind : int {
    kEpiStore = 0,       // D = alpha * acc, or D += acc
    kEpiMoeL1 = 1,       // Mega MoE: gated activation + requantisation
    kEpiMoeL2 = 2,       // Mega MoE: BF16 rows pushed to the source ranks
    kEpiStochastic = 3,  // BF16 D with stochastic rounding (epilogue/operators.cuh:53-114 of the reference)
    kEpiFp8Cast = 4,     // E4M3 D with per-32 UE8M0 scales, optional clamp and clamp count (:116-220)
};

enum StatusCode : uint32_t {
    kStatusOk = 0,
    kStatusTimeout = 1,
};
enum WaitSite : uint32_t {
    kSiteProducerEmpty = 1,
    kSiteTransposerSfFull = 2,
    kSiteMmaTmemEmpty = 3,
    kSiteMmaFull = 4,
    kSiteEpilogueTmemFull = 5,
    kSiteMmaOverlap = 6,
    kSiteEpilogueSync = 7,
};

// One UMMA operand as the kernel sees it (all values computed on the host).

struct OperandParams {
    uint32_t mn_major;    // 0: K is the contiguous axis in global memory
    uint32_t num_boxes;   // TMA boxes per stage per CTA
    uint32_t box_bytes;   // shared-memory bytes per box
    uint32_t box_mn;      // rows (MN extent) covered by one box
    uint32_t tx_bytes;    // bytes one stage's boxes add to the barrier's transaction count
    uint32_t desc_lbo;    // UMMA descriptor: leading-dimension byte offset
    uint32_t desc_sbo;    // UMMA descriptor: stride-dimension byte offset
    uint32_t desc_kstep;  // descriptor start-address advance per UMMA_K (32 elements), bytes
    uint32_t gran_k;      // 32 or 128 K elements per scale
    uint32_t fmt;         // kFmtE4M3 / kFmtE2M1
    uint32_t batched;     // the tensor map's third coordinate is the tile's group (0: always 0)
};

// Arguments of the value epilogues (kEpiStochastic needs none; kEpiFp8Cast all).
struct CastEpilogueParams {
    uint32_t* sfd;            // packed UE8M0 words: scale of (row, column group g) in byte g % 4 of word
                              // sfd[(g / 4) * sfd_ld + row], g = (batch * n + column) / 32
    int64_t sfd_ld;
    float clamp_bound;        // BF16-rounded clamp value; +inf = no clamp
    uint32_t* clamped_count;  // optional: += elements whose BF16 magnitude exceeds the bound
};

// Arguments of the fused Mega MoE epilogues.
//   kEpi == 1 (first expert GEMM): BF16-round gate / up, gate * sigmoid(gate) * up * route weight,
//             per-32 UE8M0 E4M3 requantisation, written as the second GEMM's A operand.
//   kEpi == 2 (second expert GEMM): BF16 rows stored into the source rank's combine buffer.
struct MoeEpilogueParams {
    uint8_t* l2_acts;          // e4m3 [pool_rows, inter]
    uint8_t* l2_sf;            // UE8M0 bytes: word (kw, row) at (kw * pool_rows + row) * 4, byte k % 4
    const float* pool_w;       // route weight per pool row
    const int32_t* pool_meta;  // (source rank, token, slot) per pool row; rank < 0: no token
    uint8_t* peer_base[16];    // every rank's buffer base
    uint64_t off_combine;
    uint32_t pool_rows, inter, hidden, t_max;
    uint32_t sf_ld;            // row pitch of l2_sf
    float clamp;               // activation clamp; +inf = none
    uint32_t fast_math;
    uint32_t activation;       // 0 SwiGLU, 1 GeGLU (tanh form), 2 SiTU
    float situ_beta;           // SiTU: beta * tanh(gate / beta) * sigmoid(gate)
    float situ_linear_beta;    // SiTU: up -> lb * tanh(up / lb); +inf = up unchanged
    uint32_t post_down;        // route weight applied to the BF16 layer-2 row at the combine write instead of to the
                               // layer-2 input (impls/sm100_fp8_fp4_mega_moe.cuh:1538-1566 of the reference)
};

// Position of pool row `row` inside its 128-row group in the order tcgen05.cp.32x128b.warpx4 copies to TMEM.
__host__ __device__ inline uint32_t moe_sf_row(uint32_t row) {
    const uint32_t i = row & 127u;
    return (row & ~127u) + (i & 31u) * 4u + (i >> 5);
}

struct GemmParams {
    CUtensorMap tm_r, tm_c, tm_sfr, tm_sfc, tm_d;
    CUtensorMap tm_d_half;   // swapped tiles: D seen through boxes of 16 token rows, for a tile's last 16 rows
    // Swapped tiles with few token rows: the same C operand seen through boxes of 32 and 64 rows per CTA, so a
    // ragged last tile of an expert does not fetch 128 rows per CTA and K block (c_small != 0 when encoded)
    CUtensorMap tm_c_small[2];
    uint32_t c_small;
    OperandParams r, c;
    uint32_t gemm_type;
    uint32_t m, n, k;           // logical GEMM shape (per group where grouped)
    uint32_t num_groups;
    uint32_t alignment;         // M / K alignment of psum layouts
    const int32_t* grouped_layout;
    uint32_t num_m_blocks, num_n_blocks;   // of the (un-grouped) m x n tile grid
    uint32_t raster;            // tiles along the rasterised axis per super-row
    uint32_t num_units;         // CTAs (kCtas == 1) or CTA pairs (kCtas == 2) in the grid
    uint32_t sf_groups_r, sf_groups_c;     // packed-K words per group in the SF tensors (0: not grouped)
    float alpha;
    uint32_t accumulate;        // D += result (TMA reduce-add) instead of D = result
    uint32_t d_grouped;         // D has a group axis (masked / K-grouped): third store coordinate = group
    uint32_t split_blocks;      // contiguous layout: a schedule slot spans two alignment units (may straddle experts)
    uint32_t skip_padding;      // psum layout: compute a group's valid rows only (rounded up to 16), not its aligned extent
    // Dense layout, swapped tiles: the slots from tail_first on (the last, partly filled wave) are token tiles cut in
    // tail_split parts of UNIT_M / tail_split rows, so that more units share the wave (0 / 1: no cut)
    uint32_t tail_first, tail_split;
    uint32_t r_sf_pretransposed;  // R's scale words already sit in the 32x4 order tcgen05.cp reads (Mega MoE weights)
    uint32_t c_sf_pretransposed;  // same for C (Mega MoE activations: the pool is written in that order)
    MoeEpilogueParams moe;      // fused Mega MoE epilogues (GemmConfig::kEpi == 1, 2)
    CastEpilogueParams cast;    // kEpiFp8Cast
    uint32_t timeout_ms;
    uint32_t* status;           // 16 words: [0] code, [1] site, [2] block, [3] tile iter, [4] k block, [5] stage
    unsigned long long* trace;  // optional clock samples of block 0's first tile (builds with DG_TRACE only)
};

#ifdef DG_TRACE
#define DG_TRACE_AT(role, kb_)                                                                  \
    do {                                                                                        \
        if (p.trace != nullptr && blockIdx.x == 0 && (threadIdx.x & 31) == 0 && iter == 0 && (kb_) < 64)                   \
            p.trace[(role) * 64 + (kb_)] = static_cast<unsigned long long>(clock64());          \
    } while (0)
#else
#define DG_TRACE_AT(role, kb_) do { } while (0)
#endif

// One accumulator tile, in GEMM terms.
struct TileCoord {
    uint32_t row0;    // first GEMM-M row of the tile (inside its group for masked layouts)
    uint32_t rows;    // swapped tiles: token rows covered = UMMA N (multiple of 16); plain tiles: unused
    uint32_t n_blk, group;
    uint32_t k_start, k_len, sfk_base;
};

// Persistent tile walk shared by all roles: each role thread owns one instance and asks for the
// schedule slots unit, unit + num_units, ...  A slot yields one tile, or two where a token block
// of a contiguous layout straddles two experts (each half is then its own tile).
struct TileWalker {
    const GemmParams& p;
    const uint32_t bm, bn;   // GEMM-level extents of one schedule slot
    const bool swap;
    uint32_t group = 0;
    uint32_t m_blk_cum = 0;       // m-blocks of the groups before `group`
    uint32_t group_m_blocks = 0;  // m-blocks of `group`
    uint32_t group_rows = 0;      // rows of `group` to cover (masked: valid rows; psum: aligned extent)
    uint32_t row_start = 0;       // psum: first row of `group`
    uint32_t prev_end = 0;        // psum: unaligned end of the previous group
    uint32_t k_start = 0, k_len = 0, sfk_base = 0;
    bool primed = false;

    __device__ TileWalker(const GemmParams& p_, uint32_t bm_, uint32_t bn_, bool swap_)
        : p(p_), bm(bm_), bn(bn_), swap(swap_) {}

    __device__ int32_t layout(uint32_t i) const { return __ldg(p.grouped_layout + i); }
    __device__ static uint32_t align16(uint32_t x) { return (x + 15u) & ~15u; }

    __device__ void swizzle(uint32_t idx, uint32_t num_m, uint32_t num_n, uint32_t& m_blk, uint32_t& n_blk) const {
        // Super-rows of `raster` m-blocks; inside one, n varies slowest so that concurrently
        // running units share a small set of R and C rows in L2.
        const uint32_t per_super = p.raster * num_n;
        const uint32_t super = idx / per_super;
        const uint32_t first = super * p.raster;
        const uint32_t in_super = idx - super * per_super;
        const uint32_t rows = min(p.raster, num_m - first);
        m_blk = first + in_super % rows;
        n_blk = in_super / rows;
    }

    __device__ void load_group_m() {
        if (p.gemm_type == kGemmMMasked) {
            group_rows = static_cast<uint32_t>(layout(group));
        } else {  // psum: cover the group's whole aligned extent, so zero padding rows of A give zero rows of D
            const uint32_t end = static_cast<uint32_t>(layout(group));
            row_start = (prev_end + p.alignment - 1) / p.alignment * p.alignment;
            const uint32_t end_aligned = (end + p.alignment - 1) / p.alignment * p.alignment;
            group_rows = end > row_start ? (p.skip_padding ? end : end_aligned) - row_start : 0;
            prev_end = end;
        }
        group_m_blocks = (group_rows + bm - 1) / bm;
    }
    __device__ void load_group_k() {
        if (p.gemm_type == kGemmKGroupedPsum) {
            const uint32_t end = static_cast<uint32_t>(layout(group));
            k_start = (prev_end + p.alignment - 1) / p.alignment * p.alignment;
            k_len = end - k_start;
            prev_end = end;
        } else {
            k_len = static_cast<uint32_t>(layout(group));
        }
    }

    // Fills tc[0..return) for schedule slot t; 0 means the walk is over.
    __device__ uint32_t next(uint32_t t, TileCoord* tc) {
        TileCoord& c = tc[0];
        c.k_start = 0, c.k_len = p.k, c.sfk_base = 0, c.group = 0, c.rows = bm;
        const uint32_t num_n = p.num_n_blocks;
        uint32_t m_blk;
        if (p.gemm_type == kGemmBatched) {
            // every batch owns a full m x n tile grid
            const uint32_t per_group = p.num_m_blocks * num_n;
            if (t >= per_group * p.num_groups) return 0;
            const uint32_t g = t / per_group;
            swizzle(t - g * per_group, p.num_m_blocks, num_n, m_blk, c.n_blk);
            c.row0 = m_blk * bm, c.group = g;
            if (swap) c.rows = min(bm, align16(p.m - c.row0));
            return 1;
        }
        if (p.gemm_type == kGemmNormal && p.tail_split > 1 && t >= p.tail_first) {
            const uint32_t sub = t - p.tail_first, idx = p.tail_first + sub / p.tail_split;
            if (idx >= p.num_m_blocks * num_n) return 0;
            swizzle(idx, p.num_m_blocks, num_n, m_blk, c.n_blk);
            const uint32_t part_rows = bm / p.tail_split;
            c.row0 = m_blk * bm + (sub % p.tail_split) * part_rows;   // m is a multiple of bm: every part is full
            c.rows = part_rows;
            return 1;
        }
        if (p.gemm_type == kGemmNormal || p.gemm_type == kGemmMContiguous) {
            if (t >= p.num_m_blocks * num_n) return 0;
            swizzle(t, p.num_m_blocks, num_n, m_blk, c.n_blk);
            c.row0 = m_blk * bm;
            if (swap) c.rows = min(bm, align16(p.m - c.row0));
            if (p.gemm_type == kGemmNormal) return 1;
            const int32_t g0 = layout(c.row0);
            c.group = g0 < 0 ? 0u : static_cast<uint32_t>(g0);
            if (!p.split_blocks) return 1;
            // The slot spans two alignment units: one tile if they belong to one expert, else two
            const uint32_t half = bm / 2, row1 = c.row0 + half;
            if (row1 >= p.m) {
                c.rows = half;
                return 1;
            }
            const int32_t g1 = layout(row1);
            if (g1 < 0 || g1 == g0) return 1;          // same expert, or the second unit is pure padding
            if (g0 < 0) {                              // first unit is pure padding: use the second's expert
                c.group = static_cast<uint32_t>(g1);
                return 1;
            }
            tc[1] = c;
            c.rows = half;
            tc[1].row0 = row1, tc[1].rows = min(half, align16(p.m - row1)), tc[1].group = static_cast<uint32_t>(g1);
            return 2;
        }
        if (p.gemm_type == kGemmMMasked || p.gemm_type == kGemmMPsum) {
            if (!primed) {
                primed = true;
                load_group_m();
            }
            while (t >= (m_blk_cum + group_m_blocks) * num_n) {
                if (++group >= p.num_groups) return 0;
                m_blk_cum += group_m_blocks;
                load_group_m();
            }
            swizzle(t - m_blk_cum * num_n, group_m_blocks, num_n, m_blk, c.n_blk);
            const uint32_t in_group = m_blk * bm;
            c.row0 = in_group + (p.gemm_type == kGemmMPsum ? row_start : 0);
            if (swap) c.rows = min(bm, align16(group_rows - in_group));
            c.group = group;
            return 1;
        }
        // K-grouped: every group owns a full m x n tile grid and its own K range.
        const uint32_t per_group = p.num_m_blocks * num_n;
        if (!primed) {
            primed = true;
            load_group_k();
        }
        while (t >= (group + 1) * per_group) {
            if (++group >= p.num_groups) return 0;
            const uint32_t aligned = (k_len + p.alignment - 1) / p.alignment * p.alignment;
            sfk_base += (aligned + p.r.gran_k * 4 - 1) / (p.r.gran_k * 4);
            if (p.gemm_type == kGemmKGrouped) k_start += k_len;
            load_group_k();
        }
        if (group >= p.num_groups) return 0;
        swizzle(t - group * per_group, p.num_m_blocks, num_n, m_blk, c.n_blk);
        c.row0 = m_blk * bm;
        c.group = group, c.k_start = k_start, c.k_len = k_len, c.sfk_base = sfk_base;
        return 1;
    }
};

// kKind_: which tcgen05.mma kind the operands take
enum : int { kKindMxf8f6f4 = 0, kKindMxf4 = 1, kKindBf16 = 2 };
template <int kCtas_, int BN_, bool kSwap_, bool kCdF32_, int kEpi_ = 0, int kKind_ = kKindMxf8f6f4>
struct GemmConfig {
    static constexpr int kEpi = kEpi_;   // EpilogueKind
    static constexpr bool kMoeEpi = kEpi_ == kEpiMoeL1 || kEpi_ == kEpiMoeL2;
    static_assert(!kMoeEpi || kSwap_, "the fused Mega MoE epilogues work on D^T tiles");
    static_assert(!(kEpi_ == kEpiStochastic || kEpi_ == kEpiFp8Cast) || (!kSwap_ && !kCdF32_),
                  "the value epilogues work on D tiles with 16-bit or 8-bit output");
    static constexpr bool kMxf4 = kKind_ == kKindMxf4;   // both operands packed E2M1: kind::mxf4, 256 K elements per stage
    static constexpr bool kBf16 = kKind_ == kKindBf16;   // BF16 operands without scale factors: kind::f16, 64 K elements per stage
    static_assert(!(kBf16 && (kEpi_ == kEpiMoeL1 || kEpi_ == kEpiMoeL2 || kEpi_ == kEpiFp8Cast)), "BF16 operands: store and stochastic epilogues");
    static constexpr int kCtas = kCtas_;
    static constexpr int BN = BN_;
    static constexpr bool kSwap = kSwap_;
    static constexpr bool kCdF32 = kCdF32_;
    static_assert(!(kSwap && kCdF32), "the transposed epilogue writes BF16 only");
    static_assert(BN % 16 == 0 && BN >= 32 && BN <= 256, "UMMA N");

    // warps 0-3: R copies, UMMA, scale transposer, scale copies; 4-7: epilogue; 8: C copies; 9 (kind::mxf4 only): a second
    // scale transposer - with one scale per 32 K elements on both sides every K block brings six 128-row scale blocks
    static constexpr uint32_t kTransposers = kMxf4 ? 2 : 1;
    static constexpr uint32_t kThreads = 288 + 32 * (kTransposers - 1);
    static constexpr uint32_t BLOCK_K = 128;          // bytes of K per row and stage
    static constexpr uint32_t BLOCK_K_ELEMS = kMxf4 ? 256 : kBf16 ? 64 : 128;
    static constexpr uint32_t SF_WORDS = kMxf4 ? 2 : kBf16 ? 0 : 1;   // packed scale words (128 K elements each) per row and stage
    static constexpr uint32_t R_ROWS = 128;
    static constexpr uint32_t C_ROWS_PER_CTA = BN / kCtas;
    static constexpr uint32_t R_STAGE = R_ROWS * BLOCK_K;
    static constexpr uint32_t C_STAGE = C_ROWS_PER_CTA * BLOCK_K;
    static constexpr uint32_t SFC_ROWS = (BN + 127) / 128 * 128;
    static constexpr uint32_t SFR_STAGE = 128 * 4 * SF_WORDS;
    static constexpr uint32_t SFC_STAGE = SFC_ROWS * 4 * SF_WORDS;
    static constexpr uint32_t STAGE_BYTES = R_STAGE + C_STAGE + SFR_STAGE + SFC_STAGE;

    // Epilogue staging: each epilogue warp owns one slab per buffer and stores it by itself.
    //   D tile:   32 rows x 128 B (64 BF16 or 32 FP32 columns), 128 B swizzle
    //   D^T tile: 32 tokens x 32 BF16 (64 B rows), no swizzle
    //   E4M3 D tile (kEpiFp8Cast): 32 rows x 64 B, no swizzle
    static constexpr uint32_t CHUNK_COLS = kSwap ? 32 : (kCdF32 ? 32 : 64);
    static constexpr uint32_t SLAB_BYTES = (kSwap || kEpi == kEpiFp8Cast) ? 32 * 64 : 32 * 128;
    static constexpr uint32_t kStoreBufs = (kCtas == 1 && BN == 256) ? 1 : 2;
    // Fused epilogues stage 32 tokens x 128 rows of BF16 per buffer (row pitch padded for kEpi == 1)
    static constexpr uint32_t MOE_PITCH = kEpi == 1 ? 272 : 256;
    static constexpr uint32_t CD_BYTES = !kMoeEpi ? kStoreBufs * 4 * SLAB_BYTES
                                                  : (2 * 32 * MOE_PITCH + 2 * 256 * 8 + 1023) / 1024 * 1024;
    static constexpr uint32_t MOE_TABLE_OFF = 2 * 32 * MOE_PITCH;   // per-tile token tables, two copies

    static constexpr uint32_t kSmemLimit = 232448;
    static constexpr uint32_t kBarrierBytes = 1024;
    static constexpr uint32_t kStagesRaw = (kSmemLimit - 1024 - CD_BYTES - kBarrierBytes) / STAGE_BYTES;
    static constexpr uint32_t kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
    static_assert(kStages >= 3, "pipeline too shallow");
    static constexpr uint32_t kSmemBytes = 1024 + kStages * STAGE_BYTES + CD_BYTES + kBarrierBytes;

    // TMEM columns: two accumulator stages, then the scale factors of R (4) and C (BN / 32, >= 4).
    // When 2 BN + scale columns exceed the 512 columns of TMEM the two stages overlap in
    // kOverlap columns: the last columns of stage 0 are the first columns of stage 1.  The epilogue
    // drains the shared columns first (stage 0 back to front, stage 1 front to back) and tells the
    // UMMA issuer, which only then lets the next tile write them.
    static constexpr uint32_t SFR_COLS = 4 * SF_WORDS;
    static constexpr uint32_t SFC_COLS_PER_WORD = SFC_ROWS / 32;
    static constexpr uint32_t SFC_COLS = SFC_COLS_PER_WORD * SF_WORDS;
    static constexpr uint32_t kOverlap = (2 * BN + SFR_COLS + SFC_COLS > 512) ? (2 * BN + SFR_COLS + SFC_COLS - 512 + 15) / 16 * 16 : 0;
    static_assert(kOverlap <= CHUNK_COLS, "the shared columns must lie in one epilogue chunk");
    static constexpr uint32_t kAccStride = BN - kOverlap;
    static constexpr uint32_t kSfrCol = 2 * BN - kOverlap;
    static constexpr uint32_t kSfcCol = kSfrCol + SFR_COLS;
    static constexpr uint32_t kUsedCols = kSfcCol + SFC_COLS;
    static constexpr uint32_t kTmemCols = kUsedCols <= 32 ? 32 : kUsedCols <= 64 ? 64 : kUsedCols <= 128 ? 128
                                          : kUsedCols <= 256 ? 256 : 512;
    static_assert(kUsedCols <= 512, "TMEM overflow");

    // GEMM-level extents of one schedule slot (CTA or CTA pair).
    static constexpr uint32_t UNIT_M = kSwap ? BN : 128 * kCtas;
    static constexpr uint32_t UNIT_N = kSwap ? 128 * kCtas : BN;
};

struct alignas(8) GemmBarriers {
    uint64_t full[10];
    uint64_t empty[10];
    uint64_t sf_full[10];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t overlap[2];
    uint64_t epi_sync[2];   // fused epilogues: the four epilogue warps meet here once per chunk
    uint32_t tmem_base;
    uint32_t abort;
};
static_assert(sizeof(GemmBarriers) <= 1024, "barrier block");

static __device__ __noinline__ void report_timeout(const GemmParams& p, uint32_t site, uint32_t iter, uint32_t kb,
                                            uint32_t stage) {
    if (atomicCAS(p.status, kStatusOk, kStatusTimeout) == kStatusOk) {
        p.status[1] = site;
        p.status[2] = blockIdx.x;
        p.status[3] = iter;
        p.status[4] = kb;
        p.status[5] = stage;
        __threadfence_system();
    }
}

// Bounded mbarrier wait.  Returns false if the CTA is aborting or the budget ran out.
DG_DEVICE bool wait_barrier(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t peer_abort_addr,
                            const GemmParams& p, uint32_t site, uint32_t iter, uint32_t kb, uint32_t stage) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    const uint64_t budget = static_cast<uint64_t>(p.timeout_ms) * 1000000ull;
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 15u) == 0) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > budget) {
                report_timeout(p, site, iter, kb, stage);
                *abort_flag = 1;
                if (peer_abort_addr) st_cluster_u32(peer_abort_addr, 1);
                return false;
            }
        }
    }
}

// One 32-token chunk of the first expert GEMM's epilogue, after the chunk was staged as BF16 [token][128 rows]:
// SwiGLU on the BF16-rounded gate / up pairs, times the route weight, per-32 UE8M0 E4M3 requantisation, stored
// as rows of the second GEMM's A operand.  m0: first pool row of the tile; n0: first interleaved weight row of
// this CTA; wtab: the tile's route weights.
// tanh by the approximate unit (fast math) or the library routine
template <bool kFast>
DG_DEVICE float moe_tanh(float x) {
    if (kFast) {
        float y;
        asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
        return y;
    }
    return tanhf(x);
}

// gate -> the gated factor that multiplies `up` (deep_gemm tests/test_mega_moe.py:451-463 states the three forms)
template <bool kFast, int kAct>
DG_DEVICE float moe_gate(float g, float beta) {
    const float sig = kFast ? __fdividef(1.0f, 1.0f + __expf(-g)) : 1.0f / (1.0f + expf(-g));
    if (kAct == 0) return g * sig;
    if (kAct == 1) return 0.5f * g * (1.0f + moe_tanh<kFast>(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    return beta * moe_tanh<kFast>(kFast ? __fdividef(g, beta) : g / beta) * sig;
}

template <bool kFast, bool kClamp, int kAct>
DG_DEVICE void moe_l1_chunk_impl(const MoeEpilogueParams& m, const uint8_t* stage, uint32_t pitch, const float* wtab,
                                 uint32_t q, uint32_t lane, uint32_t ch, uint32_t chunk_rows, uint32_t m0, uint32_t n0,
                                 uint32_t sf_base) {
    // A warp takes 8 tokens; lane = (token, 32-output group g, half): 16 outputs per
    // thread = 32 interleaved rows laid out as 2 x [8 gate | 8 up] (the weights come
    // interleaved in blocks of 8 rows); the two halves of a group share their amax.
    const uint32_t t = q * 8 + (lane >> 2), g = (lane >> 1) & 1, half = lane & 1;
    const float w = m.post_down ? 1.0f : wtab[min(ch * 32 + t, 255u)];
    const float clamp = m.clamp, beta = m.situ_beta, lin_beta = m.situ_linear_beta;
    const bool squash_up = lin_beta < 3.0e38f;
    (void)beta, (void)squash_up;
    const uint4* src = reinterpret_cast<const uint4*>(stage + t * pitch + g * 128 + half * 64);
    const uint4 raw[4] = {src[0], src[1], src[2], src[3]};   // [8 gate | 8 up] x 2, BF16
    float act[16];
    float amax = 0.f;
#pragma unroll
    for (uint32_t blk = 0; blk < 2; ++blk) {
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&raw[2 * blk]);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&raw[2 * blk + 1]);
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            float2 gf = __bfloat1622float2(g2[j]), uf = __bfloat1622float2(u2[j]);
            if (kClamp) {
                gf.x = fminf(gf.x, clamp), gf.y = fminf(gf.y, clamp);
                uf.x = fminf(fmaxf(uf.x, -clamp), clamp);
                uf.y = fminf(fmaxf(uf.y, -clamp), clamp);
            }
            const float sx = moe_gate<kFast, kAct>(gf.x, beta), sy = moe_gate<kFast, kAct>(gf.y, beta);
            if (kAct == 2 && squash_up) {
                uf.x = lin_beta * moe_tanh<kFast>(kFast ? __fdividef(uf.x, lin_beta) : uf.x / lin_beta);
                uf.y = lin_beta * moe_tanh<kFast>(kFast ? __fdividef(uf.y, lin_beta) : uf.y / lin_beta);
            }
            const float ax = (sx * uf.x) * w, ay = (sy * uf.y) * w;
            act[blk * 8 + j * 2] = ax, act[blk * 8 + j * 2 + 1] = ay;
            amax = fmaxf(amax, fmaxf(fabsf(ax), fabsf(ay)));
        }
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    // Power-of-two scale 2^e >= amax / 448, floor 2^-22 (amax clamp 1e-4): the add
    // carries into the exponent iff the mantissa exceeds that of 448 = 1.75 * 2^8
    uint32_t e = (__float_as_uint(amax) + 0x1FFFFFu) >> 23;
    e = max(e, 113u) - 8u;
    const float inv = __uint_as_float((254u - e) << 23);
    uint32_t packed[4];
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j) {
        const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
            make_float2(act[4 * j] * inv, act[4 * j + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
            make_float2(act[4 * j + 2] * inv, act[4 * j + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        packed[j] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
    }
    if (t < chunk_rows) {
        const uint32_t row = m0 + ch * 32 + t;
        const uint32_t inter0 = n0 / 2 + g * 32;   // n0: first interleaved row of this CTA
        *reinterpret_cast<uint4*>(m.l2_acts + static_cast<uint64_t>(row) * m.inter + inter0 +
                                  half * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        const uint32_t kgroup = inter0 / 32;
        if (half == 0)
            // scale rows in tcgen05.cp order relative to the tile: sf_base is the tile's first scale row
            m.l2_sf[(static_cast<uint64_t>(kgroup / 4) * m.sf_ld + sf_base + moe_sf_row(ch * 32 + t)) * 4 + (kgroup & 3)] =
                static_cast<uint8_t>(e);
    }
}

template <int kAct>
DG_DEVICE void moe_l1_chunk_act(const MoeEpilogueParams& m, const uint8_t* stage, uint32_t pitch, const float* wtab,
                                uint32_t q, uint32_t lane, uint32_t ch, uint32_t chunk_rows, uint32_t m0, uint32_t n0,
                                uint32_t sf_base) {
    const bool clamp = m.clamp < 3.0e38f;   // +inf: no clamp
    if (m.fast_math) {
        if (clamp) moe_l1_chunk_impl<true, true, kAct>(m, stage, pitch, wtab, q, lane, ch, chunk_rows, m0, n0, sf_base);
        else       moe_l1_chunk_impl<true, false, kAct>(m, stage, pitch, wtab, q, lane, ch, chunk_rows, m0, n0, sf_base);
    } else {
        if (clamp) moe_l1_chunk_impl<false, true, kAct>(m, stage, pitch, wtab, q, lane, ch, chunk_rows, m0, n0, sf_base);
        else       moe_l1_chunk_impl<false, false, kAct>(m, stage, pitch, wtab, q, lane, ch, chunk_rows, m0, n0, sf_base);
    }
}

// sf_base: first scale row of the tile in l2_sf (the tile's first pool row where tiles start on 128-row boundaries)
DG_DEVICE void moe_l1_chunk(const MoeEpilogueParams& m, const uint8_t* stage, uint32_t pitch, const float* wtab,
                            uint32_t q, uint32_t lane, uint32_t ch, uint32_t chunk_rows, uint32_t m0, uint32_t n0,
                            uint32_t sf_base) {
    if (m.activation == 0)      moe_l1_chunk_act<0>(m, stage, pitch, wtab, q, lane, ch, chunk_rows, m0, n0, sf_base);
    else if (m.activation == 1) moe_l1_chunk_act<1>(m, stage, pitch, wtab, q, lane, ch, chunk_rows, m0, n0, sf_base);
    else                        moe_l1_chunk_act<2>(m, stage, pitch, wtab, q, lane, ch, chunk_rows, m0, n0, sf_base);
}

// One 32-token chunk of the second expert GEMM's epilogue: 16 lanes move one token's 256 B segment of BF16
// results to that token's slot plane in its source rank's buffer (dtab: per-token destination row address, 0 = none).
DG_DEVICE void moe_l2_chunk(const uint8_t* stage, uint32_t pitch, const uint64_t* dtab, uint32_t et, uint32_t ch,
                            uint32_t chunk_rows, uint32_t n0, const float* row_w) {
    // 32 tokens x 256 B: 16 lanes move one token's 256 B segment to its source rank.  row_w (post-down route
    // weights, one per pool row of the tile, or nullptr): every BF16 value is multiplied by its row's weight and
    // rounded to BF16 again.
#pragma unroll
    for (uint32_t i = 0; i < 4; ++i) {
        const uint32_t piece = i * 128 + et, t = piece >> 4, part = piece & 15;
        const uint64_t base = t < chunk_rows ? dtab[ch * 32 + t] : 0;
        if (base != 0) {
            uint4 val = *reinterpret_cast<const uint4*>(stage + t * pitch + part * 16);
            if (row_w != nullptr) {
                const float w = row_w[ch * 32 + t];
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&val);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h[j]);
                    h[j] = __floats2bfloat162_rn(f.x * w, f.y * w);
                }
            }
            *reinterpret_cast<uint4*>(base + static_cast<uint64_t>(n0) * 2 + part * 16) = val;
        }
    }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::kThreads, 1) gemm_bs_kernel(const __grid_constant__ GemmParams p) {
    constexpr int kCtas = Cfg::kCtas;
    constexpr uint32_t BN = Cfg::BN;
    constexpr uint32_t kStages = Cfg::kStages;
    constexpr bool kPair = kCtas == 2;
    constexpr bool kSwap = Cfg::kSwap;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // Carve-up: R stages | C stages | CD slabs (all 1024 B aligned: they are swizzled) | SFR | SFC | barriers
    const uint32_t smem_r = smem_base;
    const uint32_t smem_c = smem_r + kStages * Cfg::R_STAGE;
    const uint32_t smem_cd = smem_c + kStages * Cfg::C_STAGE;
    const uint32_t smem_sfr = smem_cd + Cfg::CD_BYTES;
    const uint32_t smem_sfc = smem_sfr + kStages * Cfg::SFR_STAGE;
    GemmBarriers* bars =
        reinterpret_cast<GemmBarriers*>(smem_gen + (smem_sfc + kStages * Cfg::SFC_STAGE - smem_base));
    uint32_t* sf_words_r = reinterpret_cast<uint32_t*>(smem_gen + (smem_sfr - smem_base));
    uint32_t* sf_words_c = reinterpret_cast<uint32_t*>(smem_gen + (smem_sfc - smem_base));

    const uint32_t warp = threadIdx.x / 32;
    const uint32_t lane = threadIdx.x % 32;
    const uint32_t cta_rank = kPair ? cluster_ctarank() : 0;
    const bool is_leader = cta_rank == 0;
    const uint32_t unit = kPair ? blockIdx.x / 2 : blockIdx.x;
    volatile uint32_t* abort_flag = &bars->abort;
    const uint32_t peer_abort = kPair ? map_to_cta(smem_u32(&bars->abort), cta_rank ^ 1) : 0;

    // ---------------------------------------------------------------- set-up
    if (warp == 0 && lane == 0) {
        prefetch_tmap(&p.tm_r);
        prefetch_tmap(&p.tm_c);
        prefetch_tmap(&p.tm_sfr);
        prefetch_tmap(&p.tm_sfc);
        prefetch_tmap(&p.tm_d);
        for (uint32_t i = 0; i < kStages; ++i) {
            mbar_init(&bars->full[i], kCtas * (Cfg::kBf16 ? 2 : 2 + Cfg::kTransposers));   // per CTA: R producer, C producer, scale transposer(s)
            mbar_init(&bars->empty[i], 1);          // UMMA commit
            mbar_init(&bars->sf_full[i], 1);        // producer (SF copies land here)
        }
        for (uint32_t i = 0; i < 2; ++i) {
            mbar_init(&bars->tmem_full[i], 1);            // UMMA commit
            mbar_init(&bars->tmem_empty[i], kCtas * 4);   // one lane per epilogue warp
            mbar_init(&bars->overlap[i], kCtas * 4);
            mbar_init(&bars->epi_sync[i], 4);
        }
        bars->abort = 0;
        fence_mbar_init();
    }
    if (kPair) cluster_sync();   // both CTAs exist before the paired TMEM allocation
    if (warp == 1) {
        tmem_alloc<kCtas>(&bars->tmem_base, Cfg::kTmemCols);
        tmem_relinquish<kCtas>();
    }
    tc_fence_before();
    if (kPair) cluster_sync(); else __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    // Everything above touched this CTA's own state only.  From here on global memory is read that an earlier kernel of
    // the stream may have written (packed scales, a producer's activations): with programmatic dependent launch this
    // is where that kernel's completion is awaited; the next kernel of the stream may start its own set-up already.
    grid_dependency_wait();
    grid_launch_dependents();

    // Barrier addresses in the leader CTA (own CTA when not paired)
    auto leader_addr = [&](uint64_t* bar) -> uint32_t {
        return kPair ? map_to_cta(smem_u32(bar), 0) : smem_u32(bar);
    };

    // K-blocks covered by one packed scale word: 4 (one scale per 128 K) or 1 (one per 32 K)
    const uint32_t sf_mask_r = p.r.gran_k == 128 ? 3 : 0, sf_shift_r = p.r.gran_k == 128 ? 2 : 0;
    const uint32_t sf_mask_c = p.c.gran_k == 128 ? 3 : 0, sf_shift_c = p.c.gran_k == 128 ? 2 : 0;

    // Shared by the role loops: smem stage / phase bookkeeping and the schedule walk.
    uint32_t stage = 0, phase = 0;
    auto advance = [&]() {
        stage = stage + 1 == kStages ? 0 : stage + 1;
        phase ^= (stage == 0);
    };
    TileWalker walker(p, Cfg::UNIT_M, Cfg::UNIT_N, kSwap);
    TileCoord tiles[2];
    // Schedule slots of this unit: unit, unit + num_units, ... (the walker says when they are used up)
    bool ok = true;
    uint32_t acc_iter = 0;   // accumulator tiles handled so far by this role

    if (warp == 0 || warp == 3 || warp == 8) {
        // ============================================================ TMA producers
        // Warp 0 fetches the R tiles, warp 8 the C tiles, warp 3 the scale factors: one thread needs some 150-200
        // cycles to issue a copy, so a K block's copies (up to four) are spread over three issuing threads.  The
        // whole warp runs the loop (uniform control flow keeps addresses and coordinates in uniform registers); one
        // elected lane issues the copies.
        const bool sf_role = warp == 3, r_role = warp == 0;
        if (Cfg::kBf16 && sf_role) ok = false;   // no scale factors: this warp has nothing to fetch
        const uint32_t full_bar0 = leader_addr(&bars->full[0]);
        const uint32_t stage_tx_bytes = p.r.tx_bytes + p.c.tx_bytes;
        const uint32_t r_boxes = p.r.num_boxes, r_box_bytes = p.r.box_bytes, r_box_mn = p.r.box_mn;
        const uint32_t c_boxes = p.c.num_boxes, c_box_bytes = p.c.box_bytes, c_box_mn = p.c.box_mn;
        const bool r_mn_major = p.r.mn_major != 0, c_mn_major = p.c.mn_major != 0;
        const uint32_t sfg_a = kSwap ? p.sf_groups_c : p.sf_groups_r;
        const uint32_t sfg_b = kSwap ? p.sf_groups_r : p.sf_groups_c;
        const bool r_batched = p.r.batched != 0, c_batched = p.c.batched != 0;
        for (uint32_t iter = 0; ok; ++iter) {
            const uint32_t slot = unit + iter * p.num_units;
            const uint32_t num_sub = walker.next(slot, tiles);
            if (num_sub == 0) break;
            for (uint32_t sub = 0; sub < num_sub && ok; ++sub, ++acc_iter) {
                const TileCoord& tc = tiles[sub];
                // Operand coordinates of this tile (GEMM A / B, then mapped to R / C)
                // Data: (K, row inside the group, group) through 3-D tensor maps; the K coordinate counts the map's
                // elements (bytes for E4M3 and for packed E2M1 under kind::mxf4)
                const uint32_t a_mn = tc.row0, b_mn = tc.n_blk * Cfg::UNIT_N;
                // (BF16 operands go through byte maps: the contiguous axis counts two bytes per element)
                const uint32_t k0 = Cfg::kMxf4 ? tc.k_start >> 1 : tc.k_start;
                const uint32_t r_esz = (Cfg::kBf16 && r_mn_major) ? 2u : 1u, c_esz = (Cfg::kBf16 && c_mn_major) ? 2u : 1u;
                const uint32_t r_kstep = (Cfg::kBf16 && r_mn_major) ? 64u : 128u, c_kstep = (Cfg::kBf16 && c_mn_major) ? 64u : 128u;
                const int32_t r_batch = r_batched ? static_cast<int32_t>(tc.group) : 0;
                const int32_t c_batch = c_batched ? static_cast<int32_t>(tc.group) : 0;
                const uint32_t sfa_k = tc.sfk_base + tc.group * sfg_a, sfb_k = tc.sfk_base + tc.group * sfg_b;
                // SF rows are addressed inside the group (the group offset is on the packed-K axis)
                const uint32_t sfa_mn = tc.row0, sfb_mn = tc.n_blk * Cfg::UNIT_N;
                uint32_t r_mn = kSwap ? b_mn : a_mn, c_mn = kSwap ? a_mn : b_mn;
                const uint32_t r_k = (Cfg::kBf16 && !r_mn_major) ? k0 * 2 : k0, c_k = (Cfg::kBf16 && !c_mn_major) ? k0 * 2 : k0;
                uint32_t sfr_mn = kSwap ? sfb_mn : sfa_mn;
                const uint32_t sfc_mn = kSwap ? sfa_mn : sfb_mn;
                const uint32_t sfr_k = kSwap ? sfb_k : sfa_k, sfc_k = kSwap ? sfa_k : sfb_k;
                // This CTA's share: its own 128 R rows and its half of the C rows the UMMA reads
                r_mn += cta_rank * 128, sfr_mn += cta_rank * 128;
                c_mn += cta_rank * ((kSwap ? tc.rows : BN) / kCtas);

                const CUtensorMap* tm_c_tile = &p.tm_c;
                uint32_t tile_tx_bytes = stage_tx_bytes;
                if constexpr (kSwap) {
                    if (p.c_small != 0) {
                        const uint32_t per_cta = tc.rows / kCtas;
                        if (per_cta <= 32) tm_c_tile = &p.tm_c_small[0], tile_tx_bytes = p.r.tx_bytes + 32 * 128;
                        else if (per_cta <= 64) tm_c_tile = &p.tm_c_small[1], tile_tx_bytes = p.r.tx_bytes + 64 * 128;
                    }
                }
                const uint32_t num_kb = max(1u, (tc.k_len + Cfg::BLOCK_K_ELEMS - 1) / Cfg::BLOCK_K_ELEMS);
                for (uint32_t kb = 0; kb < num_kb; ++kb, advance()) {
                    DG_TRACE_AT(0, kb);
                    ok = wait_barrier(&bars->empty[stage], phase ^ 1, abort_flag, peer_abort, p, kSiteProducerEmpty,
                                      acc_iter, kb, stage);
                    if (!ok) break;
                    DG_TRACE_AT(1, kb);
                    if (sf_role) {
                      if (elect_one()) {
                        uint32_t sf_bytes = 0;
                        const uint32_t sf_bar = smem_u32(&bars->sf_full[stage]);
                        if ((kb & sf_mask_r) == 0) {
                            tma_load_2d<false>(smem_sfr + stage * Cfg::SFR_STAGE, &p.tm_sfr, sf_bar,
                                               static_cast<int32_t>(sfr_mn),
                                               static_cast<int32_t>(sfr_k + (Cfg::kMxf4 ? kb * 2 : kb >> sf_shift_r)));
                            sf_bytes += Cfg::SFR_STAGE;
                        }
                        if ((kb & sf_mask_c) == 0) {
                            tma_load_2d<false>(smem_sfc + stage * Cfg::SFC_STAGE, &p.tm_sfc, sf_bar,
                                               static_cast<int32_t>(sfc_mn),
                                               static_cast<int32_t>(sfc_k + (Cfg::kMxf4 ? kb * 2 : kb >> sf_shift_c)));
                            sf_bytes += Cfg::SFC_STAGE;
                        }
                        mbar_arrive_expect_tx(&bars->sf_full[stage], sf_bytes);
                      }
                    } else if (r_role) {
                      if (elect_one()) {
                        // Operand tiles land on the leader's barrier (both CTAs of a pair feed one UMMA)
                        const uint32_t full_bar = full_bar0 + stage * 8;
                        mbar_arrive_expect_tx_cluster(full_bar, p.r.tx_bytes);
                        const uint32_t kr = r_k + kb * r_kstep;
                        for (uint32_t b = 0; b < r_boxes; ++b) {
                            const uint32_t dst = smem_r + stage * Cfg::R_STAGE + b * r_box_bytes;
                            const uint32_t mn = (r_mn + b * r_box_mn) * r_esz;
                            // Swapped tiles: R holds the weights, which every token block of the group reads again:
                            // they are the last to leave L2
                            if (r_mn_major) tma_load_3d<kPair>(dst, &p.tm_r, full_bar, mn, kr, r_batch);
                            else if (kSwap) tma_load_3d_hint<kPair>(dst, &p.tm_r, full_bar, kr, mn, r_batch, l2_policy_evict_last());
                            else            tma_load_3d<kPair>(dst, &p.tm_r, full_bar, kr, mn, r_batch);
                        }
                      }
                    } else if (elect_one()) {
                        const uint32_t full_bar = full_bar0 + stage * 8;
                        mbar_arrive_expect_tx_cluster(full_bar, tile_tx_bytes - p.r.tx_bytes);
                        const uint32_t kc = c_k + kb * c_kstep;
                        for (uint32_t b = 0; b < c_boxes; ++b) {
                            const uint32_t dst = smem_c + stage * Cfg::C_STAGE + b * c_box_bytes;
                            const uint32_t mn = (c_mn + b * c_box_mn) * c_esz;
                            if (c_mn_major) tma_load_3d<kPair>(dst, &p.tm_c, full_bar, mn, kc, c_batch);
                            else            tma_load_3d<kPair>(dst, tm_c_tile, full_bar, kc, mn, c_batch);
                        }
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == 1) {
        // ============================================================ UMMA issuer (leader CTA only)
        // Whole warp in the loop, one elected lane issues (always the same lane, so that
        // tcgen05.commit covers every UMMA issued before it).
        if (is_leader) {
            const uint32_t idesc_base = Cfg::kMxf4
                ? make_idesc_mxf4(128 * kCtas, BN)
                : Cfg::kBf16 ? make_idesc_bf16(p.r.mn_major != 0, p.c.mn_major != 0, 128 * kCtas, BN)
                : make_idesc_mxf8f6f4(p.r.fmt, p.c.fmt, p.r.mn_major != 0, p.c.mn_major != 0, 128 * kCtas, BN);
            const uint64_t sf_desc_hi = make_smem_desc(0, 0, 128, kSwizzleNone);
            // Operand descriptors: constant high word; the low word carries (address >> 4) and the LBO field
            const uint32_t r_hi = static_cast<uint32_t>(make_smem_desc(0, p.r.desc_lbo, p.r.desc_sbo, kSwizzle128B) >> 32);
            const uint32_t c_hi = static_cast<uint32_t>(make_smem_desc(0, p.c.desc_lbo, p.c.desc_sbo, kSwizzle128B) >> 32);
            const uint32_t r_lo0 = static_cast<uint32_t>(make_smem_desc(smem_r, p.r.desc_lbo, p.r.desc_sbo, kSwizzle128B));
            const uint32_t c_lo0 = static_cast<uint32_t>(make_smem_desc(smem_c, p.c.desc_lbo, p.c.desc_sbo, kSwizzle128B));
            const uint32_t r_kstep = p.r.desc_kstep >> 4, c_kstep = p.c.desc_kstep >> 4;
            // Scale byte selectors: per-32 scales pick byte ks of the word, per-128 scales byte (kb % 4)
            const uint32_t r_per32 = p.r.gran_k == 32 ? 1u : 0u, c_per32 = p.c.gran_k == 32 ? 1u : 0u;
            const uint32_t sfr_tmem = tmem_base + Cfg::kSfrCol, sfc_tmem = tmem_base + Cfg::kSfcCol;
            for (uint32_t iter = 0; ok; ++iter) {
                const uint32_t slot = unit + iter * p.num_units;
                const uint32_t num_sub = walker.next(slot, tiles);
                if (num_sub == 0) break;
                for (uint32_t sub = 0; sub < num_sub && ok; ++sub, ++acc_iter) {
                    const TileCoord& tc = tiles[sub];
                    const uint32_t acc = acc_iter & 1;
                    const uint32_t acc_phase = (acc_iter >> 1) & 1;
                    ok = wait_barrier(&bars->tmem_empty[acc], acc_phase ^ 1, abort_flag, peer_abort, p,
                                      kSiteMmaTmemEmpty, acc_iter, 0, acc);
                    if (!ok) break;
                    if (Cfg::kOverlap > 0 && acc_iter > 0) {
                        // The previous tile's epilogue must have drained the columns both stages share
                        const uint32_t prev = acc_iter - 1;
                        ok = wait_barrier(&bars->overlap[prev & 1], (prev >> 1) & 1, abort_flag, peer_abort, p,
                                          kSiteMmaOverlap, acc_iter, 0, acc);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + acc * Cfg::kAccStride;
                    const uint32_t idesc_tile = kSwap ? idesc_with_n(idesc_base, tc.rows) : idesc_base;
                    const uint32_t num_kb = max(1u, (tc.k_len + Cfg::BLOCK_K_ELEMS - 1) / Cfg::BLOCK_K_ELEMS);
                    for (uint32_t kb = 0; kb < num_kb; ++kb, advance()) {
                        DG_TRACE_AT(3, kb);
                        ok = wait_barrier(&bars->full[stage], phase, abort_flag, peer_abort, p, kSiteMmaFull, acc_iter,
                                          kb, stage);
                        if (!ok) break;
                        DG_TRACE_AT(4, kb);
                        tc_fence_after();
                        if (elect_one()) {
                            // Fresh scale factors: shared memory (already in 32x4 order) -> TMEM
                            // (kind::mxf4: two scale words per row; word w of 128 rows i sits at
                            // (w * rows + i * 128) * 4 in the stage and goes to columns w * rows / 32 + i * 4)
                            if constexpr (!Cfg::kBf16) {
                            if ((kb & sf_mask_r) == 0) {
#pragma unroll
                                for (uint32_t w = 0; w < Cfg::SF_WORDS; ++w) {
                                    const uint32_t a = smem_sfr + stage * Cfg::SFR_STAGE + w * 512;
                                    utccp_32x128b_warpx4<kCtas>(sfr_tmem + w * 4, sf_desc_hi | (a >> 4));
                                }
                            }
                            if ((kb & sf_mask_c) == 0) {
#pragma unroll
                                for (uint32_t w = 0; w < Cfg::SF_WORDS; ++w) {
#pragma unroll
                                    for (uint32_t i = 0; i < Cfg::SFC_ROWS / 128; ++i) {
                                        const uint32_t a = smem_sfc + stage * Cfg::SFC_STAGE + (w * Cfg::SFC_ROWS + i * 128) * 4;
                                        utccp_32x128b_warpx4<kCtas>(sfc_tmem + w * Cfg::SFC_COLS_PER_WORD + i * 4,
                                                                    sf_desc_hi | (a >> 4));
                                    }
                                }
                            }
                            }
                            const uint32_t r_lo = r_lo0 + stage * (Cfg::R_STAGE >> 4);
                            const uint32_t c_lo = c_lo0 + stage * (Cfg::C_STAGE >> 4);
                            const uint32_t id128 = kb & 3;
                            const uint32_t idesc_kb = idesc_tile | ((c_per32 ? 0u : id128) << 4) |
                                                      ((r_per32 ? 0u : id128) << 29);
                            const uint32_t idesc_ks = (c_per32 << 4) | (r_per32 << 29);
#pragma unroll
                            for (uint32_t ks = 0; ks < 4; ++ks) {
                                const uint64_t r_desc = (static_cast<uint64_t>(r_hi) << 32) | (r_lo + ks * r_kstep);
                                const uint64_t c_desc = (static_cast<uint64_t>(c_hi) << 32) | (c_lo + ks * c_kstep);
                                if constexpr (Cfg::kBf16) {
                                    umma_bf16<kCtas>(d_tmem, r_desc, c_desc, idesc_tile, (kb | ks) != 0);
                                } else if constexpr (Cfg::kMxf4) {
                                    // UMMA K = 64: scale bytes (ks % 2) * 2 and + 1 of word ks / 2, on both sides
                                    const uint32_t id = (ks & 1u) * 2u;
                                    umma_mxf4<kCtas>(d_tmem, r_desc, c_desc, idesc_tile | (id << 4) | (id << 29),
                                                     sfr_tmem + (ks >> 1) * 4, sfc_tmem + (ks >> 1) * Cfg::SFC_COLS_PER_WORD,
                                                     (kb | ks) != 0);
                                } else {
                                    umma_mxf8f6f4<kCtas>(d_tmem, r_desc, c_desc, idesc_kb + ks * idesc_ks, sfr_tmem,
                                                         sfc_tmem, (kb | ks) != 0);
                                }
                            }
                            umma_commit<kCtas>(&bars->empty[stage]);   // frees the stage (in both CTAs)
                            if (kb + 1 == num_kb) umma_commit<kCtas>(&bars->tmem_full[acc]);
                        }
                        __syncwarp();
                        DG_TRACE_AT(5, kb);
                    }
                }
            }
        }
    } else if (warp == 2 || warp == 9) {
        // ============================================================ scale-factor transposer(s)
        // tcgen05.cp 32x128b.warpx4 wants, per 128 rows, row i's word at position (i % 32) * 4 + i / 32.  The 128-row
        // blocks of a K block (R's, then C's) are dealt to the transposer warps in turn.
        const uint32_t full_bar = leader_addr(&bars->full[0]);
        const uint32_t tr = warp == 2 ? 0u : 1u;
        if constexpr (!Cfg::kBf16) {   // BF16 operands carry no scale factors
        for (uint32_t iter = 0; ok; ++iter) {
            const uint32_t slot = unit + iter * p.num_units;
            const uint32_t num_sub = walker.next(slot, tiles);
            if (num_sub == 0) break;
            for (uint32_t sub = 0; sub < num_sub && ok; ++sub, ++acc_iter) {
                const uint32_t num_kb = max(1u, (tiles[sub].k_len + Cfg::BLOCK_K_ELEMS - 1) / Cfg::BLOCK_K_ELEMS);
                for (uint32_t kb = 0; kb < num_kb; ++kb, advance()) {
                    ok = wait_barrier(&bars->sf_full[stage], phase, abort_flag, peer_abort, p, kSiteTransposerSfFull,
                                      acc_iter, kb, stage);
                    if (!ok) break;
                    DG_TRACE_AT(2, kb);
                    auto transpose_128 = [&](uint32_t* w) {
                        uint32_t v0 = w[lane], v1 = w[32 + lane], v2 = w[64 + lane], v3 = w[96 + lane];
                        __syncwarp();
                        reinterpret_cast<uint4*>(w)[lane] = make_uint4(v0, v1, v2, v3);
                    };
                    const bool new_r = (kb & sf_mask_r) == 0, new_c = (kb & sf_mask_c) == 0;
                    constexpr uint32_t kRBlocks = Cfg::SF_WORDS, kCBlocks = Cfg::SF_WORDS * Cfg::SFC_ROWS / 128;
                    if (new_r && !p.r_sf_pretransposed) {
#pragma unroll
                        for (uint32_t i = 0; i < kRBlocks; ++i)
                            if (i % Cfg::kTransposers == tr) transpose_128(sf_words_r + stage * (Cfg::SFR_STAGE / 4) + i * 128);
                    }
                    if (new_c && !p.c_sf_pretransposed) {
#pragma unroll
                        for (uint32_t i = 0; i < kCBlocks; ++i)
                            if ((kRBlocks + i) % Cfg::kTransposers == tr)
                                transpose_128(sf_words_c + stage * (Cfg::SFC_STAGE / 4) + i * 128);
                    }
                    if ((new_r && !p.r_sf_pretransposed) || (new_c && !p.c_sf_pretransposed)) {
                        fence_proxy_async_smem();   // generic-proxy writes -> visible to tcgen05.cp
                        __syncwarp();
                    }
                    if (lane == 0) mbar_arrive_cluster(full_bar + stage * 8);
                }
            }
        }
        }
    } else if (warp >= 4) {
        // ============================================================ epilogue
        const uint32_t q = warp - 4;   // TMEM lane quadrant == warp % 4
        const uint32_t tmem_empty_bar = leader_addr(&bars->tmem_empty[0]);
        const uint32_t overlap_bar = leader_addr(&bars->overlap[0]);
        const uint32_t slab0 = smem_cd + q * Cfg::SLAB_BYTES;
        uint8_t* slab0_gen = smem_gen + (slab0 - smem_base);
        uint32_t buf = 0, moe_buf = 0, moe_chunks = 0, clamp_count = 0;
        (void)buf, (void)moe_buf, (void)moe_chunks, (void)clamp_count;
        for (uint32_t iter = 0; ok; ++iter) {
            const uint32_t slot = unit + iter * p.num_units;
            const uint32_t num_sub = walker.next(slot, tiles);
            if (num_sub == 0) break;
            for (uint32_t sub = 0; sub < num_sub && ok; ++sub, ++acc_iter) {
                const TileCoord& tc = tiles[sub];
                const uint32_t acc = acc_iter & 1;
                const uint32_t acc_phase = (acc_iter >> 1) & 1;
                if constexpr (Cfg::kMoeEpi) {
                    // Per-token data of this tile, fetched while the UMMAs still run: route weights (kEpi 1) or
                    // destination addresses in the source ranks' combine planes (kEpi 2; 0 = row carries no token)
                    uint64_t* table = reinterpret_cast<uint64_t*>(smem_gen + (smem_cd - smem_base) + Cfg::MOE_TABLE_OFF) +
                                      acc * 256;
                    for (uint32_t tok = q * 32 + lane; tok < tc.rows; tok += 128) {
                        const uint32_t row = tc.row0 + tok;
                        if constexpr (Cfg::kEpi == 1) {
                            reinterpret_cast<float*>(table)[tok] = p.moe.pool_w[row];
                        } else {
                            const int32_t src_rank = p.moe.pool_meta[row * 3];
                            uint64_t dst = 0;
                            if (src_rank >= 0) {
                                const uint64_t token = static_cast<uint32_t>(p.moe.pool_meta[row * 3 + 1]);
                                const uint64_t slot = static_cast<uint32_t>(p.moe.pool_meta[row * 3 + 2]);
                                dst = reinterpret_cast<uint64_t>(p.moe.peer_base[src_rank]) + p.moe.off_combine +
                                      (slot * p.moe.t_max + token) * p.moe.hidden * 2;
                            }
                            table[tok] = dst;
                        }
                    }
                }
                ok = wait_barrier(&bars->tmem_full[acc], acc_phase, abort_flag, peer_abort, p, kSiteEpilogueTmemFull,
                                  acc_iter, 0, acc);
                if (!ok) break;
                tc_fence_after();
                const uint32_t t_acc = tmem_base + acc * Cfg::kAccStride + ((q * 32) << 16);
                // Where this warp's 32 lanes land in D
                //   D tile  : rows m0 + q*32 .. +31, columns n0 + chunk
                //   D^T tile: columns n0 + q*32 .. +31 (lanes), rows m0 + chunk (TMEM columns)
                const uint32_t m0 = tc.row0 + (kSwap ? 0 : cta_rank * 128);
                const uint32_t n0 = tc.n_blk * Cfg::UNIT_N + (kSwap ? cta_rank * 128 : 0);
                const uint32_t num_chunks = kSwap ? (tc.rows + Cfg::CHUNK_COLS - 1) / Cfg::CHUNK_COLS
                                                  : BN / Cfg::CHUNK_COLS;
                // Stage 0 shares its last columns, stage 1 its first: drain the shared ones first
                const bool reverse = Cfg::kOverlap > 0 && acc == 0;
#pragma unroll 1
                for (uint32_t i = 0; i < num_chunks; ++i) {
                    const uint32_t ch = reverse ? num_chunks - 1 - i : i;
                    uint32_t v[Cfg::CHUNK_COLS];
#pragma unroll
                    for (uint32_t j = 0; j < Cfg::CHUNK_COLS / 32; ++j)
                        tmem_ld_32x32b_x32(t_acc + ch * Cfg::CHUNK_COLS + j * 32, v + j * 32);
                    tmem_ld_wait();
                    if (i == 0 || i + 1 == num_chunks) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            // First chunk read: the shared columns may be overwritten by the next tile.
                            // Last chunk read: the whole stage goes back to the UMMA issuer.
                            if (Cfg::kOverlap > 0 && i == 0) mbar_arrive_cluster(overlap_bar + acc * 8);
                            if (i + 1 == num_chunks) mbar_arrive_cluster(tmem_empty_bar + acc * 8);
                        }
                    }
                    if constexpr (!Cfg::kMoeEpi) {
                    // A K group without rows (K-grouped layouts allow them) contributes nothing: its single K block
                    // ran on whatever follows it in memory, so the accumulator is replaced by zeros
                    // (D = 0, or D unchanged when accumulating).
                    if (tc.k_len == 0) {
#pragma unroll
                        for (uint32_t j = 0; j < Cfg::CHUNK_COLS; ++j) v[j] = 0;
                    }
                    // The slab we are about to overwrite must have been read by its previous store
                    if (lane == 0) tma_store_wait_read<Cfg::kStoreBufs - 1>();
                    __syncwarp();
                    const uint32_t slab = slab0 + buf * 4 * Cfg::SLAB_BYTES;
                    uint8_t* slab_gen = slab0_gen + buf * 4 * Cfg::SLAB_BYTES;
                    if constexpr (!kSwap) {
                        // Row `lane` of the slab: 128 B, 16 B chunks XOR-swizzled by (row % 8)
                        uint4* row = reinterpret_cast<uint4*>(slab_gen + lane * 128);
                        if constexpr (Cfg::kEpi == kEpiFp8Cast) {
                            // E4M3 output with one UE8M0 scale per row and 32 columns: BF16 rounding first, so that the
                            // bytes equal a BF16 D followed by the per-token cast (deep_gemm/utils/math.py:26-49)
                            const bool counted = m0 + q * 32 + lane < p.m && n0 + ch * 64 < p.n;
                            const float bound = p.cast.clamp_bound;
                            uint4* row64 = reinterpret_cast<uint4*>(slab_gen + lane * 64);
                            uint32_t sf_bytes = 0;
#pragma unroll
                            for (uint32_t g = 0; g < 2; ++g) {
                                float x[32];
                                float amax = 0.f;
                                uint32_t over = 0;
#pragma unroll
                                for (uint32_t j = 0; j < 32; ++j) {
                                    x[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(v[g * 32 + j])));
                                    const float ax = fabsf(x[j]);
                                    over += ax > bound ? 1u : 0u;
                                    amax = fmaxf(amax, ax);
                                }
                                if (counted) clamp_count += over;
                                amax = fminf(amax, bound);
                                // power-of-two scale 2^e >= amax / 448, floor 2^-22 (as in moe_l1_chunk_impl)
                                uint32_t e = (__float_as_uint(amax) + 0x1FFFFFu) >> 23;
                                e = max(e, 113u) - 8u;
                                const float inv = __uint_as_float((254u - e) << 23);
                                sf_bytes |= e << (8 * g);
#pragma unroll
                                for (uint32_t c16 = 0; c16 < 2; ++c16) {
                                    uint32_t w[4];
#pragma unroll
                                    for (uint32_t j = 0; j < 4; ++j) {
                                        float f[4];
#pragma unroll
                                        for (uint32_t l = 0; l < 4; ++l)
                                            f[l] = fminf(fmaxf(x[c16 * 16 + j * 4 + l], -bound), bound) * inv;
                                        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[0], f[1]), __NV_SATFINITE, __NV_E4M3);
                                        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[2], f[3]), __NV_SATFINITE, __NV_E4M3);
                                        w[j] = lo | (hi << 16);
                                    }
                                    row64[g * 2 + c16] = make_uint4(w[0], w[1], w[2], w[3]);
                                }
                            }
                            if (counted) {
                                const uint32_t sf_idx = (tc.group * p.n + n0 + ch * 64) >> 5;   // even: two scales of one word
                                uint8_t* dst = reinterpret_cast<uint8_t*>(p.cast.sfd + static_cast<uint64_t>(sf_idx >> 2) * p.cast.sfd_ld +
                                                                          (m0 + q * 32 + lane)) + (sf_idx & 3u);
                                *reinterpret_cast<uint16_t*>(dst) = static_cast<uint16_t>(sf_bytes);
                            }
                        } else if constexpr (Cfg::kEpi == kEpiStochastic) {
                            // BF16 with stochastic rounding: the 16 dropped bits of each FP32 value plus 16 random bits,
                            // carried into the kept half.  The random bits come from a hash of the four FP32 bit patterns
                            // of the value's column quartet (columns 4i .. 4i+3 of D) and the quartet's index, so the
                            // result is a function of the FP32 result alone (epilogue/operators.cuh:53-114 and
                            // tests/utils.py:53-79 of the reference state the hash)
#pragma unroll
                            for (uint32_t c16 = 0; c16 < 8; ++c16) {
                                uint32_t w[4];
#pragma unroll
                                for (uint32_t h4 = 0; h4 < 2; ++h4) {
                                    const uint32_t* a = v + c16 * 8 + h4 * 4;
                                    uint32_t h = a[0] * 0x5671d42bu + a[1] * 0x9995e499u + a[2] * 0xace1b8a5u + a[3] * 0xe153538du +
                                                 ((n0 + ch * 64 + c16 * 8 + h4 * 4) >> 2);
                                    h = (h ^ (h >> 23)) * 0x7feb352du;
                                    h ^= h >> 16;
                                    uint32_t h1 = h * 0x846ca68bu, h2 = h * 0xd35a2d97u;
                                    h1 ^= h1 >> 11, h2 ^= h2 >> 11;
                                    const uint32_t r0 = (a[0] >> 16) + (((a[0] & 0xffffu) + (h1 & 0xffffu)) >> 16);
                                    const uint32_t r1 = (a[1] >> 16) + (((a[1] & 0xffffu) + (h1 >> 16)) >> 16);
                                    const uint32_t r2 = (a[2] >> 16) + (((a[2] & 0xffffu) + (h2 & 0xffffu)) >> 16);
                                    const uint32_t r3 = (a[3] >> 16) + (((a[3] & 0xffffu) + (h2 >> 16)) >> 16);
                                    w[h4 * 2] = (r0 & 0xffffu) | (r1 << 16);
                                    w[h4 * 2 + 1] = (r2 & 0xffffu) | (r3 << 16);
                                }
                                row[c16 ^ (lane & 7)] = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        } else if constexpr (Cfg::kCdF32) {
#pragma unroll
                            for (uint32_t c16 = 0; c16 < 8; ++c16) {
                                float4 f;
                                f.x = __uint_as_float(v[c16 * 4 + 0]) * p.alpha;
                                f.y = __uint_as_float(v[c16 * 4 + 1]) * p.alpha;
                                f.z = __uint_as_float(v[c16 * 4 + 2]) * p.alpha;
                                f.w = __uint_as_float(v[c16 * 4 + 3]) * p.alpha;
                                reinterpret_cast<float4*>(row)[c16 ^ (lane & 7)] = f;
                            }
                        } else {
#pragma unroll
                            for (uint32_t c16 = 0; c16 < 8; ++c16) {
                                uint32_t w[4];
#pragma unroll
                                for (uint32_t j = 0; j < 4; ++j) {
                                    const float lo = __uint_as_float(v[c16 * 8 + j * 2]) * p.alpha;
                                    const float hi = __uint_as_float(v[c16 * 8 + j * 2 + 1]) * p.alpha;
                                    const __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                                    w[j] = *reinterpret_cast<const uint32_t*>(&b2);
                                }
                                row[c16 ^ (lane & 7)] = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    } else {
                        // D^T: lane holds column n0 + q*32 + lane for 32 tokens; slab is [token][32 n] BF16
                        __nv_bfloat16* s = reinterpret_cast<__nv_bfloat16*>(slab_gen);
#pragma unroll
                        for (uint32_t t = 0; t < 32; ++t)
                            s[t * 32 + lane] = __float2bfloat16_rn(__uint_as_float(v[t]) * p.alpha);
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        int32_t cn, cm;
                        if constexpr (!kSwap) {
                            cn = static_cast<int32_t>(n0 + ch * Cfg::CHUNK_COLS);
                            cm = static_cast<int32_t>(m0 + q * 32);
                        } else {
                            cn = static_cast<int32_t>(n0 + q * 32);
                            cm = static_cast<int32_t>(m0 + ch * 32);
                        }
                        const int32_t cg = p.d_grouped ? static_cast<int32_t>(tc.group) : 0;
                        // a swapped tile's rows are a multiple of 16: its last chunk may hold 16 token rows only, and
                        // the rows after them belong to another tile
                        const CUtensorMap* tm_out = (kSwap && tc.rows - ch * 32 == 16) ? &p.tm_d_half : &p.tm_d;
                        // D is written once and not read again by this kernel: its lines are the first to leave L2,
                        // which keeps the operands there longer (measured on the grouped headline shape: 5 % fewer
                        // DRAM reads)
                        if (p.accumulate) tma_reduce_add_3d(tm_out, slab, cn, cm, cg);
                        else              tma_store_3d_hint(tm_out, slab, cn, cm, cg, l2_policy_evict_first());
                        tma_store_commit();
                    }
                    buf = buf + 1 == Cfg::kStoreBufs ? 0 : buf + 1;
                    } else {
                        // Fused Mega MoE epilogues: the four warps stage this chunk's 32 tokens x 128 rows as
                        // BF16 [token][row] in shared memory (two buffers, one named barrier per chunk: a
                        // buffer is rewritten two chunks later, after its readers passed the next barrier).
                        uint8_t* stage_gen = smem_gen + (smem_cd - smem_base) + moe_buf * 32 * Cfg::MOE_PITCH;
#pragma unroll
                        for (uint32_t t = 0; t < 32; ++t)
                            *reinterpret_cast<__nv_bfloat16*>(stage_gen + t * Cfg::MOE_PITCH + (q * 32 + lane) * 2) =
                                __float2bfloat16_rn(__uint_as_float(v[t]));
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bars->epi_sync[moe_buf]);
                        ok = wait_barrier(&bars->epi_sync[moe_buf], (moe_chunks >> 1) & 1, abort_flag, peer_abort, p,
                                          kSiteEpilogueSync, acc_iter, ch, moe_buf);
                        ++moe_chunks;
                        if (!ok) break;
                        const uint32_t chunk_rows = min(32u, tc.rows - ch * 32);
                        const uint64_t* table = reinterpret_cast<const uint64_t*>(smem_gen + (smem_cd - smem_base) +
                                                                                  Cfg::MOE_TABLE_OFF) + acc * 256;
                        if constexpr (Cfg::kEpi == 1)
                            moe_l1_chunk(p.moe, stage_gen, Cfg::MOE_PITCH, reinterpret_cast<const float*>(table), q, lane, ch,
                                         chunk_rows, m0, n0, /*sf_base=*/m0);   // tiles start on 128-row boundaries here
                        else
                            moe_l2_chunk(stage_gen, Cfg::MOE_PITCH, table, q * 32 + lane, ch, chunk_rows, n0,
                                         p.moe.post_down ? p.moe.pool_w + m0 : nullptr);
                        moe_buf ^= 1;
                    }
                }
            }
        }
        if (!Cfg::kMoeEpi && lane == 0) tma_store_wait<0>();
        if constexpr (Cfg::kEpi == kEpiFp8Cast) {
            if (p.cast.clamped_count != nullptr) {      // one atomic per warp
                const uint32_t total = __reduce_add_sync(0xffffffffu, clamp_count);
                if (lane == 0 && total != 0) atomicAdd(p.cast.clamped_count, total);
            }
        }
    }

    // ---------------------------------------------------------------- tear-down
    if (*abort_flag) {
        // Copies issued before the abort may still be landing in this CTA's shared memory
        for (int i = 0; i < 20; ++i) __nanosleep(10000);
    }
    __syncwarp();
    tc_fence_before();
    if (kPair) cluster_sync(); else __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<kCtas>(tmem_base, Cfg::kTmemCols);
    }
}

}  // namespace dg
