/* C ABI of libdeepgemm_b200.so: block-scaled FP8 / FP8xFP4 GEMMs for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; every tensor is borrowed for the duration of the enqueued
 * work and must be device memory of the current CUDA device unless stated otherwise.  All
 * entry points return 0 on success and a non-zero code on failure, in which case
 * dg_last_error() (thread-local) describes the failed check.  Work is enqueued on the
 * given stream and the call returns without synchronising.
 *
 * Each entry point names the function of the reference (fw-ai/DeepGEMM, paths relative to
 * its root) whose role it takes behind the `deep_gemm` Python operator surface.
 */
#ifndef DEEPGEMM_B200_H_
#define DEEPGEMM_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum dg_status {
    DG_OK = 0,
    DG_ERR_INVALID = 1,   /* an argument check failed; see dg_last_error() */
    DG_ERR_CUDA = 2,      /* a CUDA runtime / driver call failed */
    DG_ERR_DEVICE = 3,    /* a kernel gave up on a bounded wait; see dg_check_status() */
};

enum dg_gemm_type {
    DG_GEMM_NORMAL = 0,
    DG_GEMM_M_CONTIGUOUS = 1,    /* grouped_layout: int32[M], expert id per row, -1 = padding */
    DG_GEMM_M_MASKED = 2,        /* grouped_layout: int32[G], valid rows per group (read on device) */
    DG_GEMM_M_PSUM = 3,          /* grouped_layout: int32[G], cumulative un-aligned row ends */
    DG_GEMM_K_GROUPED = 4,       /* grouped_layout: int32[G], padded K per group */
    DG_GEMM_K_GROUPED_PSUM = 5,  /* grouped_layout: int32[G], cumulative un-aligned K ends */
    DG_GEMM_BATCHED = 6,         /* num_groups independent problems of one shape; no layout tensor */
};

/* What happens to the FP32 accumulator (deep_gemm/include/deep_gemm/epilogue/operators.cuh of the reference). */
enum dg_epilogue {
    DG_EPILOGUE_STORE = 0,            /* D = alpha * acc cast to d_dtype, or D += acc (Identity / ScaleByAlpha, :12-51) */
    DG_EPILOGUE_STOCHASTIC_BF16 = 1,  /* BF16 D, stochastically rounded with bits hashed from the FP32 result (:53-114) */
    DG_EPILOGUE_FP8_CAST = 2,         /* E4M3 D + per-row, per-32-column UE8M0 scales, optional clamp (:116-220) */
};

enum dg_dtype { DG_E4M3 = 0, DG_E2M1_PACKED = 1, DG_BF16 = 2, DG_F32 = 3 };   /* d_dtype: BF16, F32, or E4M3 (FP8_CAST) */

/* One operand: quantised data plus packed UE8M0 scale factors, or BF16 data without scales (sf = NULL, gran_k 0;
 * bf16_gemm_* and their grouped forms, csrc/apis/gemm.hpp:492-726 of the reference).
 *   data : E4M3 bytes, E2M1 codes two per byte (low nibble first), or BF16.
 *   ld   : distance in bytes between consecutive rows of the non-contiguous axis
 *          (K-major: between MN rows; MN-major: between K rows).
 *   sf   : int32, four UE8M0 exponents per word in K order, MN-major:
 *          element (g, mn, kw) at  g * sf_group_stride + kw * sf_ld + mn   (in words).
 *          K-grouped GEMMs: (kw, mn) at kw * sf_ld + mn with groups stacked along kw.
 */
typedef struct dg_operand {
    const void* data;
    const int32_t* sf;
    int64_t ld;
    int64_t sf_ld;
    int32_t dtype;      /* DG_E4M3, DG_E2M1_PACKED or DG_BF16 (then both operands) */
    int32_t mn_major;   /* 0: K contiguous, 1: MN contiguous (E4M3 and BF16) */
    int32_t gran_k;     /* K elements per scale: 32 or 128 */
    int32_t reserved;
    int64_t batch_stride; /* bytes between the groups / batches of `data`; 0 = stacked without gaps
                             (rows * ld for a K-major operand, k * ld for an MN-major one) */
    int64_t sf_k_rows;    /* K-grouped GEMMs: rows (packed-K words) the sf tensor holds; 0 = not known */
} dg_operand;

/* Arguments of dg_gemm_bs.  Shapes are logical GEMM shapes: D[m, n] = A[m, k] * B[n, k]^T.
 *   NORMAL        : a [m,k], b [n,k], d [m,n]
 *   M_CONTIGUOUS  : a [m,k] (m = all groups' rows), b [G,n,k], d [m,n]
 *   M_PSUM        : as M_CONTIGUOUS; group g owns rows [align(end[g-1], alignment), end[g])
 *   M_MASKED      : a [G,m,k], b [G,n,k], d [G,m,n] (m = max rows per group)
 *   K_GROUPED*    : a [sum_k, m], b [sum_k, n] (both MN-major), d [G,m,n], k = sum of padded K;
 *                   FP4 x FP4: a [m, sum_k], b [n, sum_k] K-major with the groups along K
 *   BATCHED       : a [G,m,k], b [G,n,k], d [G,m,n], every tensor with its own batch stride
 * Both operands DG_E2M1_PACKED selects the FP4 x FP4 path (tcgen05 kind::mxf4, twice the FP8 rate): K-major
 * operands, gran_k 32 on both sides, k % 128 == 0.
 * Both operands DG_BF16 selects the unscaled path (tcgen05 kind::f16, FP32 accumulation): every layout but BATCHED,
 * the STORE and STOCHASTIC_BF16 epilogues, ld a multiple of 16 bytes.
 */
typedef struct dg_gemm_args {
    int32_t gemm_type;
    int32_t m, n, k;
    int32_t num_groups;
    int32_t alignment;        /* M (psum) or K (k-grouped) group alignment */
    dg_operand a, b;
    void* d;
    int64_t ldd;              /* bytes between rows of d */
    int32_t d_dtype;          /* DG_BF16 or DG_F32 */
    int32_t accumulate;       /* d += result instead of d = result */
    float alpha;              /* result scale; pass 1.0f when unused */
    int32_t expected_m;       /* heuristic hint for grouped layouts; 0 = none */
    const int32_t* grouped_layout;
    void* stream;             /* cudaStream_t */
    int64_t d_batch_stride;   /* bytes between the groups / batches of d; 0 = m * ldd */
    int32_t epilogue;         /* enum dg_epilogue; the value epilogues: NORMAL / BATCHED, alpha 1, no accumulate */
    float clamp_value;        /* FP8_CAST: BF16 values are clamped to +-clamp_value before scaling; 0 = no clamp */
    int32_t* sfd;             /* FP8_CAST: packed UE8M0 scales of d seen as [m, groups * n]: the scale of row r and
                                 column group g = (batch * n + column) / 32 is byte g % 4 of word sfd[(g / 4) * sfd_ld + r] */
    int64_t sfd_ld;
    uint32_t* clamped_count;  /* FP8_CAST with a clamp, optional: receives the number of elements whose BF16 magnitude
                                 exceeded clamp_value (overwritten, in stream order) */
    int32_t skip_padding_rows; /* M_PSUM: 0 = every group's whole aligned extent is computed, so zero padding rows of a
                                  give zero rows of d; 1 = only the valid rows, rounded up to 16 (the reference's
                                  ensure_zero_padding = false, deep_gemm/include/deep_gemm/scheduler/gemm.cuh:178-184) */
    int32_t reserved;
} dg_gemm_args;

/* Block-scaled GEMM, all layouts.  Takes the role of sm100_fp8_fp4_gemm_1d1d and its grouped, batched and FP4 x FP4
 * variants (csrc/jit_kernels/impls/sm100_fp8_fp4_gemm_1d1d.hpp:101-561) as called from
 * fp8_fp4_gemm_nt, m_grouped_fp8_fp4_gemm_nt_contiguous, m_grouped_fp8_fp4_gemm_nt_masked,
 * k_grouped_fp8_gemm_tn_contiguous, k_grouped_fp4_gemm_nt_contiguous (csrc/apis/gemm.hpp:78-491) and fp8_einsum
 * (csrc/apis/einsum.hpp:182-304). */
int dg_gemm_bs(const dg_gemm_args* args);

/* FP32 power-of-two scales -> packed UE8M0, MN-major, 16-byte-aligned columns.
 *   sf  : float32, the scale of row mn is element (b, mn / gran_mn, k) at
 *         b * stride_b + (mn / gran_mn) * stride_mn + k * stride_k (elements); gran_mn = 1 for
 *         per-row scales, 128 to broadcast 128x128 block scales to rows (csrc/apis/layout.hpp:47-50)
 *   out : int32 [num_batches, mn, ceil(sf_k / 4)], element (b, mn, kw) at
 *         b * ceil(sf_k/4) * align(mn, 4) + kw * align(mn, 4) + mn
 *   psum_layout (optional, int32[num_psum_groups], device): rows outside
 *         [align(end[g-1], psum_alignment), end[g]) are written as zero.
 * Takes the role of get_mn_major_tma_aligned_packed_ue8m0_tensor
 * (csrc/jit_kernels/impls/smxx_layout.hpp:133-246) and its kernel
 * transpose_and_pack_fp32_into_ue8m0 (deep_gemm/include/deep_gemm/impls/smxx_layout.cuh:76-191). */
int dg_sf_pack_ue8m0(const float* sf, int32_t* out, int32_t num_batches, int32_t mn, int32_t sf_k,
                     int32_t gran_mn, int64_t stride_b, int64_t stride_mn, int64_t stride_k,
                     const int32_t* psum_layout, int32_t num_psum_groups, int32_t psum_alignment, void* stream);

/* K-grouped packing: sf float32 [sum(sf_k_g), mn] (mn contiguous) -> out int32 [sum(ceil(sf_k_g / 4)), mn];
 * every group starts a new packed row and zero-fills the unused bytes of its last row.
 *   grouped_layout (device int32[num_groups]): padded K per group, or (use_psum) cumulative K ends.
 * Takes the role of get_k_grouped_mn_major_tma_aligned_packed_ue8m0_tensor
 * (csrc/jit_kernels/impls/smxx_layout.hpp:248-313, kernel pack_fp32_into_ue8m0,
 * deep_gemm/include/deep_gemm/impls/smxx_layout.cuh:305-405). */
int dg_sf_pack_ue8m0_k_grouped(const float* sf, int32_t* out, const int32_t* grouped_layout, int32_t num_groups,
                               int32_t mn, int32_t sf_k_rows, int32_t packed_rows, int32_t gran_k,
                               int32_t k_alignment, int32_t use_psum, void* stream);


/* ---- Mega MoE forward (expert parallel over the GPUs of one node) ------------------------------------
 * One symmetric buffer per rank (same layout everywhere) holds the caller's inputs, the exchange tables,
 * the expert-sorted token pool and the combine planes; `buffer_ptrs[r]` is rank r's buffer as mapped into
 * the calling process (peer access over NVLink; with one rank, the buffer itself). */
typedef struct dg_moe_config {
    int32_t num_ranks, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden;
    /* Rows (token, expert pairs) the expert-sorted pool of one rank must hold, the role of the reference's
     * `num_ring_tokens` (csrc/apis/mega_moe.hpp:49-96): 0 = the worst case num_max_tokens_per_rank * num_ranks *
     * min(num_topk, experts per rank); a smaller value saves memory, and a call that receives more rows than fit
     * is abandoned and reported by dg_check_status (code 3). */
    int32_t num_ring_tokens;
    /* Shared experts: applied to every token on the token's own rank, E4M3 weights [2 * S * I, H] and [H, S * I]
     * (S = num_shared_experts; they act as one expert of intermediate size S * I), no route weight; their row enters
     * the final sum first (csrc/apis/mega_moe.hpp:82-119,392-415 of the reference).  0 = none. */
    int32_t num_shared_experts;
} dg_moe_config;

/* Byte offsets of the views inside one rank's buffer (shapes as in csrc/apis/mega_moe.hpp:137-226 of the
 * reference): x e4m3 [T, H]; x_sf int32 [T, H/128]; topk_idx int64 [T, K]; topk_weights f32 [T, K];
 * l1_acts e4m3 [P, H]; l1_acts_sf int32 [Q, H/128] with strides (1, Q); l2_acts e4m3 [P, I];
 * l2_acts_sf int32 [Q, I/128] with strides (1, Q); token_src_metadata int32 [P, 3];
 * combine bf16 [K (+ 1 with shared experts), T, H].  P = pool_rows, Q = sf_rows >= P.  The scale words of l1_acts_sf
 * and l2_acts_sf sit in blocks of 128 rows in the order tcgen05.cp consumes (row r of a block at (r % 32) * 4 + r / 32);
 * the single-kernel forward gives every token tile (dg_get_block_m_for_mega_moe rows) 256 scale rows of its own (tile j: rows [256 j, 256 j + 256)),
 * the kernel-per-phase forward uses the first P rows, pool row for pool row.
 * With shared experts (offsets 0 otherwise): shared_l1_acts_sf int32 [T', H/128] with strides (1, T'), T' = T rounded
 * up to 128 - the scales of x once more, in that same row order, filled by the caller along with x_sf;
 * shared_l2_acts e4m3 [T', S*I]; shared_l2_acts_sf int32 [T', S*I/128] with strides (1, T'). */
typedef struct dg_moe_layout {
    int64_t num_bytes, pool_rows;
    int64_t off_x, off_x_sf, off_topk_idx, off_topk_weights;
    int64_t off_l1_acts, off_l1_acts_sf, off_l2_acts, off_l2_acts_sf, off_token_src_metadata, off_combine;
    int64_t off_shared_l1_acts_sf, off_shared_l2_acts, off_shared_l2_acts_sf;
    int64_t sf_rows;
} dg_moe_layout;

/* Size and view offsets of the symmetric buffer.  Takes the role of get_symm_buffer_size_for_mega_moe_v3
 * (csrc/apis/mega_moe.hpp:73-229); the byte layout is this library's own. */
int dg_mega_moe_buffer_layout(const dg_moe_config* cfg, dg_moe_layout* out);

/* Row granularity of num_max_tokens_per_rank (csrc/apis/mega_moe.hpp:34-36). */
int dg_get_token_alignment_for_mega_moe(void);

/* Token rows per expert tile of the single-kernel forward; an expert's last tile shrinks to its rows rounded up to 16
 * (get_block_m_for_mega_moe, csrc/apis/mega_moe.hpp:38-47, which chooses per configuration; here it is one constant). */
int dg_get_block_m_for_mega_moe(void);

/* SMs the Mega MoE grid takes: dg_get_num_sms() (capped at the device's count) minus the environment variable
 * DG_MEGA_MOE_SM_HEADROOM rounded up to an even number; -1 with dg_last_error() set when the headroom is negative,
 * leaves no SM, or the result is odd (get_mega_moe_num_sms, csrc/jit_kernels/impls/runtime_utils.hpp:35-82). */
int dg_get_mega_moe_num_sms(void);

enum { DG_ACT_SWIGLU = 0, DG_ACT_GEGLU = 1, DG_ACT_SITU = 2 };

typedef struct dg_moe_args {
    dg_moe_config cfg;
    void* const* buffer_ptrs;   /* host array [num_ranks] of device addresses */
    int32_t rank;
    int32_t num_tokens;         /* rows of y and of the inputs in use on this rank */
    void* y;                    /* bf16 [num_tokens, hidden] */
    int64_t ldy;                /* elements between rows of y */
    /* Expert weights of this rank as produced by transform_weights_for_mega_moe
     * (deep_gemm/mega/__init__.py:201-220): MXFP4 codes [E_local, 2I, H/2] with gate / up rows interleaved in
     * blocks of 8 and [E_local, H, I/2]; packed UE8M0 scales MN-major, rows permuted per 128 for tcgen05.cp. */
    const void* l1_w;
    const int32_t* l1_sf;
    const void* l2_w;
    const int32_t* l2_sf;
    int64_t l1_sf_ld, l2_sf_ld; /* words between packed-K columns of the scale tensors */
    int32_t* stats;             /* optional int32 [E_local]: += rows received per local expert */
    float activation_clamp;     /* +inf: none */
    int32_t fast_math;
    void* stream;
    /* Gated activation (tests/test_mega_moe.py:451-463 of the reference): DG_ACT_SWIGLU gate * sigmoid(gate) * up;
     * DG_ACT_GEGLU the tanh form of GELU(gate) * up; DG_ACT_SITU situ_beta * tanh(gate / situ_beta) * sigmoid(gate)
     * * up', up' = situ_linear_beta * tanh(up / situ_linear_beta), or up when situ_linear_beta is +inf.
     * situ_beta <= 0 means the default 1. */
    int32_t activation;
    float situ_beta, situ_linear_beta;
    /* 0 (pre-down, default): the route weight multiplies the gated activation before it is requantised for the
     * second GEMM.  1 (post-down): the activation stays unweighted and each BF16 row of the second GEMM's output
     * is multiplied by its route weight and rounded to BF16 again where it is written to the combine plane
     * (impls/sm100_fp8_fp4_mega_moe.cuh:1538-1566 of the reference). */
    int32_t post_down;
    /* 0: expert weights are MXFP4 (two E2M1 codes per byte, [E_local, 2I, H/2] and [E_local, H, I/2]);
     * 1: E4M3 bytes ([E_local, 2I, H] and [E_local, H, I]), the reference's mma_type "fp8xfp8"
     * (csrc/apis/mega_moe.hpp:374-377,473).  Scales are packed 1 x 32 UE8M0 in both cases. */
    int32_t weights_fp8;
    /* Shared experts' weights as produced by transform_weights_for_mega_moe (E4M3, gate / up rows interleaved, packed
     * 1 x 32 scales in tcgen05.cp row order); all null when cfg.num_shared_experts == 0. */
    const void* shared_l1_w;      /* e4m3 [2 * S * I, H] */
    const int32_t* shared_l1_sf;
    const void* shared_l2_w;      /* e4m3 [H, S * I] */
    const int32_t* shared_l2_sf;
    int64_t shared_l1_sf_ld, shared_l2_sf_ld;
} dg_moe_args;

/* y[t] = bf16( sum over slots of bf16( Q32( SwiGLU(bf16(x_t W13_e^T)) * w_{t,slot} ) W2_e^T ) ) with the tokens
 * dispatched to the experts' ranks and the results combined back over NVLink peer memory.  Takes the role of
 * fp8_fp4_mega_moe (csrc/apis/mega_moe.hpp:321-519, impls/sm100_fp8_fp4_mega_moe.cuh).  Every rank of the
 * group must make the call; calls on one buffer must not overlap. */
int dg_mega_moe_forward(const dg_moe_args* args);

/* 1 (default): the forward runs as one persistent kernel (dispatch, both expert GEMMs, combine and reduction in a
 * single launch; needs all of the GPU's SMs free, hidden % 256 == 0 and experts_per_rank * ranks <= 511).
 * 0: one kernel per phase (7 launches), the same arithmetic; also the path taken when the conditions fail. */
int dg_set_mega_moe_fused(int32_t enable);

/* ---- Fused activation cast ------------------------------------------------------------------------------
 * BF16 [rows, cols] -> E4M3 [rows, cols] + one UE8M0 scale per 1 x gran_k group, in one kernel.  The arithmetic is
 * per_token_cast_to_fp8(use_ue8m0=True) of the reference (deep_gemm/utils/math.py:13-49); the reference runs it as
 * torch eager code and recommends fusing it into the producer (README.md:71,133-138), which this is.  The scales
 * are written directly in the form the consumer wants (no separate dg_sf_pack_ue8m0 launch):
 *   DG_CAST_SF_FLOAT             float32 [rows, ceil(cols / gran_k)], sf_ld elements between rows
 *   DG_CAST_SF_PACKED_ROW_MAJOR  int32 [rows, ceil(groups / 4)], four exponent bytes per word, sf_ld words between
 *                                rows (the use_packed_ue8m0 form; the x_sf view of the Mega MoE buffer)
 *   DG_CAST_SF_PACKED_MN_MAJOR   the same words at [kw * sf_ld + row]: what dg_gemm_bs reads (sf_ld >= align(rows, 4))
 * Groups of a word that cover no data get the exponent byte 127, as the reference pads.
 * x: 16-byte aligned, ldx (elements) % 8 == 0, cols % 8 == 0; q: 8-byte aligned, ldq (bytes) % 8 == 0. */
enum { DG_CAST_SF_FLOAT = 0, DG_CAST_SF_PACKED_ROW_MAJOR = 1, DG_CAST_SF_PACKED_MN_MAJOR = 2 };

typedef struct dg_cast_args {
    const void* x;      /* bf16 */
    int64_t ldx;
    int32_t rows, cols, gran_k; /* gran_k: 32 or 128 */
    void* q;            /* e4m3 bytes */
    int64_t ldq;
    void* sf;
    int32_t sf_mode;
    int64_t sf_ld;
    void* stream;
} dg_cast_args;

int dg_per_token_cast_to_fp8(const dg_cast_args* args);

/* ---- Dense FP8 GEMM that allocates nothing ------------------------------------------------------------
 * No counterpart in the reference.  For callers that must not call cudaMalloc (or any allocating library
 * routine) around the GEMM - a plugin running inside another runtime's memory plan, a real-time loop, code
 * between the nodes of a captured region's set-up - and therefore cannot provide the temporary packed scale
 * tensors that dg_sf_pack_ue8m0 + dg_gemm_bs need.  This entry point takes the FP32 power-of-two scales
 * directly and packs them into a scratch array built into the library image (4 MiB per GPU that loads the
 * library, held until the process exits), then runs the same GEMM kernel as dg_gemm_bs.
 *
 *   a : E4M3 [m, k], K contiguous, lda bytes between rows;  sfa : float32 [m, ceil(k / gran_k)] contiguous
 *   b : E4M3 [n, k], K contiguous, ldb bytes between rows;  sfb : float32 [ceil(n / gran_mn_b), ceil(k / gran_k)]
 *   d : BF16 or FP32 [m, n], ldd bytes between rows
 *
 * Limits and rules:
 *   - with w = ceil(k / (4 * gran_k)) packed words per row:
 *         round_up(align(m,4) * w * 4, 256) + align(n,4) * w * 4  bytes  <=  dg_noalloc_scratch_bytes()
 *     (the scales of a, rounded up to a 256-byte boundary, then those of b); larger problems are rejected with
 *     DG_ERR_INVALID and a message naming the sizes.
 *   - The first call on a device looks up the scratch array's device address (no allocation); make that
 *     first call before starting any stream capture.
 *   - All calls on one GPU share the one array, which keeps the last call's contents: each call rewrites
 *     every word it later reads, but two calls whose kernels overlap on the GPU (different streams) race. */
typedef struct dg_gemm_noalloc_args {
    int32_t m, n, k;
    int32_t gran_k;        /* 32 or 128 */
    int32_t gran_mn_b;     /* 1: per-row scales of b; 128: 128 x 128 block scales */
    int32_t d_dtype;       /* DG_BF16 or DG_F32 */
    const void* a;
    const float* sfa;
    const void* b;
    const float* sfb;
    void* d;
    int64_t lda, ldb, ldd;
    void* stream;
} dg_gemm_noalloc_args;
int dg_gemm_fp8_fp32sf_noalloc(const dg_gemm_noalloc_args* args);
int dg_noalloc_scratch_bytes(void);

/* Process-wide knobs (csrc/apis/config.hpp:8-48, csrc/apis/layout.hpp:138-146 of the reference). */
int dg_set_num_sms(int32_t num_sms);
int dg_get_num_sms(void);           /* device SM count unless overridden */
int dg_set_pdl(int32_t enable);     /* launch the GEMM, scale-packing and cast kernels with programmatic dependent launch */
int dg_get_pdl(void);
int dg_set_tc_util(int32_t percent);
int dg_get_tc_util(void);
int dg_set_mk_alignment_for_contiguous_layout(int32_t alignment);
int dg_get_mk_alignment_for_contiguous_layout(void);
int dg_get_theoretical_mk_alignment_for_contiguous_layout(int32_t expected_m);
int dg_set_wait_timeout_ms(int32_t ms);  /* budget of every device-side wait; default 2000 */

/* Test and tuning aid, not part of the operator surface (the reference's counterpart is its heuristics'
 * candidate enumeration, csrc/jit_kernels/heuristics/sm100.hpp:30-163): pins the tile that later dg_gemm_bs calls
 * of this process use.  cta_group 1 / 2, block_n = UMMA N (32 .. 256), swap 1 = tokens on the UMMA M axis,
 * 2 = weights on the UMMA M axis; 0 in any field = choose automatically. */
int dg_debug_set_tile_override(int32_t cta_group, int32_t block_n, int32_t swap);

/* Measurement aid (no counterpart in the reference): copies `bytes` (a multiple of 16, both addresses 16-byte
 * aligned) with plain 16-byte loads and stores by all SMs, the way the Mega MoE forward pulls token rows.  Given a
 * peer GPU's mapped address as `src` it measures the NVLink bandwidth that path can reach. */
int dg_debug_copy(void* dst, const void* src, int64_t bytes, void* stream);

/* Synchronises the device and reports whether any kernel of this library abandoned a wait
 * since the last call.  Returns DG_OK, or DG_ERR_DEVICE with the record in info[0..7]
 * ([0] code, [1] wait site, [2] block, [3] tile iteration, [4] K block, [5] stage) and in
 * dg_last_error().  The record is cleared. */
int dg_check_status(uint32_t info[8]);

const char* dg_last_error(void);
const char* dg_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DEEPGEMM_B200_H_ */
