// Host side of libdeepgemm_b200.so: argument checks, tile selection, tensor-map encoding and
// launches behind the C ABI declared in include/deepgemm_b200.h.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include "../../include/deepgemm_b200.h"
#include "gemm_launch.cuh"
#include "sf_pack.cuh"
#include "mega_moe.cuh"
#include "mega_moe_fused.cuh"
#include "cast_fp8.cuh"

namespace {

thread_local std::string g_last_error;

int fail(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

// The condition text may contain '%': it is passed as an argument, never as the format.
#define DG_REQUIRE(cond, ...)                                                                 \
    do {                                                                                      \
        if (!(cond)) return fail(DG_ERR_INVALID, "%s", "Assertion failed: " #cond " (" __VA_ARGS__ ")"); \
    } while (0)

#define DG_CUDA(call)                                                                                   \
    do {                                                                                                \
        cudaError_t e_ = (call);                                                                        \
        if (e_ != cudaSuccess) return fail(DG_ERR_CUDA, "CUDA error: %s at %s", cudaGetErrorString(e_), #call); \
    } while (0)

// Device status block the kernels report abandoned waits into (one per device, zero at load).
__device__ uint32_t g_status[16];

unsigned long long* g_trace = nullptr;   // clock-sample buffer for builds with DG_TRACE (tuning aid)

struct Knobs {
    std::mutex mu;
    int num_sms = 0;        // 0: use the device's count
    int tc_util = 100;
    int mk_alignment = 128;
    int timeout_ms = 2000;
    int moe_fused = 1;     // Mega MoE: one persistent kernel (1) or the kernel-per-phase path (0)
    int pdl = 0;           // launch with programmatic stream serialisation
    int force_cta_group = 0, force_block_n = 0, force_swap = 0;   // dg_debug_set_tile_override
} g_knobs;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int encode_tmap(CUtensorMap* tm, CUtensorMapDataType dtype, uint32_t rank, const void* base, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle, const char* what) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return fail(DG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t gdims[5];
    cuuint64_t gstrides[4];
    cuuint32_t bdims[5], estr[5];
    for (uint32_t i = 0; i < rank; ++i) gdims[i] = dims[i], bdims[i] = box[i], estr[i] = 1;
    for (uint32_t i = 0; i + 1 < rank; ++i) gstrides[i] = strides_bytes[i];
    if (reinterpret_cast<uintptr_t>(base) % 16 != 0)
        return fail(DG_ERR_INVALID, "Assertion failed: %s base address is 16-byte aligned", what);
    for (uint32_t i = 0; i + 1 < rank; ++i)
        if (gstrides[i] % 16 != 0)
            return fail(DG_ERR_INVALID, "Assertion failed: %s stride %llu bytes is a multiple of 16", what,
                        static_cast<unsigned long long>(gstrides[i]));
    CUresult r = fn(tm, dtype, rank, const_cast<void*>(base), gdims, gstrides, bdims, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(DG_ERR_CUDA,
                    "cuTensorMapEncodeTiled(%s) failed with %d (rank %u dims %llu,%llu,%llu box %u,%u,%u)", what,
                    static_cast<int>(r), rank, static_cast<unsigned long long>(dims[0]),
                    static_cast<unsigned long long>(rank > 1 ? dims[1] : 0),
                    static_cast<unsigned long long>(rank > 2 ? dims[2] : 0), box[0], rank > 1 ? box[1] : 0,
                    rank > 2 ? box[2] : 0);
    return DG_OK;
}

// Launch of a kernel that takes one parameter struct, with programmatic stream serialisation when the knob is on
template <class Params>
cudaError_t launch_with_pdl(void (*kernel)(const Params), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            const Params& params) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem, cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    int pdl;
    {
        std::lock_guard<std::mutex> lk(g_knobs.mu);
        pdl = g_knobs.pdl;
    }
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr, cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, params);
}

int device_sm_count(int* out) {
    static int cached[64] = {0};
    int dev = 0;
    DG_CUDA(cudaGetDevice(&dev));
    if (dev < 64 && cached[dev] != 0) {
        *out = cached[dev];
        return DG_OK;
    }
    int n = 0;
    DG_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    if (dev < 64) cached[dev] = n;
    *out = n;
    return DG_OK;
}

// --------------------------------------------------------------------------- GEMM launch
struct TileChoice {
    int ctas, bn;
    bool swap;
};

struct OperandPlan {
    CUtensorMap tm, tm_sf;
    dg::OperandParams params;
    uint32_t sf_groups;
};

// Build the tensor maps and kernel parameters of one GEMM operand in the role of R (128 rows per
// CTA) or C (`box_rows` rows per CTA).  Data maps are 3-D: (K, row inside the group, group) for a K-major operand,
// (row, K row, group) for an MN-major one; an operand without a group axis has a third extent of 1.
// sf_mn: rows of the scale tensor where they differ from the operand's (scales stored in whole 128-row blocks); 0 = same
int plan_operand(const dg_gemm_args& a, const dg_operand& op, bool is_a, uint32_t box_rows, uint32_t sf_box_rows,
                 bool mxf4, OperandPlan* out, uint32_t sf_mn = 0) {
    const uint32_t mn = is_a ? a.m : a.n;
    const bool fp4 = op.dtype == DG_E2M1_PACKED;
    const bool bf16 = op.dtype == DG_BF16;   // moved as bytes: two per element on the contiguous axis
    const bool k_grouped = a.gemm_type == DG_GEMM_K_GROUPED || a.gemm_type == DG_GEMM_K_GROUPED_PSUM;
    // Which operands carry a group axis
    uint32_t groups = 1;
    if (a.gemm_type == DG_GEMM_M_MASKED || a.gemm_type == DG_GEMM_BATCHED) groups = a.num_groups;
    if ((a.gemm_type == DG_GEMM_M_CONTIGUOUS || a.gemm_type == DG_GEMM_M_PSUM) && !is_a) groups = a.num_groups;
    dg::OperandParams& q = out->params;
    memset(&q, 0, sizeof(q));
    q.gran_k = op.gran_k;
    q.fmt = fp4 ? dg::kFmtE2M1 : dg::kFmtE4M3;
    q.mn_major = op.mn_major ? 1 : 0;
    q.batched = groups > 1 ? 1 : 0;
    out->sf_groups = 0;
    const char* name = is_a ? "a" : "b";
    int rc;
    if (!op.mn_major) {
        // K contiguous.  Packed E2M1 is seen as bytes under kind::mxf4 (two codes per byte in shared memory too) and as
        // 4-bit elements that TMA spreads to one per byte otherwise (kind::mxf8f6f4 reads 8-bit containers).
        const bool unpack = fp4 && !mxf4;
        const uint64_t k_extent = mxf4 ? static_cast<uint64_t>(a.k) / 2 : bf16 ? static_cast<uint64_t>(a.k) * 2 : static_cast<uint64_t>(a.k);
        const uint64_t batch_stride = op.batch_stride > 0 ? static_cast<uint64_t>(op.batch_stride)
                                                          : static_cast<uint64_t>(op.ld) * mn;
        const uint64_t dims[3] = {k_extent, static_cast<uint64_t>(mn), groups};
        const uint64_t strides[2] = {static_cast<uint64_t>(op.ld), batch_stride};
        const uint32_t box[3] = {128, box_rows, 1};
        rc = encode_tmap(&out->tm, unpack ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 3,
                         op.data, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B, name);
        if (rc != DG_OK) return rc;
        q.num_boxes = 1;
        q.box_bytes = box_rows * 128;
        q.box_mn = box_rows;
        q.tx_bytes = box_rows * 128 / (unpack ? 2 : 1);
        q.desc_lbo = 0, q.desc_sbo = 1024, q.desc_kstep = 32;
    } else {
        // MN contiguous (E4M3, BF16): rows of the map are K rows; K-grouped layouts stack all groups' K rows on that axis.
        // A stage holds 128 B of K per row: 128 K rows of E4M3, 64 of BF16; one box is one 128-byte-wide column of
        // swizzle atoms (128 MN elements of E4M3, 64 of BF16)
        if (fp4) return fail(DG_ERR_INVALID, "Assertion failed: packed FP4 operands are K-major (%s)", name);
        if (box_rows % 128 != 0)
            return fail(DG_ERR_INVALID, "Assertion failed: MN-major %s needs a tile of whole 128-row atoms", name);
        const uint32_t esz = bf16 ? 2 : 1, k_rows = 128 / esz, box_mn = 128 / esz;
        const uint64_t batch_stride = op.batch_stride > 0 ? static_cast<uint64_t>(op.batch_stride)
                                                          : static_cast<uint64_t>(op.ld) * a.k;
        const uint64_t dims[3] = {static_cast<uint64_t>(mn) * esz, static_cast<uint64_t>(a.k), groups};
        const uint64_t strides[2] = {static_cast<uint64_t>(op.ld), batch_stride};
        const uint32_t box[3] = {128, k_rows, 1};
        rc = encode_tmap(&out->tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, op.data, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_128B, name);
        if (rc != DG_OK) return rc;
        q.num_boxes = box_rows / box_mn;
        q.box_bytes = 128 * k_rows;
        q.box_mn = box_mn;
        q.tx_bytes = box_rows * 128;
        q.desc_lbo = 128 * k_rows, q.desc_sbo = 1024, q.desc_kstep = (32 / esz) * 128;
    }
    if (bf16) return DG_OK;   // no scale factors
    // Scale factors: int32 [groups * packed_k, mn] seen with MN innermost
    uint64_t packed_k;
    if (k_grouped) {
        // the real row count where the caller knows it (TMA then zero-fills what lies beyond, e.g. the scale row of a
        // trailing group without K rows); else an upper bound: every group may round up once
        packed_k = op.sf_k_rows > 0 ? static_cast<uint64_t>(op.sf_k_rows)
                                    : (static_cast<uint64_t>(a.k) / op.gran_k + 3 * static_cast<uint64_t>(a.num_groups)) / 4 + 1;
    } else {
        packed_k = (static_cast<uint64_t>(a.k) + op.gran_k * 4 - 1) / (op.gran_k * 4);
    }
    {
        const uint64_t dims[2] = {static_cast<uint64_t>(sf_mn > 0 ? sf_mn : mn), packed_k * groups};
        const uint64_t strides[1] = {static_cast<uint64_t>(op.sf_ld) * 4};
        const uint32_t box[2] = {sf_box_rows, mxf4 ? 2u : 1u};   // kind::mxf4: two scale words per row and stage
        rc = encode_tmap(&out->tm_sf, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, op.sf, dims, strides, box,
                         CU_TENSOR_MAP_SWIZZLE_NONE, is_a ? "sfa" : "sfb");
        if (rc != DG_OK) return rc;
        if (groups > 1) out->sf_groups = static_cast<uint32_t>(packed_k);
    }
    return DG_OK;
}

int choose_tile(const dg_gemm_args& a, int num_sms, TileChoice* t) {
    const bool m_grouped = a.gemm_type == DG_GEMM_M_CONTIGUOUS || a.gemm_type == DG_GEMM_M_PSUM ||
                           a.gemm_type == DG_GEMM_M_MASKED;
    const bool k_grouped = a.gemm_type == DG_GEMM_K_GROUPED || a.gemm_type == DG_GEMM_K_GROUPED_PSUM;
    TileChoice c;
    if (m_grouped) {
        // Tokens on the UMMA N axis: a CTA pair shares one token block of any expert.  256-token
        // tiles halve the number of UMMAs per flop; short groups shrink the UMMA N at run time.
        c.swap = true;
        c.bn = 256;
        if (a.gemm_type == DG_GEMM_M_MASKED && a.expected_m > 0 && a.expected_m <= 128) c.bn = a.expected_m <= 64 ? 64 : 128;
        if (a.gemm_type == DG_GEMM_M_CONTIGUOUS) {
            const int align = dg_get_mk_alignment_for_contiguous_layout();
            if (align % 128 != 0) c.bn = align % 64 == 0 ? 64 : 128;   // odd alignments: one unit per tile
            if (align % 256 != 0 && align % 128 == 0 && a.m < 256) c.bn = 128;
        }
        c.ctas = (a.n % 256 == 0 && num_sms % 2 == 0) ? 2 : 1;
    } else if (k_grouped) {
        c.swap = false;
        c.bn = a.n % 256 == 0 ? 256 : 128;
        c.ctas = (a.m % 256 == 0 && c.bn == 256 && num_sms % 2 == 0) ? 2 : 1;
        if (!a.b.mn_major && c.bn == 256 && a.m > 128 && num_sms % 2 == 0) c.ctas = 2;   // K-major operands (FP4 x FP4)
    } else {
        c.swap = false;
        const bool mn_major_b = a.b.mn_major != 0;
        c.ctas = (a.m > 128 && num_sms % 2 == 0) ? 2 : 1;
        c.bn = a.n >= 256 ? 256 : 128;
        if (c.ctas == 2 && c.bn == 128 && mn_major_b) c.ctas = 1;   // half tiles of an MN-major B need 128 rows
        // Weights on the UMMA M axis for the plain BF16 case with K-major operands: measured 3-5 % faster at the dense
        // configurations (4096 x 4096 x 7168: 82.9 vs 87.1 us; 8192 x 7168 x 2048: 82.9 vs 85.0 us), and the last wave's
        // token tiles can then be cut to spread over more units.  FP4 x FP4 measured faster the other way round.
        const bool both_fp4 = a.a.dtype == DG_E2M1_PACKED && a.b.dtype == DG_E2M1_PACKED;
        if (a.gemm_type == DG_GEMM_NORMAL && a.d_dtype == DG_BF16 && !a.accumulate && a.epilogue == DG_EPILOGUE_STORE &&
            !a.a.mn_major && !a.b.mn_major && a.n % 256 == 0 && a.m >= 256 && num_sms % 2 == 0 && !both_fp4)
            c.swap = true, c.ctas = 2, c.bn = 256;
    }
    {
        std::lock_guard<std::mutex> lk(g_knobs.mu);
        if (g_knobs.force_cta_group) c.ctas = g_knobs.force_cta_group;
        if (g_knobs.force_block_n) c.bn = g_knobs.force_block_n;
        if (g_knobs.force_swap) c.swap = g_knobs.force_swap == 2;
    }
    *t = c;
    return DG_OK;
}

uint32_t choose_raster(uint32_t num_m_blocks, uint32_t unit_m, uint32_t unit_n, uint32_t units) {
    uint32_t best = 1;
    uint64_t best_cost = ~0ull;
    for (uint32_t cand : {1u, 2u, 4u, 8u, 16u, 32u}) {
        if (cand > num_m_blocks && cand != 1) continue;
        const uint64_t cost = static_cast<uint64_t>(cand) * unit_m + static_cast<uint64_t>((units + cand - 1) / cand) * unit_n;
        if (cost < best_cost) best_cost = cost, best = cand;
    }
    return best;
}

}  // namespace

extern "C" {

const char* dg_last_error(void) { return g_last_error.c_str(); }
#ifdef DG_TRACE
void dg_debug_set_trace(void* device_buffer) { g_trace = static_cast<unsigned long long*>(device_buffer); }
#endif
const char* dg_version(void) { return "deepgemm_b200 0.1 (sm_100a)"; }

int dg_set_num_sms(int32_t n) {
    DG_REQUIRE(n >= 0, "num_sms");
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    g_knobs.num_sms = n;
    return DG_OK;
}
int dg_get_num_sms(void) {
    {
        std::lock_guard<std::mutex> lk(g_knobs.mu);
        if (g_knobs.num_sms > 0) return g_knobs.num_sms;
    }
    int n = 0;
    if (device_sm_count(&n) != DG_OK) return -1;
    return n;
}
int dg_set_pdl(int32_t enable) {
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    g_knobs.pdl = enable ? 1 : 0;
    return DG_OK;
}
int dg_get_pdl(void) {
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    return g_knobs.pdl;
}
int dg_set_tc_util(int32_t v) {
    DG_REQUIRE(v >= 0 && v <= 100, "tc_util");
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    g_knobs.tc_util = v;
    return DG_OK;
}
int dg_get_tc_util(void) {
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    return g_knobs.tc_util;
}
int dg_set_mk_alignment_for_contiguous_layout(int32_t v) {
    DG_REQUIRE(v > 0 && v % 16 == 0, "alignment");
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    g_knobs.mk_alignment = v;
    return DG_OK;
}
int dg_get_mk_alignment_for_contiguous_layout(void) {
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    return g_knobs.mk_alignment;
}
int dg_get_theoretical_mk_alignment_for_contiguous_layout(int32_t expected_m) {
    // UMMA N = 256 makes a fixed 256-row alignment the best choice on sm_100, whatever the expected group size
    // (csrc/jit_kernels/heuristics/runtime.hpp:57-64 of the reference; expected_m is ignored there too)
    (void)expected_m;
    return 256;
}
int dg_debug_set_tile_override(int32_t cta_group, int32_t block_n, int32_t swap) {
    DG_REQUIRE(cta_group >= 0 && cta_group <= 2 && block_n >= 0 && block_n <= 256 && swap >= 0 && swap <= 2, "tile override");
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    g_knobs.force_cta_group = cta_group, g_knobs.force_block_n = block_n, g_knobs.force_swap = swap;
    return DG_OK;
}
// Plain 16-byte loads / stores, four in flight per thread: the access pattern of the Mega MoE token pull
__global__ void __launch_bounds__(256) debug_copy_kernel(uint4* dst, const uint4* src, uint64_t n_vec) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * 256;
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    for (; i + 3 * stride < n_vec; i += 4 * stride) {
        const uint4 v0 = src[i], v1 = src[i + stride], v2 = src[i + 2 * stride], v3 = src[i + 3 * stride];
        dst[i] = v0, dst[i + stride] = v1, dst[i + 2 * stride] = v2, dst[i + 3 * stride] = v3;
    }
    for (; i < n_vec; i += stride) dst[i] = src[i];
}

int dg_debug_copy(void* dst, const void* src, int64_t bytes, void* stream) {
    DG_REQUIRE(dst != nullptr && src != nullptr && bytes >= 0 && bytes % 16 == 0, "dst / src / bytes % 16 == 0");
    DG_REQUIRE(reinterpret_cast<uintptr_t>(dst) % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0, "16-byte alignment");
    if (bytes == 0) return DG_OK;
    int num_sms = dg_get_num_sms();
    DG_REQUIRE(num_sms > 0, "num_sms");
    debug_copy_kernel<<<num_sms * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint4*>(dst), static_cast<const uint4*>(src), static_cast<uint64_t>(bytes) / 16);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}

int dg_set_wait_timeout_ms(int32_t ms) {
    DG_REQUIRE(ms > 0, "timeout");
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    g_knobs.timeout_ms = ms;
    return DG_OK;
}

int dg_check_status(uint32_t info[8]) {
    uint32_t host[16];
    DG_CUDA(cudaDeviceSynchronize());
    DG_CUDA(cudaMemcpyFromSymbol(host, g_status, sizeof(host)));
    if (info != nullptr) memcpy(info, host, 8 * sizeof(uint32_t));
    if (host[0] == dg::kStatusOk) return DG_OK;
    uint32_t zero[16] = {0};
    DG_CUDA(cudaMemcpyToSymbol(g_status, zero, sizeof(zero)));
    if (host[0] == dg::kStatusPoolOverflow)
        return fail(DG_ERR_DEVICE,
                    "Mega MoE: rank %u received %u rows but its pool holds %u (num_ring_tokens is too small); the call "
                    "was abandoned, y is not meaningful", host[2], host[3], host[4]);
    return fail(DG_ERR_DEVICE,
                "a kernel abandoned a bounded wait: code %u site %u block %u tile-iteration %u k-block %u stage %u",
                host[0], host[1], host[2], host[3], host[4], host[5]);
}

int dg_sf_pack_ue8m0(const float* sf, int32_t* out, int32_t num_batches, int32_t mn, int32_t sf_k, int32_t gran_mn,
                     int64_t stride_b, int64_t stride_mn, int64_t stride_k, const int32_t* psum_layout,
                     int32_t num_psum_groups, int32_t psum_alignment, void* stream) {
    DG_REQUIRE(sf != nullptr && out != nullptr, "sf/out");
    DG_REQUIRE(num_batches >= 0 && mn >= 0 && sf_k >= 0 && gran_mn >= 1, "shape");
    if (num_batches == 0 || mn == 0 || sf_k == 0) return DG_OK;
    DG_REQUIRE(psum_layout == nullptr || (num_psum_groups > 0 && psum_alignment > 0), "psum_layout");
    dg::SfPackParams p;
    p.sf = sf, p.out = out, p.mn = mn, p.sf_k = sf_k;
    p.packed_k = (sf_k + 3) / 4;
    p.aligned_mn = (mn + 3) / 4 * 4;
    p.gran_mn = gran_mn;
    p.stride_b = stride_b, p.stride_mn = stride_mn, p.stride_k = stride_k;
    p.psum_layout = psum_layout, p.num_psum_groups = num_psum_groups, p.psum_alignment = psum_alignment;
    DG_REQUIRE(num_batches <= 65535 && (p.packed_k + 31) / 32 <= 65535, "grid");
    dim3 grid((mn + 31) / 32, (p.packed_k + 31) / 32, num_batches);
    DG_CUDA(launch_with_pdl(dg::sf_pack_ue8m0_kernel, grid, dim3(32, 8, 1), 0, static_cast<cudaStream_t>(stream), p));
    return DG_OK;
}

int dg_per_token_cast_to_fp8(const dg_cast_args* args) {
    DG_REQUIRE(args != nullptr, "args");
    const dg_cast_args& a = *args;
    DG_REQUIRE(a.x != nullptr && a.q != nullptr && a.sf != nullptr, "x/q/sf");
    DG_REQUIRE(a.rows >= 0 && a.cols >= 0, "shape");
    DG_REQUIRE(a.gran_k == 32 || a.gran_k == 128, "gran_k");
    DG_REQUIRE(a.cols % 8 == 0 && a.ldx % 8 == 0 && a.ldx >= a.cols, "cols % 8 == 0 and ldx % 8 == 0");
    DG_REQUIRE(a.ldq % 8 == 0 && a.ldq >= a.cols, "ldq % 8 == 0");
    DG_REQUIRE(reinterpret_cast<uintptr_t>(a.x) % 16 == 0 && reinterpret_cast<uintptr_t>(a.q) % 8 == 0, "alignment of x / q");
    DG_REQUIRE(a.sf_mode >= DG_CAST_SF_FLOAT && a.sf_mode <= DG_CAST_SF_PACKED_MN_MAJOR, "sf_mode");
    if (a.rows == 0 || a.cols == 0) return DG_OK;
    const int64_t groups = (a.cols + a.gran_k - 1) / a.gran_k, words = (groups + 3) / 4;
    if (a.sf_mode == DG_CAST_SF_FLOAT) DG_REQUIRE(a.sf_ld >= groups, "sf_ld >= groups");
    if (a.sf_mode == DG_CAST_SF_PACKED_ROW_MAJOR) DG_REQUIRE(a.sf_ld >= words, "sf_ld >= packed words per row");
    if (a.sf_mode == DG_CAST_SF_PACKED_MN_MAJOR) DG_REQUIRE(a.sf_ld >= a.rows, "sf_ld >= rows");
    dg::CastParams p;
    p.x = static_cast<const __nv_bfloat16*>(a.x), p.ldx = a.ldx;
    p.rows = static_cast<uint32_t>(a.rows), p.cols = static_cast<uint32_t>(a.cols), p.gran_k = static_cast<uint32_t>(a.gran_k);
    p.q = static_cast<uint8_t*>(a.q), p.ldq = a.ldq, p.sf = a.sf, p.sf_mode = static_cast<uint32_t>(a.sf_mode), p.sf_ld = a.sf_ld;
    const uint32_t warps_per_cta = dg::kCastThreads / 32;
    int num_sms = 0;
    {
        std::lock_guard<std::mutex> lk(g_knobs.mu);
        num_sms = g_knobs.num_sms;
    }
    if (num_sms <= 0) {
        int dev = 0;
        DG_CUDA(cudaGetDevice(&dev));
        DG_CUDA(cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev));
    }
    const uint32_t want = (p.rows + warps_per_cta - 1) / warps_per_cta;
    const uint32_t grid = want < static_cast<uint32_t>(num_sms) * 8u ? want : static_cast<uint32_t>(num_sms) * 8u;
    DG_CUDA(launch_with_pdl(dg::cast_bf16_to_fp8_ue8m0_kernel, dim3(grid, 1, 1), dim3(dg::kCastThreads, 1, 1), 0,
                            static_cast<cudaStream_t>(a.stream), p));
    return DG_OK;
}

int dg_sf_pack_ue8m0_k_grouped(const float* sf, int32_t* out, const int32_t* grouped_layout, int32_t num_groups,
                               int32_t mn, int32_t sf_k_rows, int32_t packed_rows, int32_t gran_k, int32_t k_alignment,
                               int32_t use_psum, void* stream) {
    DG_REQUIRE(sf != nullptr && out != nullptr && grouped_layout != nullptr, "pointers");
    DG_REQUIRE(gran_k == 32 || gran_k == 128, "gran_k");
    DG_REQUIRE(k_alignment > 0 && k_alignment % 128 == 0, "k_alignment");
    if (packed_rows == 0 || mn == 0) return DG_OK;
    DG_REQUIRE(packed_rows <= 65535, "grid");
    dg::SfPackKGroupedParams p;
    p.sf = sf, p.out = out, p.grouped_layout = grouped_layout, p.num_groups = num_groups, p.mn = mn;
    p.sf_k_rows = sf_k_rows, p.packed_rows = packed_rows, p.gran_k = gran_k, p.k_alignment = k_alignment;
    p.use_psum = use_psum;
    dim3 grid((mn + 255) / 256, packed_rows, 1);
    DG_CUDA(launch_with_pdl(dg::sf_pack_ue8m0_k_grouped_kernel, grid, dim3(256, 1, 1), 0, static_cast<cudaStream_t>(stream), p));
    return DG_OK;
}

// Shared by dg_gemm_bs and the two expert GEMMs of dg_mega_moe_forward (moe_epi == 1, 2).
static int run_gemm(const dg_gemm_args& a, int moe_epi, const dg::MoeEpilogueParams* moe) {
    DG_REQUIRE(a.gemm_type >= DG_GEMM_NORMAL && a.gemm_type <= DG_GEMM_BATCHED, "gemm_type");
    DG_REQUIRE(a.m >= 0 && a.n >= 0 && a.k >= 0, "shape");
    if (a.m == 0 || a.n == 0) return DG_OK;
    DG_REQUIRE(a.k > 0, "k == 0 is handled by the caller");
    // BF16 operands (both, without scale factors) run the same kernel on kind::f16
    const bool bf16 = a.a.dtype == DG_BF16 || a.b.dtype == DG_BF16;
    DG_REQUIRE(!bf16 || (a.a.dtype == DG_BF16 && a.b.dtype == DG_BF16), "a and b are both BF16");
    DG_REQUIRE(a.a.data && a.b.data && (bf16 || (a.a.sf && a.b.sf)) && (a.d || moe_epi != 0), "null tensor");
    DG_REQUIRE(bf16 || a.a.dtype == DG_E4M3 || a.a.dtype == DG_E2M1_PACKED, "a dtype");
    DG_REQUIRE(bf16 || a.b.dtype == DG_E4M3 || a.b.dtype == DG_E2M1_PACKED, "b dtype");
    DG_REQUIRE(a.epilogue >= DG_EPILOGUE_STORE && a.epilogue <= DG_EPILOGUE_FP8_CAST, "epilogue");
    const bool fp8_out = a.epilogue == DG_EPILOGUE_FP8_CAST;
    DG_REQUIRE(fp8_out ? a.d_dtype == DG_E4M3 : (a.d_dtype == DG_BF16 || a.d_dtype == DG_F32), "d dtype");
    DG_REQUIRE(bf16 || a.a.gran_k == 32 || a.a.gran_k == 128, "gran_k of a");
    DG_REQUIRE(bf16 || a.b.gran_k == 32 || a.b.gran_k == 128, "gran_k of b");
    if (bf16) {
        DG_REQUIRE(moe_epi == 0 && a.epilogue != DG_EPILOGUE_FP8_CAST, "BF16 operands take the store and stochastic-rounding epilogues");
        DG_REQUIRE(a.gemm_type != DG_GEMM_BATCHED, "batched GEMMs take FP8 operands");
        DG_REQUIRE(a.a.ld % 16 == 0 && a.b.ld % 16 == 0, "leading dimensions are multiples of 16 bytes");
    }
    // Both operands packed E2M1: the dedicated kind::mxf4 path (K-major, one scale per 32 elements)
    const bool mxf4 = a.a.dtype == DG_E2M1_PACKED && a.b.dtype == DG_E2M1_PACKED;
    if (mxf4) {
        DG_REQUIRE(!a.a.mn_major && !a.b.mn_major, "major_a == cute::UMMA::Major::K and major_b == cute::UMMA::Major::K");
        DG_REQUIRE(a.a.gran_k == 32 && a.b.gran_k == 32, "FP4 x FP4 takes 1 x 32 scales on both sides");
        DG_REQUIRE(moe_epi == 0 && a.epilogue == DG_EPILOGUE_STORE, "FP4 x FP4 has the plain epilogue only");
    }
    const bool grouped = a.gemm_type != DG_GEMM_NORMAL;
    const bool batched = a.gemm_type == DG_GEMM_BATCHED;
    DG_REQUIRE(!grouped || a.num_groups > 0, "num_groups");
    DG_REQUIRE(!grouped || batched || a.grouped_layout != nullptr, "grouped_layout");
    const bool k_grouped = a.gemm_type == DG_GEMM_K_GROUPED || a.gemm_type == DG_GEMM_K_GROUPED_PSUM;
    const bool m_grouped = grouped && !k_grouped && !batched;
    // K-grouped: A^T B over MN-major E4M3 operands, or (FP4 x FP4) A B^T over K-major ones whose K axis holds the groups
    DG_REQUIRE(!k_grouped || a.a.gran_k == a.b.gran_k, "k-grouped scale granularities match");
    DG_REQUIRE(!k_grouped || mxf4 || (a.a.mn_major && a.b.mn_major), "k-grouped FP8 operands are MN-major");
    DG_REQUIRE(!m_grouped || !a.a.mn_major, "m-grouped A is K-major");
    DG_REQUIRE(!m_grouped || a.d_dtype == DG_BF16, "m-grouped D is BF16");
    DG_REQUIRE(a.a.dtype != DG_E2M1_PACKED || a.k % 128 == 0, "FP4 K is a multiple of 128");
    DG_REQUIRE(a.b.dtype != DG_E2M1_PACKED || a.k % 128 == 0, "FP4 K is a multiple of 128");
    if (a.epilogue != DG_EPILOGUE_STORE) {
        DG_REQUIRE(a.gemm_type == DG_GEMM_NORMAL || batched, "value epilogues belong to the dense and batched GEMMs");
        DG_REQUIRE(!a.accumulate && a.alpha == 1.0f, "value epilogues write D directly");
        DG_REQUIRE(a.epilogue != DG_EPILOGUE_STOCHASTIC_BF16 || a.d_dtype == DG_BF16, "stochastic rounding writes BF16");
    }
    if (fp8_out) {
        DG_REQUIRE(a.sfd != nullptr && a.sfd_ld > 0, "sfd");
        DG_REQUIRE(a.n % 128 == 0, "n % 128 == 0");
        DG_REQUIRE(a.clamp_value >= 0.0f, "clamp_value > 0");
    }

    int num_sms = dg_get_num_sms();
    DG_REQUIRE(num_sms > 0, "num_sms");
    TileChoice t;
    choose_tile(a, num_sms, &t);
    if (moe_epi != 0) {
        std::lock_guard<std::mutex> lk(g_knobs.mu);
        t.swap = true, t.bn = g_knobs.force_block_n ? g_knobs.force_block_n : 256;
        if (!g_knobs.force_cta_group) t.ctas = (a.n % 256 == 0 && num_sms % 2 == 0) ? 2 : 1;   // a CTA pair splits the weight rows
    }
    if (a.epilogue != DG_EPILOGUE_STORE) t.swap = false;
    DG_REQUIRE(t.ctas == 1 || t.ctas == 2, "cta group");
    DG_REQUIRE(!(t.swap && a.d_dtype == DG_F32), "swapped tiles write BF16 only");
    DG_REQUIRE(!(t.swap && a.accumulate), "swapped tiles do not accumulate");

    const uint32_t unit_m = t.swap ? t.bn : 128 * t.ctas;
    const uint32_t unit_n = t.swap ? 128 * t.ctas : t.bn;
    uint32_t split_blocks = 0;
    if (a.gemm_type == DG_GEMM_M_CONTIGUOUS) {
        // Tiles must not mix experts: a tile is one alignment unit, or two units that are split
        // on the device where they belong to different experts.
        const int align = dg_get_mk_alignment_for_contiguous_layout();
        DG_REQUIRE(align > 0 && align % 32 == 0, "group alignment is a multiple of 32");
        if (align % static_cast<int>(unit_m) != 0) {
            DG_REQUIRE(t.swap && unit_m % 2 == 0 && align % static_cast<int>(unit_m / 2) == 0,
                       "group alignment is a multiple of half the token tile");
            split_blocks = 1;
        }
    }
    if (a.gemm_type == DG_GEMM_M_PSUM) DG_REQUIRE(a.alignment > 0 && a.alignment % 32 == 0, "psum alignment");
    if (a.gemm_type == DG_GEMM_M_PSUM || a.gemm_type == DG_GEMM_M_MASKED)
        DG_REQUIRE(t.swap, "psum / masked layouts run with swapped operands");
    if (k_grouped) DG_REQUIRE(a.alignment > 0 && a.alignment % (mxf4 ? 256 : 128) == 0, "k alignment");

    // Operand roles
    const dg_operand& op_r = t.swap ? a.b : a.a;
    const dg_operand& op_c = t.swap ? a.a : a.b;
    const uint32_t c_rows_per_cta = t.bn / t.ctas;
    const uint32_t sfc_rows = (t.bn + 127) / 128 * 128;
    OperandPlan plan_r, plan_c;
    int rc = plan_operand(a, op_r, /*is_a=*/!t.swap, 128, 128, mxf4, &plan_r);
    if (rc != DG_OK) return rc;
    // The fused Mega MoE epilogues read token scales stored in tcgen05.cp order, 128 rows to a block: a token's word
    // may lie anywhere inside its block, so the map covers whole blocks
    const uint32_t sfc_mn = moe_epi != 0 ? (static_cast<uint32_t>(a.m) + 127u) / 128u * 128u : 0u;
    rc = plan_operand(a, op_c, /*is_a=*/t.swap, c_rows_per_cta, sfc_rows, mxf4, &plan_c, sfc_mn);
    if (rc != DG_OK) return rc;

    dg::GemmLaunch launch;
    memset(&launch, 0, sizeof(launch));
    dg::GemmParams& p = launch.p;
    p.tm_r = plan_r.tm, p.tm_c = plan_c.tm, p.tm_sfr = plan_r.tm_sf, p.tm_sfc = plan_c.tm_sf;
    if (t.swap && !op_c.mn_major && (op_c.dtype == DG_E4M3 || mxf4 || bf16) && c_rows_per_cta == 128) {
        // narrower views of the token operand for ragged tiles
        for (int i = 0; i < 2; ++i) {
            OperandPlan small;
            rc = plan_operand(a, op_c, /*is_a=*/true, i == 0 ? 32 : 64, sfc_rows, mxf4, &small);
            if (rc != DG_OK) return rc;
            p.tm_c_small[i] = small.tm;
        }
        p.c_small = 1;
    }
    p.r = plan_r.params, p.c = plan_c.params;
    p.sf_groups_r = plan_r.sf_groups, p.sf_groups_c = plan_c.sf_groups;
    p.gemm_type = a.gemm_type;
    p.m = a.m, p.n = a.n, p.k = a.k;
    p.num_groups = grouped ? a.num_groups : 1;
    p.alignment = a.alignment > 0 ? a.alignment : 128;
    p.grouped_layout = a.grouped_layout;
    p.num_m_blocks = (a.m + unit_m - 1) / unit_m;
    p.num_n_blocks = (a.n + unit_n - 1) / unit_n;
    p.alpha = a.alpha;
    p.accumulate = a.accumulate ? 1 : 0;
    p.d_grouped = (a.gemm_type == DG_GEMM_M_MASKED || k_grouped || batched) ? 1 : 0;
    p.split_blocks = split_blocks;
    p.skip_padding = a.skip_padding_rows ? 1 : 0;
    {
        std::lock_guard<std::mutex> lk(g_knobs.mu);
        p.timeout_ms = g_knobs.timeout_ms;
        launch.pdl = g_knobs.pdl;
    }
    void* status_ptr = nullptr;
    DG_CUDA(cudaGetSymbolAddress(&status_ptr, g_status));
    p.status = static_cast<uint32_t*>(status_ptr);
    p.trace = g_trace;

    if (moe_epi != 0) {
        p.moe = *moe;
        p.r_sf_pretransposed = 1;
        p.c_sf_pretransposed = 1;
    }
    cudaStream_t stream = static_cast<cudaStream_t>(a.stream);
    if (fp8_out) {
        p.cast.sfd = reinterpret_cast<uint32_t*>(a.sfd);
        p.cast.sfd_ld = a.sfd_ld;
        // the kernel compares BF16 values with the BF16-rounded bound (torch compares a BF16 tensor with a scalar so)
        p.cast.clamp_bound = a.clamp_value > 0.0f ? __bfloat162float(__float2bfloat16_rn(a.clamp_value)) : INFINITY;
        p.cast.clamped_count = a.clamp_value > 0.0f ? a.clamped_count : nullptr;
        // the count replaces the word's previous contents: cleared in stream order before the launch
        if (a.clamped_count != nullptr) DG_CUDA(cudaMemsetAsync(a.clamped_count, 0, sizeof(uint32_t), stream));
    }
    // D: [groups, m, n] row-major
    if (moe_epi == 0) {
        const uint32_t es = a.d_dtype == DG_F32 ? 4 : (fp8_out ? 1 : 2);
        const uint64_t d_groups = p.d_grouped ? a.num_groups : 1;
        const uint64_t d_batch = a.d_batch_stride > 0 ? static_cast<uint64_t>(a.d_batch_stride) : static_cast<uint64_t>(a.ldd) * a.m;
        const uint64_t dims[3] = {static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.m), d_groups};
        const uint64_t strides[2] = {static_cast<uint64_t>(a.ldd), d_batch};
        uint32_t box[3];
        CUtensorMapSwizzle sw;
        if (t.swap) {
            box[0] = 32, box[1] = 32, box[2] = 1, sw = CU_TENSOR_MAP_SWIZZLE_NONE;
        } else if (fp8_out) {
            box[0] = 64, box[1] = 32, box[2] = 1, sw = CU_TENSOR_MAP_SWIZZLE_NONE;
        } else {
            box[0] = 128 / es, box[1] = 32, box[2] = 1, sw = CU_TENSOR_MAP_SWIZZLE_128B;
        }
        const CUtensorMapDataType dt = a.d_dtype == DG_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                       : fp8_out            ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                                            : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        rc = encode_tmap(&p.tm_d, dt, 3, a.d, dims, strides, box, sw, "d");
        if (rc != DG_OK) return rc;
        if (t.swap) {
            box[1] = 16;
            rc = encode_tmap(&p.tm_d_half, dt, 3, a.d, dims, strides, box, sw, "d");
            if (rc != DG_OK) return rc;
        }
    }

    // Grid: persistent units, never more than there are tiles (when the host can know)
    uint32_t units = static_cast<uint32_t>(num_sms) / t.ctas;
    uint64_t tiles = static_cast<uint64_t>(p.num_m_blocks) * p.num_n_blocks;
    if (k_grouped || batched) tiles *= a.num_groups;
    if (a.gemm_type == DG_GEMM_M_MASKED) tiles *= a.num_groups;   // upper bound: m = max rows per group
    uint64_t slots = tiles;
    if (a.gemm_type == DG_GEMM_NORMAL && t.swap && moe_epi == 0 && a.m % static_cast<int>(unit_m) == 0 && unit_m == 256) {
        // The last wave (or the only one): when fewer than half (a quarter) of the units would have a tile, its token
        // tiles are cut in two (four) parts: a half tile costs more than half a tile, but the wave ends sooner.
        const uint32_t tail = static_cast<uint32_t>(tiles % units);
        if (tail != 0) {
            const uint32_t split = tail * 4 <= units ? 4u : tail * 2 <= units ? 2u : 1u;
            if (split > 1) {
                p.tail_first = static_cast<uint32_t>(tiles) - tail, p.tail_split = split;
                slots = tiles - tail + static_cast<uint64_t>(tail) * split;
            }
        }
    }
    if (a.gemm_type != DG_GEMM_M_PSUM && slots < units) units = static_cast<uint32_t>(slots);
    DG_REQUIRE(units > 0, "empty grid");
    p.num_units = units;
    p.raster = choose_raster(p.num_m_blocks, unit_m, unit_n, units);
    // M-grouped layouts whose weights of one group fit L2 comfortably walk the n blocks of a token block first: all of
    // the group's weight blocks stay hot and each token block is read from DRAM exactly once.  Measured on the grouped
    // headline shape (8 x ~8192 x 4096 x 7168, 29 MB of weights per group): DRAM reads 0.96 GB against 1.44 GB with
    // super-rows of eight token blocks, 3 % faster.  (K-grouped shapes measured 5 % slower that way; dense ones equal.)
    if (m_grouped && static_cast<uint64_t>(a.n) * static_cast<uint64_t>(a.k) <= (40ull << 20)) p.raster = 1;
    launch.stream = stream, launch.units = units;
    launch.ctas = t.ctas, launch.bn = t.bn, launch.swap = t.swap, launch.f32 = a.d_dtype == DG_F32;
    launch.epi = moe_epi != 0 ? moe_epi : a.epilogue == DG_EPILOGUE_STOCHASTIC_BF16 ? dg::kEpiStochastic
                 : fp8_out                                                          ? dg::kEpiFp8Cast
                                                                                    : dg::kEpiStore;
    launch.kind = mxf4 ? dg::kKindMxf4 : bf16 ? dg::kKindBf16 : dg::kKindMxf8f6f4;
    int lrc = mxf4 ? dg::dispatch_gemm_mxf4(launch)
              : bf16 ? dg::dispatch_gemm_bf16(launch)
              : moe_epi != 0 ? dg::dispatch_gemm_moe(launch)
              : launch.epi != dg::kEpiStore ? dg::dispatch_gemm_epi(launch)
                                            : dg::dispatch_gemm_plain(launch);
    if (lrc == dg::kLaunchNoKernel)
        return fail(DG_ERR_INVALID, "no kernel built for cta_group %d, block_n %d, swap %d, f32 %d, epilogue %d, kind %d",
                    t.ctas, t.bn, static_cast<int>(t.swap), static_cast<int>(launch.f32), launch.epi, launch.kind);
    if (lrc != 0)
        return fail(DG_ERR_CUDA, "CUDA error: %s launching the GEMM kernel", cudaGetErrorString(static_cast<cudaError_t>(lrc)));
    return DG_OK;
}


int dg_gemm_bs(const dg_gemm_args* args) {
    DG_REQUIRE(args != nullptr, "args");
    return run_gemm(*args, 0, nullptr);
}

// --------------------------------------------------------------------------- Mega MoE
static int check_moe_config(const dg_moe_config& c) {
    DG_REQUIRE(c.num_ranks > 0 && c.num_ranks <= static_cast<int>(dg::kMoeMaxRanks), "num_ranks");
    DG_REQUIRE(c.num_experts > 0 && c.num_experts % c.num_ranks == 0, "num_experts % num_ranks == 0");
    DG_REQUIRE(c.num_experts <= static_cast<int>(dg::kMoeMaxExperts), "num_experts <= 4032");
    DG_REQUIRE(c.num_topk > 0 && c.num_topk <= c.num_experts, "num_topk");
    DG_REQUIRE(c.num_max_tokens_per_rank > 0, "num_max_tokens_per_rank");
    DG_REQUIRE(c.num_ring_tokens >= 0, "num_ring_tokens >= 0");
    DG_REQUIRE(c.num_shared_experts >= 0 && c.num_shared_experts <= 64, "num_shared_experts >= 0");
    DG_REQUIRE(c.hidden > 0 && c.hidden % 128 == 0 && c.intermediate_hidden > 0 && c.intermediate_hidden % 128 == 0,
               "hidden % 128 == 0 and intermediate_hidden % 128 == 0");
    return DG_OK;
}


// Epilogue arguments and the two expert GEMMs' descriptions, shared by both Mega MoE paths.
static void fill_moe_gemm_args(const dg_moe_args& m, const dg::MoeArgs& a, dg::MoeEpilogueParams* e, dg_gemm_args* g1,
                               dg_gemm_args* g2) {
    const dg::MoeLayout& L = a.L;
    uint8_t* mine = a.base[m.rank];
    memset(e, 0, sizeof(*e));
    e->l2_acts = mine + L.off_l2_acts, e->l2_sf = mine + L.off_l2_sf;
    e->pool_w = reinterpret_cast<const float*>(mine + L.off_pool_w);
    e->pool_meta = reinterpret_cast<const int32_t*>(mine + L.off_pool_meta);
    for (uint32_t r = 0; r < L.ranks; ++r) e->peer_base[r] = a.base[r];
    e->off_combine = L.off_combine, e->pool_rows = L.pool_rows, e->sf_ld = L.pool_rows, e->inter = L.inter, e->hidden = L.hidden, e->t_max = L.t_max;
    e->clamp = m.activation_clamp, e->fast_math = m.fast_math ? 1 : 0;
    e->activation = static_cast<uint32_t>(m.activation);
    e->post_down = m.post_down ? 1u : 0u;
    e->situ_beta = m.situ_beta > 0.0f ? m.situ_beta : 1.0f;
    e->situ_linear_beta = m.situ_linear_beta > 0.0f ? m.situ_linear_beta : INFINITY;
    dg_gemm_args g;
    memset(&g, 0, sizeof(g));
    g.gemm_type = DG_GEMM_M_PSUM, g.num_groups = L.experts_local, g.alignment = dg::kMoePoolAlign;
    g.grouped_layout = reinterpret_cast<const int32_t*>(mine + L.off_work) + dg::MoeWork::psum_end();
    g.stream = m.stream, g.alpha = 1.0f, g.d_dtype = DG_BF16;
    g.m = L.pool_rows, g.n = 2 * L.inter, g.k = L.hidden;
    g.a.data = mine + L.off_l1_acts, g.a.sf = reinterpret_cast<const int32_t*>(mine + L.off_l1_sf);
    g.a.ld = L.hidden, g.a.sf_ld = L.pool_rows, g.a.dtype = DG_E4M3, g.a.gran_k = 32;
    const int wdiv = m.weights_fp8 ? 1 : 2;   // weight bytes per row: K, or K / 2 for packed FP4
    g.b.data = m.l1_w, g.b.sf = m.l1_sf, g.b.ld = L.hidden / wdiv, g.b.sf_ld = m.l1_sf_ld;
    g.b.dtype = m.weights_fp8 ? DG_E4M3 : DG_E2M1_PACKED;
    g.b.gran_k = 32;
    *g1 = g;
    g.n = L.hidden, g.k = L.inter;
    g.a.data = mine + L.off_l2_acts, g.a.sf = reinterpret_cast<const int32_t*>(mine + L.off_l2_sf), g.a.ld = L.inter;
    g.b.data = m.l2_w, g.b.sf = m.l2_sf, g.b.ld = L.inter / wdiv, g.b.sf_ld = m.l2_sf_ld;
    *g2 = g;
}

// SMs the persistent Mega MoE grid may take: the num_sms knob (at most the device's SMs: every CTA must be resident at
// the same time for the kernel's grid barrier) minus DG_MEGA_MOE_SM_HEADROOM rounded up to even, which leaves room for
// kernels of other streams that run beside it (csrc/jit_kernels/impls/runtime_utils.hpp:35-82 of the reference).
static int mega_moe_num_sms(int* out) {
    int num_sms = dg_get_num_sms();
    DG_REQUIRE(num_sms > 0, "num_sms");
    int device_sms = 0;
    if (device_sm_count(&device_sms) == DG_OK && device_sms > 0 && num_sms > device_sms) num_sms = device_sms;
    int headroom = 0;
    if (const char* env = getenv("DG_MEGA_MOE_SM_HEADROOM")) headroom = atoi(env);
    DG_REQUIRE(headroom >= 0, "DG_MEGA_MOE_SM_HEADROOM must be non-negative");
    headroom = (headroom + 1) / 2 * 2;
    DG_REQUIRE(headroom < num_sms, "DG_MEGA_MOE_SM_HEADROOM leaves no SMs for the mega-MoE grid");
    num_sms -= headroom;
    DG_REQUIRE(num_sms % 2 == 0, "num_sms % 2 == 0");
    *out = num_sms;
    return DG_OK;
}

// Shared experts: two dense GEMMs over this rank's own tokens with the fused epilogues of the routed path (gated
// activation + requantisation without a route weight; BF16 rows written to plane `topk` of this rank's combine
// buffer), enqueued ahead of the routed forward, whose reduction adds that plane first.
static int run_shared_experts(const dg_moe_args& m, const dg::MoeArgs& a) {
    const dg::MoeLayout& L = a.L;
    DG_REQUIRE(m.shared_l1_w && m.shared_l1_sf && m.shared_l2_w && m.shared_l2_sf, "shared expert weights");
    DG_REQUIRE(!m.post_down, "shared experts take route_weight_mode pre_down");
    if (m.num_tokens == 0) return DG_OK;
    cudaStream_t stream = static_cast<cudaStream_t>(m.stream);
    uint8_t* mine = a.base[m.rank];
    const uint32_t t_al = (L.t_max + 127) / 128 * 128, inter_s = L.shared * L.inter;
    dg::moe_shared_meta_kernel<<<(t_al + 255) / 256, 256, 0, stream>>>(a);
    DG_CUDA(cudaGetLastError());
    dg::MoeEpilogueParams e;
    dg_gemm_args unused1, unused2;
    fill_moe_gemm_args(m, a, &e, &unused1, &unused2);
    e.l2_acts = mine + L.off_shared_l2_acts, e.l2_sf = mine + L.off_shared_l2_sf;
    e.pool_w = reinterpret_cast<const float*>(mine + L.off_topk_w);   // read into the per-tile table, never applied
    e.pool_meta = reinterpret_cast<const int32_t*>(mine + L.off_shared_meta);
    e.pool_rows = t_al, e.sf_ld = t_al, e.inter = inter_s;
    dg_gemm_args g;
    memset(&g, 0, sizeof(g));
    g.gemm_type = DG_GEMM_NORMAL, g.num_groups = 1, g.stream = m.stream, g.alpha = 1.0f, g.d_dtype = DG_BF16;
    g.m = m.num_tokens, g.n = 2 * static_cast<int32_t>(inter_s), g.k = L.hidden;
    g.a.data = mine + L.off_x, g.a.sf = reinterpret_cast<const int32_t*>(mine + L.off_shared_sf);
    g.a.ld = L.hidden, g.a.sf_ld = t_al, g.a.dtype = DG_E4M3, g.a.gran_k = 32;
    g.b.data = m.shared_l1_w, g.b.sf = m.shared_l1_sf, g.b.ld = L.hidden, g.b.sf_ld = m.shared_l1_sf_ld;
    g.b.dtype = DG_E4M3, g.b.gran_k = 32;
    dg::MoeEpilogueParams e1 = e;
    e1.post_down = 1;          // first GEMM: no route weight on the activation
    int rc = run_gemm(g, 1, &e1);
    if (rc != DG_OK) return rc;
    g.n = L.hidden, g.k = static_cast<int32_t>(inter_s);
    g.a.data = mine + L.off_shared_l2_acts, g.a.sf = reinterpret_cast<const int32_t*>(mine + L.off_shared_l2_sf), g.a.ld = inter_s;
    g.b.data = m.shared_l2_w, g.b.sf = m.shared_l2_sf, g.b.ld = inter_s, g.b.sf_ld = m.shared_l2_sf_ld;
    dg::MoeEpilogueParams e2 = e;
    e2.post_down = 0;          // second GEMM: rows go to the combine plane as they are
    return run_gemm(g, 2, &e2);
}

static int launch_moe_fused(const dg_moe_args& m, const dg::MoeArgs& a, int num_sms) {
    dg::MoeFusedParams p;
    memset(&p, 0, sizeof(p));
    p.a = a;
    dg_gemm_args g[2];
    fill_moe_gemm_args(m, a, &p.e, &g[0], &g[1]);
    p.e.sf_ld = a.L.sf_rows;
    for (int i = 0; i < 2; ++i) {
        // weights are the UMMA row operand (128 rows per CTA), tokens the column operand (half a token tile per CTA)
        OperandPlan w, act;
        int rc = plan_operand(g[i], g[i].b, /*is_a=*/false, 128, 128, false, &w);
        if (rc != DG_OK) return rc;
        rc = plan_operand(g[i], g[i].a, /*is_a=*/true, dg::FusedCfg::BN / 2, 256, false, &act);
        if (rc != DG_OK) return rc;
        // the tokens' scale words: 256 rows per token tile, tile after tile
        dg_gemm_args gs = g[i];
        gs.m = a.L.sf_rows, gs.a.sf_ld = a.L.sf_rows;
        OperandPlan act_sf;
        rc = plan_operand(gs, gs.a, /*is_a=*/true, 32, 256, false, &act_sf);
        if (rc != DG_OK) return rc;
        p.tm_w[i] = w.tm, p.tm_wsf[i] = w.tm_sf, p.tm_act[i] = act.tm, p.tm_actsf[i] = act_sf.tm_sf;
        for (int j = 0; j < 2; ++j) {
            OperandPlan small;
            rc = plan_operand(g[i], g[i].a, /*is_a=*/true, j == 0 ? 32 : 64, 256, false, &small);
            if (rc != DG_OK) return rc;
            p.tm_act_small[i][j] = small.tm;
        }
    }
    p.y = static_cast<__nv_bfloat16*>(m.y), p.ldy = m.ldy;
    p.w_fp8 = m.weights_fp8 ? 1u : 0u;
    p.num_ctas = static_cast<uint32_t>(num_sms) / 2 * 2;
    p.trace = g_trace;
    p.lag = 8;
    DG_CUDA(cudaFuncSetAttribute(dg::mega_moe_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(dg::FusedCfg::kSmemBytes)));
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(p.num_ctas, 1, 1), cfg.blockDim = dim3(dg::kFusedThreads, 1, 1);
    cfg.dynamicSmemBytes = dg::FusedCfg::kSmemBytes, cfg.stream = static_cast<cudaStream_t>(m.stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr, cfg.numAttrs = 1;
    DG_CUDA(cudaLaunchKernelEx(&cfg, dg::mega_moe_fused_kernel, p));
    return DG_OK;
}

int dg_set_mega_moe_fused(int32_t enable) {
    std::lock_guard<std::mutex> lk(g_knobs.mu);
    g_knobs.moe_fused = enable ? 1 : 0;
    return DG_OK;
}

int dg_get_token_alignment_for_mega_moe(void) { return 128; }
int dg_get_block_m_for_mega_moe(void) { return static_cast<int>(dg::kMoeTileRows); }

int dg_get_mega_moe_num_sms(void) {
    int n = 0;
    return mega_moe_num_sms(&n) == DG_OK ? n : -1;
}

int dg_mega_moe_buffer_layout(const dg_moe_config* cfg, dg_moe_layout* out) {
    DG_REQUIRE(cfg != nullptr && out != nullptr, "null argument");
    int rc = check_moe_config(*cfg);
    if (rc != DG_OK) return rc;
    DG_REQUIRE(cfg->num_max_tokens_per_rank % dg_get_token_alignment_for_mega_moe() == 0, "token alignment");
    const dg::MoeLayout L = dg::make_moe_layout(cfg->num_ranks, cfg->num_experts, cfg->num_max_tokens_per_rank,
                                                cfg->num_topk, cfg->hidden, cfg->intermediate_hidden, cfg->num_ring_tokens,
                                                cfg->num_shared_experts);
    out->num_bytes = static_cast<int64_t>(L.total_bytes);
    out->pool_rows = static_cast<int64_t>(L.pool_rows);
    out->off_x = L.off_x, out->off_x_sf = L.off_x_sf, out->off_topk_idx = L.off_topk_idx;
    out->off_topk_weights = L.off_topk_w, out->off_l1_acts = L.off_l1_acts, out->off_l1_acts_sf = L.off_l1_sf;
    out->off_l2_acts = L.off_l2_acts, out->off_l2_acts_sf = L.off_l2_sf, out->off_token_src_metadata = L.off_pool_meta;
    out->off_combine = L.off_combine;
    out->off_shared_l1_acts_sf = L.off_shared_sf, out->off_shared_l2_acts = L.off_shared_l2_acts;
    out->off_shared_l2_acts_sf = L.off_shared_l2_sf;
    out->sf_rows = static_cast<int64_t>(L.sf_rows);
    return DG_OK;
}

int dg_mega_moe_forward(const dg_moe_args* args) {
    DG_REQUIRE(args != nullptr, "args");
    const dg_moe_args& m = *args;
    int rc = check_moe_config(m.cfg);
    if (rc != DG_OK) return rc;
    DG_REQUIRE(m.rank >= 0 && m.rank < m.cfg.num_ranks, "rank");
    DG_REQUIRE(m.num_tokens >= 0 && m.num_tokens <= m.cfg.num_max_tokens_per_rank, "num_tokens <= num_max_tokens_per_rank");
    DG_REQUIRE(m.buffer_ptrs != nullptr && m.y != nullptr, "null argument");
    DG_REQUIRE(m.l1_w && m.l1_sf && m.l2_w && m.l2_sf, "null weights");
    DG_REQUIRE(m.activation >= DG_ACT_SWIGLU && m.activation <= DG_ACT_SITU, "activation");
    const dg::MoeLayout L = dg::make_moe_layout(m.cfg.num_ranks, m.cfg.num_experts, m.cfg.num_max_tokens_per_rank,
                                                m.cfg.num_topk, m.cfg.hidden, m.cfg.intermediate_hidden, m.cfg.num_ring_tokens,
                                                m.cfg.num_shared_experts);
    dg::MoeArgs a;
    memset(&a, 0, sizeof(a));
    a.L = L;
    for (int r = 0; r < m.cfg.num_ranks; ++r) {
        DG_REQUIRE(m.buffer_ptrs[r] != nullptr, "buffer_ptrs[r]");
        a.base[r] = static_cast<uint8_t*>(m.buffer_ptrs[r]);
    }
    a.rank = m.rank, a.num_tokens = m.num_tokens;
    {
        std::lock_guard<std::mutex> lk(g_knobs.mu);
        a.timeout_ms = g_knobs.timeout_ms;
    }
    void* status_ptr = nullptr;
    DG_CUDA(cudaGetSymbolAddress(&status_ptr, g_status));
    a.status = static_cast<uint32_t*>(status_ptr);
    a.stats = m.stats;
    cudaStream_t stream = static_cast<cudaStream_t>(m.stream);
    int num_sms = 0;
    rc = mega_moe_num_sms(&num_sms);
    if (rc != DG_OK) return rc;
    bool fused;
    {
        std::lock_guard<std::mutex> lk(g_knobs.mu);
        fused = g_knobs.moe_fused != 0;
    }
    fused = fused && L.hidden % 256 == 0 && L.inter % 128 == 0 && L.experts_local * L.ranks <= dg::FusedCfg::kMaxSegments &&
            num_sms >= 2;
    if (L.shared != 0) {
        rc = run_shared_experts(m, a);
        if (rc != DG_OK) return rc;
    }
    if (fused) return launch_moe_fused(m, a, num_sms);

    // 1. count + index scatter, 2. count exchange + barrier + pool layout, 3. pull
    const uint32_t pairs = static_cast<uint32_t>(m.num_tokens) * L.topk;
    if (pairs > 0) dg::moe_scatter_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(a);
    dg::moe_exchange_kernel<<<1, 256, 0, stream>>>(a);
    const uint32_t seg_smem = (L.experts_local * L.ranks + 1) * 4;
    dg::moe_pull_kernel<<<num_sms * 4, 256, seg_smem, stream>>>(a);
    DG_CUDA(cudaGetLastError());

    // 4. first expert GEMM (+ SwiGLU, route weight, FP8 requantisation), 5. second (+ combine push)
    dg::MoeEpilogueParams e;
    dg_gemm_args g1, g2;
    fill_moe_gemm_args(m, a, &e, &g1, &g2);
    rc = run_gemm(g1, 1, &e);
    if (rc != DG_OK) return rc;
    rc = run_gemm(g2, 2, &e);
    if (rc != DG_OK) return rc;

    // 6. every rank has pushed its results, 7. local top-k reduction
    dg::moe_barrier_kernel<<<1, 32, 0, stream>>>(a);
    if (m.num_tokens > 0)
        dg::moe_reduce_kernel<<<m.num_tokens, 128, 0, stream>>>(a, static_cast<__nv_bfloat16*>(m.y), m.ldy);
    DG_CUDA(cudaGetLastError());
    return DG_OK;
}


// --------------------------------------------------------------------------- no-allocation entry point
// Scratch for dg_gemm_fp8_fp32sf_noalloc: the packed UE8M0 scale tensors of both operands live here instead
// of in caller-allocated memory.  One copy per GPU that loads the library, held until the process exits.
constexpr size_t kNoAllocScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// `g_noalloc_scratch` is a host-side stand-in in host code, not a device address: the address the kernels
// get comes from cudaGetSymbolAddress, asked once per device with that device current.
static int noalloc_scratch_address(unsigned char** out) {
    static std::mutex mu;
    static unsigned char* cached[64] = {nullptr};
    int dev = 0;
    DG_CUDA(cudaGetDevice(&dev));
    DG_REQUIRE(dev >= 0 && dev < 64, "device index");
    std::lock_guard<std::mutex> lk(mu);
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        DG_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_scratch));
        cached[dev] = static_cast<unsigned char*>(ptr);
    }
    *out = cached[dev];
    return DG_OK;
}

int dg_noalloc_scratch_bytes(void) { return static_cast<int>(kNoAllocScratchBytes); }

int dg_gemm_fp8_fp32sf_noalloc(const dg_gemm_noalloc_args* args) {
    DG_REQUIRE(args != nullptr, "args");
    const dg_gemm_noalloc_args& a = *args;
    DG_REQUIRE(a.m >= 0 && a.n >= 0 && a.k > 0, "shape");
    if (a.m == 0 || a.n == 0) return DG_OK;
    DG_REQUIRE(a.a && a.sfa && a.b && a.sfb && a.d, "null tensor");
    DG_REQUIRE(a.gran_k == 32 || a.gran_k == 128, "gran_k");
    DG_REQUIRE(a.gran_mn_b == 1 || a.gran_mn_b == 128, "gran_mn_b");
    DG_REQUIRE(a.d_dtype == DG_BF16 || a.d_dtype == DG_F32, "d dtype");
    const int64_t sf_k = (static_cast<int64_t>(a.k) + a.gran_k - 1) / a.gran_k;
    const int64_t packed_k = (sf_k + 3) / 4;
    const int64_t amn_a = (static_cast<int64_t>(a.m) + 3) / 4 * 4, amn_b = (static_cast<int64_t>(a.n) + 3) / 4 * 4;
    // Both packed scale tensors, each starting on a 256-byte boundary
    const int64_t bytes_a = (packed_k * amn_a * 4 + 255) / 256 * 256, bytes_b = packed_k * amn_b * 4;
    if (bytes_a + bytes_b > static_cast<int64_t>(kNoAllocScratchBytes))
        return fail(DG_ERR_INVALID,
                    "dg_gemm_fp8_fp32sf_noalloc: the packed scales of m=%d n=%d k=%d need %lld bytes, the built-in "
                    "scratch holds %zu; use dg_sf_pack_ue8m0 + dg_gemm_bs with caller-owned memory",
                    a.m, a.n, a.k, static_cast<long long>(bytes_a + bytes_b), kNoAllocScratchBytes);
    unsigned char* scratch = nullptr;
    int rc = noalloc_scratch_address(&scratch);
    if (rc != DG_OK) return rc;
    int32_t* sfa_packed = reinterpret_cast<int32_t*>(scratch);
    int32_t* sfb_packed = reinterpret_cast<int32_t*>(scratch + bytes_a);
    // Every word the GEMM reads is rewritten by the two pack launches: nothing relies on the array's old contents
    rc = dg_sf_pack_ue8m0(a.sfa, sfa_packed, 1, a.m, static_cast<int32_t>(sf_k), 1, 0, sf_k, 1, nullptr, 0, 0, a.stream);
    if (rc != DG_OK) return rc;
    rc = dg_sf_pack_ue8m0(a.sfb, sfb_packed, 1, a.n, static_cast<int32_t>(sf_k), a.gran_mn_b, 0, sf_k, 1, nullptr, 0, 0,
                          a.stream);
    if (rc != DG_OK) return rc;
    dg_gemm_args g;
    memset(&g, 0, sizeof(g));
    g.gemm_type = DG_GEMM_NORMAL, g.m = a.m, g.n = a.n, g.k = a.k, g.num_groups = 1;
    g.a.data = a.a, g.a.sf = sfa_packed, g.a.ld = a.lda, g.a.sf_ld = amn_a, g.a.dtype = DG_E4M3, g.a.gran_k = a.gran_k;
    g.b.data = a.b, g.b.sf = sfb_packed, g.b.ld = a.ldb, g.b.sf_ld = amn_b, g.b.dtype = DG_E4M3, g.b.gran_k = a.gran_k;
    g.d = a.d, g.ldd = a.ldd, g.d_dtype = a.d_dtype, g.alpha = 1.0f, g.stream = a.stream;
    return run_gemm(g, 0, nullptr);
}

}  // extern "C"
