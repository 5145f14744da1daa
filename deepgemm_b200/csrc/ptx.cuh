// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05
// (TMEM allocation, UMMA, UTCCP, TMEM loads), cluster helpers and the descriptor
// encoders the block-scaled UMMA needs.  Bit layouts follow the PTX ISA tables for
// the tcgen05 shared-memory matrix descriptor and the block-scaled instruction
// descriptor.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace dg {

#define DG_DEVICE __device__ __forceinline__

// --------------------------------------------------------------------------- misc
DG_DEVICE uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
DG_DEVICE uint32_t lane_id() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%laneid;" : "=r"(r));
    return r;
}
DG_DEVICE uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
DG_DEVICE bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

// Programmatic dependent launch: wait until the kernels this launch depends on have completed and flushed (returns at
// once when the launch carries no such dependency); let the next kernel in the stream start its prologue.
DG_DEVICE void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
DG_DEVICE void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// --------------------------------------------------------------------------- cluster
DG_DEVICE uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
DG_DEVICE void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
DG_DEVICE void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
DG_DEVICE void cluster_sync() {
    cluster_arrive();
    cluster_wait();
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
DG_DEVICE uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}
DG_DEVICE void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

// --------------------------------------------------------------------------- mbarrier
DG_DEVICE void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
DG_DEVICE void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
DG_DEVICE void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Arrive on a barrier given by a shared::cluster address (possibly in the peer CTA).
DG_DEVICE void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
DG_DEVICE void mbar_arrive_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
                 : "memory");
}
DG_DEVICE void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
DG_DEVICE bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Kept as a separate name for waits whose arrivals come from the peer CTA of a pair.
DG_DEVICE bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// --------------------------------------------------------------------------- fences
DG_DEVICE void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
DG_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DG_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
DG_DEVICE void named_barrier_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// --------------------------------------------------------------------------- TMA
DG_DEVICE void prefetch_tmap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 2-D / 3-D tiled loads into this CTA's shared memory.  `mbar_addr` is a shared::cluster
// address: the CTA's own barrier, or (kCtaGroup2) the leader CTA's barrier of a CTA pair.
template <bool kCtaGroup2>
DG_DEVICE void tma_load_2d(uint32_t dst_smem, const void* tmap, uint32_t mbar_addr, int32_t c0, int32_t c1) {
    if constexpr (kCtaGroup2) {
        asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst_smem),
            "l"(reinterpret_cast<uint64_t>(tmap)), "r"(mbar_addr), "r"(c0), "r"(c1)
            : "memory");
    } else {
        asm volatile(
            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst_smem),
            "l"(reinterpret_cast<uint64_t>(tmap)), "r"(mbar_addr), "r"(c0), "r"(c1)
            : "memory");
    }
}
template <bool kCtaGroup2>
DG_DEVICE void tma_load_3d(uint32_t dst_smem, const void* tmap, uint32_t mbar_addr, int32_t c0, int32_t c1,
                           int32_t c2) {
    if constexpr (kCtaGroup2) {
        asm volatile(
            "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst_smem),
            "l"(reinterpret_cast<uint64_t>(tmap)), "r"(mbar_addr), "r"(c0), "r"(c1), "r"(c2)
            : "memory");
    } else {
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst_smem),
            "l"(reinterpret_cast<uint64_t>(tmap)), "r"(mbar_addr), "r"(c0), "r"(c1), "r"(c2)
            : "memory");
    }
}
DG_DEVICE void tma_store_2d(const void* tmap, uint32_t src_smem, int32_t c0, int32_t c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(src_smem), "r"(c0), "r"(c1)
                 : "memory");
}
DG_DEVICE void tma_store_3d(const void* tmap, uint32_t src_smem, int32_t c0, int32_t c1, int32_t c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(src_smem), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
template <bool kCtaGroup2>
DG_DEVICE void tma_load_3d_hint(uint32_t dst_smem, const void* tmap, uint32_t mbar_addr, int32_t c0, int32_t c1,
                                int32_t c2, uint64_t policy) {
    if constexpr (kCtaGroup2) {
        asm volatile(
            "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%3, %4, %5}], [%2], %6;" ::"r"(dst_smem),
            "l"(reinterpret_cast<uint64_t>(tmap)), "r"(mbar_addr), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
            : "memory");
    } else {
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
            " [%0], [%1, {%3, %4, %5}], [%2], %6;" ::"r"(dst_smem),
            "l"(reinterpret_cast<uint64_t>(tmap)), "r"(mbar_addr), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
            : "memory");
    }
}
// L2 eviction priorities for bulk copies (createpolicy): lines fetched or written with evict_first leave L2 before
// others, evict_last ones stay longest.
DG_DEVICE uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
DG_DEVICE uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
DG_DEVICE void tma_store_3d_hint(const void* tmap, uint32_t src_smem, int32_t c0, int32_t c1, int32_t c2, uint64_t policy) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3, %4}], [%1], %5;" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(src_smem), "r"(c0), "r"(c1), "r"(c2), "l"(policy)
                 : "memory");
}
DG_DEVICE void tma_reduce_add_2d(const void* tmap, uint32_t src_smem, int32_t c0, int32_t c1) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(tmap)),
                 "r"(src_smem), "r"(c0), "r"(c1)
                 : "memory");
}
DG_DEVICE void tma_reduce_add_3d(const void* tmap, uint32_t src_smem, int32_t c0, int32_t c1, int32_t c2) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
            reinterpret_cast<uint64_t>(tmap)),
        "r"(src_smem), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Untiled bulk copy global -> this CTA's shared memory, completing `bytes` on an mbarrier of this CTA.
// Both addresses 16-byte aligned, bytes a multiple of 16.
DG_DEVICE void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t mbar_addr) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(mbar_addr)
                 : "memory");
}

DG_DEVICE void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
DG_DEVICE void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
DG_DEVICE void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// --------------------------------------------------------------------------- TMEM / tcgen05
template <int kCtas>
DG_DEVICE void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    if constexpr (kCtas == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                     "r"(ncols)
                     : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                     "r"(ncols)
                     : "memory");
}
template <int kCtas>
DG_DEVICE void tmem_relinquish() {
    if constexpr (kCtas == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int kCtas>
DG_DEVICE void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    if constexpr (kCtas == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] with per-32/128-K UE8M0 scales read from TMEM.
template <int kCtas>
DG_DEVICE void umma_mxf8f6f4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                             uint32_t sfb_tmem, uint32_t accumulate) {
    if constexpr (kCtas == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
            : "memory");
}

// D[tmem] (+)= A[smem] * B[smem] for BF16 operands without scale factors (kind::f16, UMMA K = 16, FP32 accumulation).
template <int kCtas>
DG_DEVICE void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    if constexpr (kCtas == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
}

// The same with both operands packed E2M1 (two values per byte in shared memory), UMMA K = 64 and one UE8M0 scale
// per 32 K elements: two scale bytes per row and instruction (scale_vec::2X), byte ids 0 or 2 of the TMEM word.
template <int kCtas>
DG_DEVICE void umma_mxf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                         uint32_t sfb_tmem, uint32_t accumulate) {
    if constexpr (kCtas == 1)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n\t}" ::"r"(d_tmem),
            "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
            : "memory");
}

// Arrive on mbarrier(s) once every tcgen05 op issued so far by this thread has completed.
// kCtas == 2: the arrive is multicast to the same barrier offset in both CTAs of the pair.
template <int kCtas>
DG_DEVICE void umma_commit(uint64_t* bar) {
    if constexpr (kCtas == 1) {
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                     : "memory");
    } else {
        const uint16_t mask = 0x3;
        asm volatile(
            "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                smem_u32(bar)),
            "h"(mask)
            : "memory");
    }
}

// Copy 32 rows x 16 bytes of shared memory into 4 TMEM columns, replicated to all four
// 32-lane quadrants (the layout block-scaled UMMA reads its scale factors from).
template <int kCtas>
DG_DEVICE void utccp_32x128b_warpx4(uint32_t tmem_addr, uint64_t smem_desc) {
    if constexpr (kCtas == 1)
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
    else
        asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_addr), "l"(smem_desc) : "memory");
}

// 32 lanes x 32 columns of 32-bit accumulators -> 32 registers per thread (lane = row).
DG_DEVICE void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
DG_DEVICE void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// --------------------------------------------------------------------------- descriptors
// tcgen05 shared-memory matrix descriptor (64 bit):
//   [0,14)  start address >> 4        [16,30) leading-dimension byte offset >> 4
//   [32,46) stride-dimension byte offset >> 4      [46,48) version = 1 on sm_100
//   [49,52) base offset (0: tiles are 1024 B aligned)   [61,64) swizzle: 0 none, 2 128 B, 4 64 B, 6 32 B
constexpr uint32_t kSwizzleNone = 0, kSwizzle128B = 2, kSwizzle64B = 4, kSwizzle32B = 6;
DG_DEVICE uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3FFF);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(swizzle & 7) << 61;
    return d;
}

// Block-scaled instruction descriptor (32 bit), kind::mxf8f6f4:
//   [4,6) B scale-factor byte id   [7,10) A format   [10,13) B format (0 = E4M3, 5 = E2M1)
//   [15] A is MN-major   [16] B is MN-major   [17,23) N >> 3   [23] scale type (1 = UE8M0)
//   [24,29) M >> 4       [29,31) A scale-factor byte id
constexpr uint32_t kFmtE4M3 = 0, kFmtE2M1 = 5;
__host__ __device__ inline uint32_t make_idesc_mxf8f6f4(uint32_t fmt_a, uint32_t fmt_b, bool a_mn_major,
                                                       bool b_mn_major, uint32_t umma_m, uint32_t umma_n) {
    uint32_t d = 0;
    d |= (fmt_a & 7) << 7;
    d |= (fmt_b & 7) << 10;
    d |= (a_mn_major ? 1u : 0u) << 15;
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= ((umma_n >> 3) & 0x3F) << 17;
    d |= 1u << 23;
    d |= ((umma_m >> 4) & 0x1F) << 24;
    return d;
}
// kind::mxf4: the same fields; the only operand format is E2M1 (code 1), both operands K-major.
__host__ __device__ inline uint32_t make_idesc_mxf4(uint32_t umma_m, uint32_t umma_n) {
    uint32_t d = 0;
    d |= 1u << 7;
    d |= 1u << 10;
    d |= ((umma_n >> 3) & 0x3F) << 17;
    d |= 1u << 23;
    d |= ((umma_m >> 4) & 0x1F) << 24;
    return d;
}
// kind::f16 with BF16 operands and an FP32 accumulator: no scale fields; [4,6) accumulator format (1 = F32),
// [7,10) / [10,13) operand formats (1 = BF16), [15] / [16] MN-major flags, [17,23) N >> 3, [24,29) M >> 4.
__host__ __device__ inline uint32_t make_idesc_bf16(bool a_mn_major, bool b_mn_major, uint32_t umma_m, uint32_t umma_n) {
    uint32_t d = 0;
    d |= 1u << 4;
    d |= 1u << 7;
    d |= 1u << 10;
    d |= (a_mn_major ? 1u : 0u) << 15;
    d |= (b_mn_major ? 1u : 0u) << 16;
    d |= ((umma_n >> 3) & 0x3F) << 17;
    d |= ((umma_m >> 4) & 0x1F) << 24;
    return d;
}
DG_DEVICE uint32_t idesc_with_sf_ids(uint32_t idesc, uint32_t a_sf_id, uint32_t b_sf_id) {
    return idesc | ((b_sf_id & 3) << 4) | ((a_sf_id & 3) << 29);
}
DG_DEVICE uint32_t idesc_with_n(uint32_t idesc, uint32_t umma_n) {
    return (idesc & ~(0x3Fu << 17)) | (((umma_n >> 3) & 0x3F) << 17);
}

}  // namespace dg
