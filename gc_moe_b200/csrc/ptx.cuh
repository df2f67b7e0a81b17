// Inline-PTX building blocks for sm_100a: mbarriers, TMA (bulk and tiled, no
// cluster multicast anywhere), tcgen05 (TMEM allocation, block-scaled MMA,
// scale copy, commit, accumulator load), system-scope flags.
//
// The instruction list is the one the reference's SM100 path is written with
// (gc_moe/ptx/tcgen05.py, gc_moe/ptx/tma.py, gc_moe/ptx/ld_st.py), issued here
// for a single CTA (cta_group::1) in the decode regime and for a CTA pair
// (cta_group::2, cluster of two) in the large-token regime.  Where the
// reference signals both CTAs of a pair with one multicast commit, the pair
// path here issues two plain commits (local barrier, then the peer's).
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace gcmoe {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ long long clock_cycles() {
    long long t;
    asm volatile("mov.u64 %0, %%clock64;" : "=l"(t));
    return t;
}

// Programmatic dependent launch.  `grid_dependency_wait` returns once every
// kernel this launch depends on has finished and its writes are visible;
// before it a kernel may only do work that reads nothing those kernels wrote.
// `launch_dependents` lets the next kernel of the stream start its own
// prologue while this one is still running.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// True in exactly one lane of a converged warp.  Unlike `lane == 0`, the
// compiler knows the guarded code runs in a single thread and can feed the
// TMA / tcgen05 instructions from uniform registers directly.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }"
        : "=r"(pred));
    return pred != 0;
}

// ---------------------------------------------------------------- cluster of two CTAs
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_u64(uint32_t cluster_addr, uint64_t v) {
    asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(cluster_addr), "l"(v) : "memory");
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// Arrivals on a barrier of either CTA of the cluster (shared::cluster address).
// The producers' arrival only announces bytes (the data itself is ordered by the
// copies' complete_tx), so it carries no cluster-scope release: measured, a
// release.cluster in front of every stage's copies cost about a memory latency
// per stage.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_bar),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; "
        "selp.u32 %0, 1, 0, p; }"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// ---------------------------------------------------------------- fences
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() {
    asm volatile("fence.proxy.async.global;" ::: "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ void fence_acq_rel_gpu() {
    asm volatile("fence.acq_rel.gpu;" ::: "memory");
}

// ---------------------------------------------------------------- TMA
// L2 eviction-priority policies for the .L2::cache_hint operand.
constexpr uint64_t kEvictNormal = 0x1000000000000000ull;
constexpr uint64_t kEvictFirst = 0x12F0000000000000ull;
constexpr uint64_t kEvictLast = 0x14F0000000000000ull;

__device__ __forceinline__ void prefetch_tensormap(const void* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// Tiled loads: coordinate 0 is the innermost; x * element size must be a
// multiple of 16 bytes (callers only pass multiples of 128 elements).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* map, uint32_t bar,
                                            int c0, int c1, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(bar), "l"(hint)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* map, uint32_t bar,
                                            int c0, int c1, int c2, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar), "l"(hint)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cta.global.tile.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar), "l"(hint)
        : "memory");
}
// Loads of a CTA pair: the data lands in the executing CTA's shared memory, the
// bytes are reported to `cluster_bar`, a barrier of the pair's leader CTA
// (shared::cluster address).  No cluster multicast: each CTA fetches its own tile.
__device__ __forceinline__ void tma_pair_load_2d(uint32_t dst, const void* map, uint32_t cluster_bar,
                                                 int c0, int c1, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(cluster_bar), "l"(hint)
        : "memory");
}
__device__ __forceinline__ void tma_pair_load_3d(uint32_t dst, const void* map, uint32_t cluster_bar,
                                                 int c0, int c1, int c2, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(cluster_bar), "l"(hint)
        : "memory");
}
__device__ __forceinline__ void tma_pair_load_4d(uint32_t dst, const void* map, uint32_t cluster_bar,
                                                 int c0, int c1, int c2, int c3, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        ".L2::cache_hint [%0], [%1, {%2, %3, %4, %5}], [%6], %7;" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(cluster_bar), "l"(hint)
        : "memory");
}
// Untiled bulk load: both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar, uint64_t hint) {
    asm volatile(
        "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(hint)
        : "memory");
}

// ---------------------------------------------------------------- tcgen05
// Every tcgen05 instruction of a kernel names the same CTA group: kPair = false
// is cta_group::1 (one CTA), kPair = true is cta_group::2 (the two CTAs of a
// cluster act as one 256-row MMA; allocation and deallocation are executed by
// the same warp of both CTAs, MMAs, scale copies and commits by one thread of
// the leader CTA only).
template <bool kPair>
__device__ __forceinline__ void tmem_alloc(uint32_t result_slot_smem, uint32_t columns) {
    if constexpr (kPair)
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot_smem),
                     "r"(columns)
                     : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_slot_smem),
                     "r"(columns)
                     : "memory");
}
template <bool kPair>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (kPair)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
template <bool kPair>
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    if constexpr (kPair)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// The four K32 MMAs of one K128 stage in one block:
// D[tmem] (+)= A[smem] * B[smem] with per-32-K UE8M0 scales read from TMEM.
// Both descriptors advance by 32 bytes (+2 in 16-byte units) per step and the
// instruction descriptor by `idesc_step` (the scale-byte selectors); the first
// MMA overwrites the accumulator when `accumulate_first` is 0.  For a CTA pair
// the descriptors and TMEM addresses are offsets valid in both CTAs: each CTA
// reads its own 128 weight rows and its own half of the token rows.
#define GCMOE_MMA_K128(group)                                                                                          \
    asm volatile(                                                                                                      \
        "{ .reg .pred p; .reg .b64 da, db; .reg .b32 id;\n"                                                            \
        "mov.b64 da, %1; mov.b64 db, %2; mov.b32 id, %3;\n"                                                            \
        "setp.ne.b32 p, %5, 0;\n"                                                                                      \
        "tcgen05.mma." group ".kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, id, [%6], [%7], p;\n"            \
        "add.u64 da, da, 2; add.u64 db, db, 2; add.u32 id, id, %4;\n"                                                  \
        "setp.ne.b32 p, 1, 0;\n"                                                                                       \
        "tcgen05.mma." group ".kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, id, [%6], [%7], p;\n"            \
        "add.u64 da, da, 2; add.u64 db, db, 2; add.u32 id, id, %4;\n"                                                  \
        "tcgen05.mma." group ".kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, id, [%6], [%7], p;\n"            \
        "add.u64 da, da, 2; add.u64 db, db, 2; add.u32 id, id, %4;\n"                                                  \
        "tcgen05.mma." group ".kind::mxf8f6f4.block_scale.scale_vec::1X [%0], da, db, id, [%6], [%7], p;\n"            \
        "}" ::"r"(d_tmem),                                                                                             \
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(idesc_step), "r"(accumulate_first), "r"(sfa_tmem), "r"(sfb_tmem)     \
        : "memory")
template <bool kPair>
__device__ __forceinline__ void mma_mxf8f6f4_k128(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                  uint32_t idesc, uint32_t idesc_step, uint32_t sfa_tmem,
                                                  uint32_t sfb_tmem, uint32_t accumulate_first) {
    if constexpr (kPair) GCMOE_MMA_K128("cta_group::2");
    else GCMOE_MMA_K128("cta_group::1");
}
#undef GCMOE_MMA_K128
// 32 rows x 16 bytes of shared memory -> 4 TMEM columns, replicated to the
// four 32-lane quarters (the layout block-scale factors are read from).  For a
// CTA pair each CTA copies from its own shared memory into its own TMEM.
template <bool kPair>
__device__ __forceinline__ void tmem_cp_sf(uint32_t tmem_col, uint64_t smem_desc) {
    if constexpr (kPair)
        asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(smem_desc) : "memory");
    else
        asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(smem_desc) : "memory");
}
// Arrive on an mbarrier once every tcgen05 op issued so far by this thread has
// completed.  `bar` is a shared::cta address of this CTA or, for a pair, a
// shared::cluster address of either CTA (one plain commit per barrier; no
// multicast).
template <bool kPair>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    if constexpr (kPair)
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                     : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                     : "memory");
}
// Each thread reads 16 consecutive columns of its own TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (sm_100 format): 16-byte units for the
// start address and the stride between 8-row groups, descriptor version 1 in
// bit 46, swizzle mode in bits 61..63 (0 = none, 2 = 128-byte).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t group_stride_bytes,
                                              bool swizzle128) {
    return static_cast<uint64_t>((saddr >> 4) & 0x3FFF) |
           (static_cast<uint64_t>(group_stride_bytes >> 4) << 32) | (1ull << 46) |
           (static_cast<uint64_t>(swizzle128 ? 2 : 0) << 61);
}

// Instruction descriptor of the block-scaled MMA, A = weights (M = 128 rows, or
// 256 over a CTA pair), B = FP8 activations (N columns): UE8M0 scales (bit 23),
// M/16 in 24..28, N/8 in 17..22, A format in 7..9 (5 = e2m1, 0 = e4m3), B
// format 0 = e4m3, both K-major.  The scale byte selectors (A in 29..30, B in
// 4..5) are OR-ed in per K32 step.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n, uint32_t a_format, bool pair) {
    return (1u << 23) | (((pair ? 256u : 128u) >> 4) << 24) | ((n >> 3) << 17) | (a_format << 7);
}

// ---------------------------------------------------------------- flags
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ---------------------------------------------------------------- math
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx_ftz(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Low byte <- lo, high byte <- hi, round to nearest even, saturate to +-448.
__device__ __forceinline__ uint16_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(r) : "f"(lo), "f"(hi));
    return r;
}

}  // namespace ptx
}  // namespace gcmoe
