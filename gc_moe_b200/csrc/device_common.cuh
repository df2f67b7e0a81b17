// Types shared by the kernels and the host side of the library: the device
// status block, bounded waits, and the small integer helpers of the pool
// layout.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace gcmoe {

constexpr int kMaxRanks = 72;
constexpr int kMaxLocalExperts = 512;
constexpr int kMaxExperts = 2048;

// Status block in plan-private device memory.  word 0 is zero while every
// bounded wait of the call has succeeded; the first wait that runs out
// records where it gave up and the kernels return instead of spinning.
enum StatusWord : int {
    kStatusCode = 0,      // 0 = ok, else a StatusCode
    kStatusKernel = 1,    // KernelId of the reporter
    kStatusSite = 2,      // wait site inside that kernel
    kStatusBlock = 3,     // blockIdx.x of the reporter
    kStatusObserved = 4,  // value seen when the wait gave up
    kStatusExpected = 5,  // value waited for
    kStatusAux = 6,
    kStatusWords = 8
};
enum StatusCode : uint32_t { kOk = 0, kWaitTimeout = 1, kBadGeometry = 2 };
enum KernelId : uint32_t { kKernelDispatch = 1, kKernelGemmL1 = 2, kKernelGemmL2 = 3, kKernelCombine = 4 };

struct WaitCtl {
    uint32_t* status;          // global status block
    uint32_t* failed;          // workspace-wide sticky word: set once, every later kernel returns at once
    volatile uint32_t* abort;  // CTA-local abort word in shared memory
    uint64_t timeout_ns;
    uint32_t kernel;
    uint32_t peer_abort = 0;   // shared::cluster address of the other CTA's abort word (CTA pairs), or 0
};

__device__ __forceinline__ void report_failure(const WaitCtl& ctl, uint32_t code, uint32_t site,
                                               uint32_t observed, uint32_t expected) {
    if (atomicCAS(&ctl.status[kStatusCode], 0u, code) == 0u) {
        ctl.status[kStatusKernel] = ctl.kernel;
        ctl.status[kStatusSite] = site;
        ctl.status[kStatusBlock] = blockIdx.x;
        ctl.status[kStatusObserved] = observed;
        ctl.status[kStatusExpected] = expected;
        __threadfence();
    }
    if (ctl.failed != nullptr) *ctl.failed = 1u;
    *ctl.abort = 1u;
    if (ctl.peer_abort != 0u) ptx::st_cluster_u32(ctl.peer_abort, 1u);   // the pair leaves together
}

// Wait for a phase of an mbarrier of this CTA.  Returns false when another
// role of the CTA has already given up or when the time limit passes; the
// caller then leaves its loop.  mbarrier.try_wait itself suspends the thread
// for a bounded, hardware-chosen time, so the loop does not spin hot.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtl& ctl,
                                          uint32_t site) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        if (ptx::mbar_try_wait(bar, parity)) return true;
        if ((++spins & 15u) == 0u) {
            if (*ctl.abort) return false;
            if (ptx::globaltimer_ns() - t0 > ctl.timeout_ns) {
                report_failure(ctl, kWaitTimeout, site, parity, 0);
                return false;
            }
        }
    }
}

// Wait until a 32-bit flag in (possibly peer-written) global memory reaches
// `expected`, with acquire semantics at system scope.
__device__ __forceinline__ bool flag_wait_eq(const uint32_t* flag, uint32_t expected,
                                             const WaitCtl& ctl, uint32_t site) {
    uint32_t v = ptx::ld_acquire_sys(flag);
    if (v == expected) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        v = ptx::ld_acquire_sys(flag);
        if (v == expected) return true;
        if ((++spins & 15u) == 0u) {
            if (*ctl.abort) return false;
            if (ptx::globaltimer_ns() - t0 > ctl.timeout_ns) {
                report_failure(ctl, kWaitTimeout, site, v, expected);
                return false;
            }
        }
        __nanosleep(64);
    }
}

// Wait until a counter written by other CTAs of this GPU reaches at least
// `target` (acquire at GPU scope).
__device__ __forceinline__ bool flag_wait_ge_gpu(const uint32_t* flag, uint32_t target,
                                                 const WaitCtl& ctl, uint32_t site) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) return true;
    const uint64_t t0 = ptx::globaltimer_ns();
    uint32_t spins = 0;
    for (;;) {
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v >= target) return true;
        if ((++spins & 15u) == 0u) {
            if (*ctl.abort) return false;
            if (ptx::globaltimer_ns() - t0 > ctl.timeout_ns) {
                report_failure(ctl, kWaitTimeout, site, v, target);
                return false;
            }
        }
        __nanosleep(32);
    }
}

// Per-call words the dispatch kernel leaves in plan-private scratch for the
// kernels that follow it in the stream.
enum CallInfoWord : int {
    kCallGeneration = 0,      // 0/1: which half of the double-buffered exchange this call uses
    kCallCombineRows = 1,     // valid routes of this rank = rows its combine waits for (per H/256 tile)
    kCallEpoch = 2,
    kCallTablesReady = 3,     // epoch + 1 once the tables of this call are in place (release by dispatch CTA 0):
                              // the GEMM launch starts while the dispatch kernel is still pushing rows
    kCallTileCursor = 4,
    kCallPairRegime = 5,      // 1: the GEMM launch of the pair regime does this call's work, 0: the single one
    kCallTileCursorPair = 6,  // tile cursor of the pair regime's launch (the two launches of a call can overlap)      // tiles claimed by the running GEMM launch beyond one per CTA (back to 0 when it ends)
    kCallInfoWords = 8
};

// Cross-rank exchange block: this library's own symmetric fields.  They live
// in the arena's `l2_full_mask` signal region (8 MiB), which the stream-ordered
// kernels here never use for its reference purpose (ring-slot flow control).
// Offsets are relative to the start of that region; everything is double
// buffered by call parity ("generation").
namespace exchange {
constexpr uint32_t kCountsReady = 0;        // u32 [2][kMaxRanks]: epoch+1 once a source's counts landed
constexpr uint32_t kSourceBlockM = 1024;    // u32 [2][kMaxRanks]: block-M each rank uses for its pool
constexpr uint32_t kFailed = 1920;          // u32: a bounded wait of some call on this workspace ran out
constexpr uint32_t kCombineArrived = 2048;  // u32 [2] (128 bytes apart): rows x tiles landed in combine_tokens
constexpr uint32_t kTilesUsed = 1928;       // u32 [2]: row tiles of the last call of each generation (how many counters to clear)
constexpr uint32_t kCounts = 8192;          // u32 [2][P][E]: routes of source s to global expert e
constexpr uint32_t kMaxRowTiles = 1u << 18;
constexpr uint32_t kTileArrived = 2u << 20; // u32 [2][kMaxRowTiles]: dispatched rows landed per GEMM row tile of this rank
// every field ends before the next one begins, for the largest group the API admits
static_assert(kCountsReady + 2u * kMaxRanks * 4u <= kSourceBlockM, "kCountsReady overlaps kSourceBlockM");
static_assert(kSourceBlockM + 2u * kMaxRanks * 4u <= kFailed, "kSourceBlockM overlaps kFailed");
static_assert(kFailed + 4u <= kTilesUsed, "kFailed overlaps kTilesUsed");
static_assert(kTilesUsed + 8u <= kCombineArrived, "kTilesUsed overlaps kCombineArrived");
static_assert(kCombineArrived + 128u + 4u <= kCounts, "kCombineArrived overlaps kCounts");
static_assert(kCounts + 2u * kMaxRanks * kMaxExperts * 4u <= kTileArrived, "kCounts overlaps kTileArrived");
constexpr uint32_t kBytes = kTileArrived + 2u * kMaxRowTiles * 4u;   // 4 MiB of the 8 MiB region
static_assert(kBytes <= (8u << 20), "exchange block exceeds the signal region it lives in");
}  // namespace exchange

// Two regimes of the expert GEMMs:
//  * single: one CTA per tile, cta_group::1, tiles of up to 64 tokens.  A tcgen05.mma
//    costs the same issue time for 16 columns as for 64, and the kernel is bound by
//    weight streaming: the regime of decode and of evenly spread routing.
//  * pair: a CTA pair per tile, cta_group::2.  The pair's MMA covers 256 weight rows
//    and up to 240 tokens with the token operand split over the two CTAs, so one
//    fetch of a weight tile serves up to 240 tokens, and two accumulator stages of
//    240 columns fit each CTA's TMEM: the regime of experts with hundreds of rows
//    (large token counts, skewed routing).  It streams the weights of experts with
//    few rows at about half the rate of the single regime (a CTA of a pair fetches
//    half a weight tile per request), so it only pays when most rows sit in large
//    experts.
// The regime of a rank is chosen per call ON THE DEVICE, from the rows its experts
// actually received: small calls are always single (dual_regime_call); otherwise
// pair when at least half of the rank's rows belong to experts with
// kPairExpertRows rows or more.  Every rank evaluates this for every owner from the exchanged count matrix
// (senders need the owner's tile geometry), so all ranks agree.  The host enqueues
// the GEMM launch of both regimes; the one that was not chosen returns at once.
// GEMM tiles are independent of the pool blocks: an expert's rows are contiguous
// in the pool, and its tiles are sized from its own row count so that an expert
// with many rows costs as few passes over its weights as possible.  The scale
// words of the tiles are kept a second time in tile order (the reference layout
// orders them by pool block).
constexpr uint32_t kPairMinBlockM = 96;
constexpr uint32_t kPairTileRows = 240;
constexpr uint32_t kPairExpertRows = 128;
constexpr uint32_t kSingleTileRows = 64;
constexpr uint32_t kDualMinRoutes = 4096;
// Whether a call enqueues the launches of both regimes (host; the flag travels to the other ranks
// with the block-M): calls large enough for some expert to collect hundreds of rows -- block-M 96
// and above, or 4096 routes in the group (taking this rank's token count for every rank).  Below
// that the second launch's microseconds (about 10 when the launches run one after the other)
// would not be earned back.
__host__ __device__ __forceinline__ bool dual_regime_call(uint32_t block_m, uint64_t group_routes) {
    return block_m >= kPairMinBlockM || group_routes >= kDualMinRoutes;
}
// the regime of one call: rows_in_large = rows of experts with >= kPairExpertRows rows
__host__ __device__ __forceinline__ bool pair_chosen(bool dual, uint32_t rows_in_large, uint32_t rows) {
    return dual && rows != 0u && 2u * rows_in_large >= rows;
}
constexpr uint32_t kBlockMDualFlag = 0x10000u;   // set in the exchanged block-M word of a rank whose call is dual

__host__ __device__ __forceinline__ uint32_t round_up_u32(uint32_t v, uint32_t m) {
    return (v + m - 1) / m * m;
}
// Rows per GEMM tile of an expert that received `n` rows, in the given regime
// (tile t covers rows [t * rows, ...)).
__host__ __device__ __forceinline__ uint32_t expert_tile_rows(bool pair, uint32_t n) {
    if (!pair) return kSingleTileRows;
    if (n <= kPairTileRows) return n <= 16u ? 16u : round_up_u32(n, 16u);
    const uint32_t tiles = (n + kPairTileRows - 1u) / kPairTileRows;
    return round_up_u32((n + tiles - 1u) / tiles, 16u);
}
// Without room for the tile-ordered scale copy the tiles are the pool blocks.
__host__ __device__ __forceinline__ uint32_t routed_tile_rows(uint32_t block_m, uint32_t n, bool tile_ordered, bool pair) {
    return tile_ordered ? expert_tile_rows(pair, n) : block_m;
}

// Row, inside a 128-row-aligned scale block, of the block's u-th token: the
// 4x32 order the tensor core's scale copy expects
// (gc_moe/gc/__init__.py:19-23).
__host__ __device__ __forceinline__ uint32_t sf_row_in_block(uint32_t u) {
    return (u & ~127u) + (u & 31u) * 4u + ((u >> 5) & 3u);
}

}  // namespace gcmoe
