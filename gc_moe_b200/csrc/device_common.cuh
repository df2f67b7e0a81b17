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
    kCallTileCursor = 4,      // tiles claimed by the running GEMM launch beyond one per CTA (back to 0 when it ends)
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
constexpr uint32_t kFailed = 1536;          // u32: a bounded wait of some call on this workspace ran out
constexpr uint32_t kCombineArrived = 2048;  // u32 [2] (128 bytes apart): rows x tiles landed in combine_tokens
constexpr uint32_t kRowsArrived = 4096;     // u32 [2][kMaxLocalExperts]: dispatched rows landed per local expert
constexpr uint32_t kCounts = 8192;          // u32 [2][P][E]: routes of source s to global expert e
__host__ __device__ __forceinline__ uint32_t bytes(uint32_t ranks, uint32_t experts) {
    return kCounts + 2u * ranks * experts * 4u;
}
}  // namespace exchange

// Rows (tokens) per GEMM tile for a pool laid out in blocks of `block_m`.  The
// tiles are independent of the pool blocks (an expert's rows are contiguous):
//  * small blocks are grouped up to 64 tokens, because a tcgen05.mma costs the
//    same issue time for 16 columns as for 64;
//  * blocks of 64 to 112 tokens are the tiles (measured: wider tiles for these
//    cost a pipeline stage and gain nothing);
//  * larger blocks (the large-token regime, block-M up to 240) are cut into
//    tiles of 112 tokens, the largest count whose two accumulator stages and
//    scale columns fit the 512 TMEM columns, so that the epilogue of one tile
//    overlaps the MMAs of the next (measured at 4080 rows over 32 experts of
//    H7168: 296 us instead of 472 us with whole 192-token blocks).
// With a fused shared expert, whose scales the caller stages in block-M order,
// the large blocks stay whole tiles.  Every rank evaluates this for every
// owner, so it depends only on values all ranks share.
constexpr uint32_t kWideTileRows = 112;
__host__ __device__ __forceinline__ uint32_t gemm_tile_rows(uint32_t block_m, bool fused_shared) {
    if (block_m < 64u) return 64u;
    if (block_m <= kWideTileRows || fused_shared) return block_m;
    return kWideTileRows;
}

__host__ __device__ __forceinline__ uint32_t round_up_u32(uint32_t v, uint32_t m) {
    return (v + m - 1) / m * m;
}

// Row, inside a 128-row-aligned scale block, of the block's u-th token: the
// 4x32 order the tensor core's scale copy expects
// (gc_moe/gc/__init__.py:19-23).
__host__ __device__ __forceinline__ uint32_t sf_row_in_block(uint32_t u) {
    return (u & ~127u) + (u & 31u) * 4u + ((u >> 5) & 3u);
}

}  // namespace gcmoe
