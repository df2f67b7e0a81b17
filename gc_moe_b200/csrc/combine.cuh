// Weighted-combine tail: y[t] = bf16( sum over the token's valid slots ).
//
// The route weights were already applied before the intermediate was
// requantised, so this is a plain sum: FP32, starting from +0, in the fixed
// order "shared-expert slot, then top-k slots 0..k-1", skipping slots whose
// expert id is not a valid expert, then one round to BF16 -- the order of the
// reference's finalize role (gc_moe/impls/sm100_fp8_fp4_gc_moe.py:549-691).
// A token without any valid slot gets zeros.  HBM-bound: each thread reduces
// one 16-byte column group of one token with 16-byte loads and one store.
#pragma once

#include <cuda_bf16.h>

#include "device_common.cuh"

namespace gcmoe {

constexpr int kCombineThreads = 256;

struct CombineParams {
    const __nv_bfloat16* slots;    // combine_tokens [k(+1)][cap][H] on this rank
    const long long* topk_idx;     // [cap][k]
    __nv_bfloat16* y;              // [T][H]
    uint32_t* epoch_word;          // per-call counter in the arena (recv_parity)
    // multi-rank: the partial rows are written by other GPUs; wait until
    // rows x 128-channel pieces have landed (null on a single rank)
    const uint32_t* call_info;     // [kCallInfoWords] written by the dispatch kernel
    const uint32_t* combine_arrived;   // this rank's exchange::kCombineArrived
    uint32_t* failed;              // this rank's exchange::kFailed
    uint32_t* status;
    uint64_t timeout_ns;
    uint32_t halves_per_row;       // H / 128: 128-channel pieces of a row, each counted once by its writer
    uint32_t num_ranks;
    uint32_t num_tokens, topk, hidden, capacity, num_experts, has_shared;
};

__global__ void __launch_bounds__(kCombineThreads) combine_kernel(const CombineParams p) {
    const uint32_t vecs_per_token = p.hidden / 8;
    const uint64_t total = static_cast<uint64_t>(p.num_tokens) * vecs_per_token;
    ptx::launch_dependents();
    ptx::grid_dependency_wait();
    if (*p.failed != 0u) return;     // an earlier wait on this workspace gave up: the host will raise
    if (p.num_ranks > 1) {
        __shared__ uint32_t abort_word;
        if (threadIdx.x == 0) {
            abort_word = 0;
            WaitCtl ctl;
            ctl.status = p.status;
            ctl.failed = p.failed;
            ctl.abort = &abort_word;
            ctl.timeout_ns = p.timeout_ns;
            ctl.kernel = kKernelCombine;
            flag_wait_eq(p.combine_arrived + p.call_info[kCallGeneration] * 32,
                         p.call_info[kCallCombineRows] * p.halves_per_row, ctl, 1);
        }
        __syncthreads();
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *p.epoch_word += 1u;   // one call retired
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kCombineThreads + threadIdx.x; i < total;
         i += static_cast<uint64_t>(gridDim.x) * kCombineThreads) {
        const uint32_t t = static_cast<uint32_t>(i / vecs_per_token);
        const uint32_t v = static_cast<uint32_t>(i - static_cast<uint64_t>(t) * vecs_per_token);
        float acc[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) acc[c] = 0.0f;
        const uint32_t nslots = p.topk + p.has_shared;
        // Slots are taken eight at a time: first every validity test, then every
        // 16-byte load (independent, so their DRAM latencies overlap), then the
        // additions in the fixed order.
        for (uint32_t g0 = 0; g0 < nslots; g0 += 8) {
            uint4 raw[8];
            uint32_t valid = 0;
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) {
                const uint32_t g = g0 + j;
                if (g >= nslots) break;
                // order: shared slot (index k) first, then 0..k-1
                const uint32_t slot = p.has_shared ? (g == 0 ? p.topk : g - 1) : g;
                bool ok = true;
                if (slot < p.topk)
                    ok = static_cast<unsigned long long>(p.topk_idx[static_cast<size_t>(t) * p.topk + slot]) < p.num_experts;
                valid |= static_cast<uint32_t>(ok) << j;
            }
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) {
                const uint32_t g = g0 + j;
                const uint32_t slot = p.has_shared ? (g == 0 ? p.topk : g - 1) : g;
                raw[j] = make_uint4(0, 0, 0, 0);
                if (valid >> j & 1u)
                    raw[j] = *reinterpret_cast<const uint4*>(
                        p.slots + (static_cast<size_t>(slot) * p.capacity + t) * p.hidden + v * 8);
            }
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) {
                if (!(valid >> j & 1u)) continue;      // an invalid slot adds nothing (not even +0)
                const uint32_t w[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    acc[2 * c] = __fadd_rn(acc[2 * c], __uint_as_float(w[c] << 16));
                    acc[2 * c + 1] = __fadd_rn(acc[2 * c + 1], __uint_as_float(w[c] & 0xFFFF0000u));
                }
            }
        }
        uint4 out;
        uint32_t* o = &out.x;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const __nv_bfloat162 pair = __floats2bfloat162_rn(acc[2 * c], acc[2 * c + 1]);
            o[c] = *reinterpret_cast<const uint32_t*>(&pair);
        }
        *reinterpret_cast<uint4*>(p.y + static_cast<size_t>(t) * p.hidden + v * 8) = out;
    }
}

}  // namespace gcmoe
