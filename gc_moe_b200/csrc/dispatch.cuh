// Top-k token dispatch into the expert owners' receive pools.
//
// One kernel, no grid-wide barrier: every CTA recomputes the (tiny) routing
// histogram of this rank's T x k routes, so every CTA knows each expert's
// total and how many of an expert's routes precede the CTA's own slice of
// routes.  A route's row in the owner's pool is then
//     expert's first pool block x BM  +  routes of earlier source ranks
//                                      +  rank of the route inside this source
// which reproduces the pool order of the reference (experts ascending, source
// ranks ascending inside an expert) with the canonical ascending token*k+slot
// order inside one (expert, source) group, where the reference's own order is
// whatever its atomics produced (gc_moe/impls/sm100_fp8_fp4_gc_moe.py:762-1107).
// Each warp then pushes whole rows -- FP8 payload, packed scale words, route
// weight, source metadata, index-table entry -- straight to their final place
// in the owner's arena; on one rank these are local stores.
//
// Data products written (same arena regions and meaning as the reference):
//   expert_recv_count[gen][src][l]        routes from src to local expert l
//   expert_recv_count_sum[gen][l]         low word: total routes to l
//   src_token_topk_idx[l][src][i]         token*k+slot of the i-th route
//   token_src_metadata[pool_row]          (src_rank, src_token, slot)
//   l1_acts[pool_row], l1_acts_sf[...], l1_topk_weights[pool_row]
//   routed_pool_blocks                    number of pool blocks of this call
// and, in plan-private memory, the per-expert token counts and pool-block
// prefix the GEMM kernels schedule from.
#pragma once

#include "device_common.cuh"

namespace gcmoe {

constexpr int kDispatchThreads = 256;

struct DispatchParams {
    // this rank's staged inputs (arena views)
    const uint8_t* x;             // e4m3 [cap][H]
    const uint32_t* x_sf;         // [cap][H/128] packed UE8M0 words, K-major
    const long long* topk_idx;    // [cap][k]
    const float* topk_weights;    // [cap][k]
    // receive-side regions, addressed through the owner's arena base
    uint64_t arena_base[kMaxRanks];
    uint64_t off_recv_count, off_recv_count_sum, off_routed_pool_blocks, off_recv_parity;
    uint64_t off_index_table, off_metadata, off_l1_acts, off_l1_acts_sf, off_l1_weights;
    // plan-private outputs
    int* expert_count;            // [E_loc]
    int* expert_block_start;      // [E_loc + 1]
    int* stats;                   // optional cumulative per-expert counter (may be null)
    uint32_t* status;
    uint64_t timeout_ns;
    uint32_t num_ranks, rank, num_experts, local_experts;
    uint32_t num_tokens, topk, hidden, capacity;
    uint32_t block_m, sf_block_m, sf_ring;   // sf_ring: words between K128 planes of l1_acts_sf
};

// Dynamic shared memory: total[E], before[E], start[E_loc + 1], then the
// CTA's slice: expert id and destination pool row per route.
__host__ __device__ inline uint32_t dispatch_smem_bytes(uint32_t num_experts, uint32_t local_experts,
                                                        uint32_t slice) {
    return (2 * num_experts + local_experts + 1 + 2 * slice) * 4;
}

__global__ void __launch_bounds__(kDispatchThreads)
dispatch_kernel(const __grid_constant__ DispatchParams p) {
    extern __shared__ uint32_t smem[];
    const uint32_t routes = p.num_tokens * p.topk;
    const uint32_t slice = (routes + gridDim.x - 1) / gridDim.x;
    const uint32_t lo = min(blockIdx.x * slice, routes), hi = min(lo + slice, routes);
    uint32_t* const total = smem;
    uint32_t* const before = total + p.num_experts;
    uint32_t* const start = before + p.num_experts;               // pool-block prefix of local experts
    int* const slice_expert = reinterpret_cast<int*>(start + p.local_experts + 1);
    uint32_t* const slice_row = reinterpret_cast<uint32_t*>(slice_expert + slice);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (uint32_t i = tid; i < 2 * p.num_experts; i += kDispatchThreads) total[i] = 0;
    __syncthreads();
    // A route is valid iff its expert id, compared as unsigned 64-bit, is below
    // the expert count (negative ids mean "no route").
    for (uint32_t a = tid; a < routes; a += kDispatchThreads) {
        const unsigned long long e = static_cast<unsigned long long>(p.topk_idx[a]);
        if (e < p.num_experts) {
            atomicAdd(&total[e], 1u);
            if (a < lo) atomicAdd(&before[e], 1u);
        }
    }
    __syncthreads();

    // Pool-block prefix over this rank's local experts (single rank: every
    // route of a local expert comes from this rank).
    const uint32_t first_local = p.rank * p.local_experts;
    if (warp == 0) {
        const uint32_t per_lane = (p.local_experts + 31) / 32;
        uint32_t sum = 0;
        for (uint32_t i = 0; i < per_lane; ++i) {
            const uint32_t l = lane * per_lane + i;
            if (l < p.local_experts) sum += (total[first_local + l] + p.block_m - 1) / p.block_m;
        }
        uint32_t incl = sum;
        for (uint32_t d = 1; d < 32; d <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
            if (lane >= d) incl += v;
        }
        uint32_t run = incl - sum;
        for (uint32_t i = 0; i < per_lane; ++i) {
            const uint32_t l = lane * per_lane + i;
            if (l < p.local_experts) {
                start[l] = run;
                run += (total[first_local + l] + p.block_m - 1) / p.block_m;
            }
        }
        if (lane == 31) start[p.local_experts] = incl;
    }
    __syncthreads();

    uint8_t* const my_arena = reinterpret_cast<uint8_t*>(p.arena_base[p.rank]);
    // The receive counters are double-buffered by call parity; the combine
    // kernel bumps the call counter when a call retires, so replays of a
    // captured graph alternate without host involvement.
    const uint32_t generation = *reinterpret_cast<const uint32_t*>(my_arena + p.off_recv_parity) & 1u;
    if (blockIdx.x == 0) {
        unsigned long long* recv = reinterpret_cast<unsigned long long*>(my_arena + p.off_recv_count) +
            static_cast<size_t>(generation) * p.num_ranks * p.local_experts +
            static_cast<size_t>(p.rank) * p.local_experts;
        unsigned long long* recv_sum = reinterpret_cast<unsigned long long*>(my_arena + p.off_recv_count_sum) +
            static_cast<size_t>(generation) * p.local_experts;
        for (uint32_t l = tid; l < p.local_experts; l += kDispatchThreads) {
            const uint32_t n = total[first_local + l];
            p.expert_count[l] = static_cast<int>(n);
            p.expert_block_start[l] = static_cast<int>(start[l]);
            recv[l] = n;
            // high word: number of source ranks that have reported
            recv_sum[l] = (static_cast<unsigned long long>(p.num_ranks) << 32) | n;
            if (p.stats != nullptr) p.stats[l] += static_cast<int>(n);
        }
        if (tid == 0) {
            p.expert_block_start[p.local_experts] = static_cast<int>(start[p.local_experts]);
            *reinterpret_cast<uint32_t*>(my_arena + p.off_routed_pool_blocks) = start[p.local_experts];
        }
    }

    // Destination of every route in this CTA's slice.
    for (uint32_t a = lo + tid; a < hi; a += kDispatchThreads) {
        const unsigned long long e64 = static_cast<unsigned long long>(p.topk_idx[a]);
        slice_expert[a - lo] = e64 < p.num_experts ? static_cast<int>(e64) : -1;
    }
    __syncthreads();
    for (uint32_t a = lo + tid; a < hi; a += kDispatchThreads) {
        const int e = slice_expert[a - lo];
        uint32_t row = 0xFFFFFFFFu;
        if (e >= 0) {
            uint32_t i = before[e];
            for (uint32_t j = 0; j < a - lo; ++j) i += (slice_expert[j] == e);
            const uint32_t owner = static_cast<uint32_t>(e) / p.local_experts;
            const uint32_t l = static_cast<uint32_t>(e) - owner * p.local_experts;
            row = start[l] * p.block_m + i;
            uint8_t* const dst_arena = reinterpret_cast<uint8_t*>(p.arena_base[owner]);
            reinterpret_cast<uint32_t*>(dst_arena + p.off_index_table)[
                (static_cast<size_t>(l) * p.num_ranks + p.rank) * p.capacity + i] = a;
            uint32_t* meta = reinterpret_cast<uint32_t*>(dst_arena + p.off_metadata) + static_cast<size_t>(row) * 3;
            meta[0] = p.rank;
            meta[1] = a / p.topk;
            meta[2] = a % p.topk;
            reinterpret_cast<float*>(dst_arena + p.off_l1_weights)[row] = p.topk_weights[a];
        }
        slice_row[a - lo] = row;
    }
    __syncthreads();

    // One warp per route: copy the FP8 row (16 bytes per lane per step) and
    // scatter its packed scale words into the MN-major scale ring.
    const uint32_t row_vecs = p.hidden / 16, sf_words = p.hidden / 128;
    for (uint32_t a = lo + warp; a < hi; a += kDispatchThreads / 32) {
        const uint32_t row = slice_row[a - lo];
        if (row == 0xFFFFFFFFu) continue;
        const uint32_t owner = static_cast<uint32_t>(slice_expert[a - lo]) / p.local_experts;
        uint8_t* const dst_arena = reinterpret_cast<uint8_t*>(p.arena_base[owner]);
        const uint32_t t = a / p.topk;
        const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(t) * p.hidden);
        uint4* dst = reinterpret_cast<uint4*>(dst_arena + p.off_l1_acts + static_cast<size_t>(row) * p.hidden);
        for (uint32_t v = lane; v < row_vecs; v += 32) dst[v] = src[v];
        const uint32_t block = row / p.block_m, u = row - block * p.block_m;
        const uint32_t sf_row = block * p.sf_block_m + sf_row_in_block(u);
        uint32_t* sf_dst = reinterpret_cast<uint32_t*>(dst_arena + p.off_l1_acts_sf);
        for (uint32_t w = lane; w < sf_words; w += 32)
            sf_dst[static_cast<size_t>(w) * p.sf_ring + sf_row] = p.x_sf[static_cast<size_t>(t) * sf_words + w];
    }
}

}  // namespace gcmoe
