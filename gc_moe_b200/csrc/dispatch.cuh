// Top-k token dispatch into the expert owners' receive pools.
//
// PUSH design, one kernel per rank, no grid-wide barrier and no pull round
// trip.  Every CTA recomputes the (tiny) routing histogram of this rank's
// T x k routes, so every CTA knows each expert's count and how many of an
// expert's routes precede the CTA's own slice of routes.  With more than one
// rank the per-expert counts are first exchanged all-to-all (each source
// stores its E counts and its block-M into every peer's exchange block, then a
// release flag; one NVLink hop), after which every source can compute, on its
// own, the final pool row of each of its routes at the route's owner:
//     expert's first pool block x BM(owner) + routes of lower source ranks
//                                           + rank of the route inside this source
// This is the pool order of the reference (experts ascending, source ranks
// ascending inside an expert; gc_moe/impls/sm100_fp8_fp4_gc_moe.py:931-953)
// with the canonical ascending token*k+slot order inside one (expert, source)
// group, where the reference's own order is whatever its atomics produced.
// Each warp then pushes whole rows -- FP8 payload, packed scale words, route
// weight, source metadata, index-table entry -- straight to their final place
// in the owner's arena (16-byte stores over NVLink, local stores on one rank)
// and bumps the owner's arrival counter of the GEMM row tile the row belongs to
// (a system-scope fence and relaxed adds, once per four rows of the warp).
// The reference instead writes indices, waits for every rank's counts and then
// PULLS each row with a remote read (impls:997-1094): one more NVLink trip on
// the critical path.
//
// Data products written (same arena regions and meaning as the reference):
//   expert_recv_count[gen][src][l]        routes from src to local expert l
//   expert_recv_count_sum[gen][l]         low word: total routes to l
//   src_token_topk_idx[l][src][i]         token*k+slot of the i-th route
//   token_src_metadata[pool_row]          (src_rank, src_token, slot)
//   l1_acts[pool_row], l1_acts_sf[...], l1_topk_weights[pool_row]
//   routed_pool_blocks                    number of pool blocks of this call
// and, in plan-private memory, the per-expert token counts, the pool-block
// prefix and the call-info words the later kernels of the call read.
#pragma once

#include "device_common.cuh"

namespace gcmoe {

constexpr int kDispatchThreads = 512;

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
    uint64_t off_exchange;
    // plan-private outputs
    int* expert_count;            // [E_loc]
    int* expert_block_start;      // [E_loc + 1] pool-block prefix (reference layout)
    int* expert_tile_start;       // [E_loc + 1] prefix of the GEMM tiles per expert
    int* expert_row_start;        // [E_loc] first pool row per expert
    int* expert_sf_start;         // [E_loc] first row of the expert's scale chunks in the scale planes the GEMMs read
    uint32_t* call_info;          // [kCallInfoWords]
    int* shared_table;            // fused shared expert: {tokens, 0, row blocks}, or null
    uint32_t* done_routed;        // per row tile: finished gate/up tiles, zeroed here for the GEMM launch
    uint32_t* done_shared;        // same for the shared expert's row blocks, or null
    int* stats;                   // optional cumulative per-expert counter (may be null)
    uint32_t* status;
    uint64_t timeout_ns;
    uint32_t num_ranks, rank, num_experts, local_experts;
    uint32_t num_tokens, topk, hidden, capacity;
    uint32_t block_m, sf_ring;    // sf_ring: words between K128 planes of l1_acts_sf
    uint32_t dual;                // the launches of both GEMM regimes are enqueued for this call
    uint32_t private_sf_row;      // row offset, in each scale plane, of the tile-ordered scale copy (0 = none)
};

// Dynamic shared memory: seven u32 per expert (own count, own routes before the
// slice, total over sources, routes of lower sources, first pool block, first
// GEMM tile, first tile-ordered scale row), one block-M and one GEMM regime per rank,
// then the CTA's slice: expert id, pool row and position inside the expert per route.
__host__ __device__ inline uint32_t dispatch_smem_bytes(uint32_t num_experts, uint32_t num_ranks,
                                                        uint32_t slice) {
    return (7 * num_experts + 2 * num_ranks + 8 + 3 * slice) * 4;
}

__global__ void __launch_bounds__(kDispatchThreads)
dispatch_kernel(const __grid_constant__ DispatchParams p) {
    extern __shared__ uint32_t smem[];
    const uint32_t P = p.num_ranks, E = p.num_experts, EL = p.local_experts;
    const uint32_t routes = p.num_tokens * p.topk;
    const uint32_t slice = (routes + gridDim.x - 1) / gridDim.x;
    const uint32_t lo = min(blockIdx.x * slice, routes), hi = min(lo + slice, routes);
    uint32_t* const own = smem;                 // [E] routes of this rank per expert
    uint32_t* const before = own + E;           // [E] ... of them before this CTA's slice
    uint32_t* const total = before + E;         // [E] routes of all ranks
    uint32_t* const lower = total + E;          // [E] routes of source ranks below this one
    uint32_t* const first_block = lower + E;    // [E] first pool block of the expert at its owner
    uint32_t* const first_tile = first_block + E;   // [E] first GEMM tile of the expert at its owner
    uint32_t* const first_sf = first_tile + E;  // [E] first row of the expert's tile-ordered scale chunks at its owner
    uint32_t* const bm_of = first_sf + E;       // [P] block-M of each rank's pool
    uint32_t* const pair_of = bm_of + P;        // [P] 1: the rank's GEMMs run in the pair regime for this call
    uint32_t* const misc = pair_of + P;         // [8] abort word, own pool blocks, own valid routes
    int* const slice_expert = reinterpret_cast<int*>(misc + 8);
    uint32_t* const slice_row = reinterpret_cast<uint32_t*>(slice_expert + slice);
    uint32_t* const slice_pos = slice_row + slice;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    ptx::launch_dependents();
    uint8_t* const my_arena = reinterpret_cast<uint8_t*>(p.arena_base[p.rank]);
    // Calls alternate between the two halves of every double-buffered counter;
    // the combine kernel bumps the call counter when a call retires, so replays
    // of a captured graph alternate without host involvement.
    const uint32_t epoch = *reinterpret_cast<const uint32_t*>(my_arena + p.off_recv_parity);
    const uint32_t gen = epoch & 1u;

    WaitCtl ctl;
    ctl.status = p.status;
    ctl.failed = reinterpret_cast<uint32_t*>(my_arena + p.off_exchange + exchange::kFailed);
    ctl.abort = misc;
    ctl.timeout_ns = p.timeout_ns;
    ctl.kernel = kKernelDispatch;

    // After a wait of an earlier call gave up the workspace's protocol state is void:
    // do nothing (the host raises when it reads the status block) instead of waiting again.
    if (*ctl.failed != 0u) return;
    for (uint32_t i = tid; i < 2 * E; i += kDispatchThreads) own[i] = 0;
    if (tid < 8) misc[tid] = 0;
    __syncthreads();
    // A route is valid iff its expert id, compared as unsigned 64-bit, is below
    // the expert count (negative ids mean "no route").
    for (uint32_t a = tid; a < routes; a += kDispatchThreads) {
        const unsigned long long e = static_cast<unsigned long long>(p.topk_idx[a]);
        if (e < E) {
            atomicAdd(&own[e], 1u);
            if (a < lo) atomicAdd(&before[e], 1u);
        }
    }
    __syncthreads();

    if (P > 1) {
        // ---- all-to-all of the counts: CTA c serves peers c, c + grid, ...
        for (uint32_t peer = blockIdx.x; peer < P; peer += gridDim.x) {
            uint8_t* const ex = reinterpret_cast<uint8_t*>(p.arena_base[peer]) + p.off_exchange;
            uint32_t* const counts = reinterpret_cast<uint32_t*>(ex + exchange::kCounts) +
                                     (static_cast<size_t>(gen) * P + p.rank) * E;
            for (uint32_t e = tid; e < E; e += kDispatchThreads) counts[e] = own[e];
            if (tid == 0)
                reinterpret_cast<uint32_t*>(ex + exchange::kSourceBlockM)[gen * kMaxRanks + p.rank] =
                    p.block_m | (p.dual ? kBlockMDualFlag : 0u);
        }
        __syncthreads();
        // One thread per served peer raises that peer's flag, all at once: each release
        // waits for the round trip of the stores above, so a loop over the peers would
        // pay it once per peer (a CTA serves every peer when the call has few tokens).
        // The releases are cumulative over the CTA's stores ordered before them by the
        // barrier.
        {
            const uint32_t peer = blockIdx.x + tid * gridDim.x;
            if (peer < P) {
                uint8_t* const ex = reinterpret_cast<uint8_t*>(p.arena_base[peer]) + p.off_exchange;
                ptx::st_release_sys(reinterpret_cast<uint32_t*>(ex + exchange::kCountsReady) + gen * kMaxRanks + p.rank,
                                    epoch + 1u);
            }
        }
        // ---- wait for every source's counts (one lane per source, bounded)
        const uint8_t* const ex = my_arena + p.off_exchange;
        for (uint32_t s = tid; s < P; s += kDispatchThreads)
            flag_wait_eq(reinterpret_cast<const uint32_t*>(ex + exchange::kCountsReady) + gen * kMaxRanks + s,
                         epoch + 1u, ctl, 1);
        __syncthreads();
        if (*ctl.abort) return;        // the whole CTA leaves together; the host reads the status block
        const uint32_t* const counts = reinterpret_cast<const uint32_t*>(ex + exchange::kCounts) +
                                       static_cast<size_t>(gen) * P * E;
        for (uint32_t e = tid; e < E; e += kDispatchThreads) {
            uint32_t n = 0, below = 0;
            for (uint32_t s = 0; s < P; ++s) {
                const uint32_t c = counts[static_cast<size_t>(s) * E + e];
                if (s < p.rank) below += c;
                n += c;
            }
            total[e] = n;
            lower[e] = below;
        }
        for (uint32_t s = tid; s < P; s += kDispatchThreads)
            bm_of[s] = reinterpret_cast<const uint32_t*>(ex + exchange::kSourceBlockM)[gen * kMaxRanks + s];
    } else {
        for (uint32_t e = tid; e < E; e += kDispatchThreads) { total[e] = own[e]; lower[e] = 0; }
        if (tid == 0) bm_of[0] = p.block_m | (p.dual ? kBlockMDualFlag : 0u);
    }
    __syncthreads();

    // Pool-block prefix, GEMM-tile prefix and scale-chunk prefix of every owner's
    // local experts (warp w: owners w, w+16, ...).  The GEMMs tile an expert's rows
    // by expert_tile_rows(BM of the owner, rows of the expert) tokens rather than by
    // pool blocks, and read the scale words of a tile from a chunk of its own
    // (the tile's rows rounded up to 128) in the tile-ordered copy.
    const bool tile_ordered = p.private_sf_row != 0u;
    for (uint32_t r = warp; r < P; r += kDispatchThreads / 32) {
        const uint32_t word = bm_of[r], bm = word & 0xFFFFu, base = r * EL;
        __syncwarp();
        if (lane == 0) bm_of[r] = bm;          // from here on the plain block-M
        const uint32_t per_lane = (EL + 31) / 32;
        // the owner's GEMM regime for this call, from the rows its experts received
        uint32_t rows_all = 0, rows_large = 0;
        for (uint32_t l = lane; l < EL; l += 32) {
            const uint32_t n = total[base + l];
            rows_all += n;
            rows_large += n >= kPairExpertRows ? n : 0u;
        }
        for (uint32_t d = 16; d > 0; d >>= 1) {
            rows_all += __shfl_xor_sync(0xffffffffu, rows_all, d);
            rows_large += __shfl_xor_sync(0xffffffffu, rows_large, d);
        }
        const bool pair = pair_chosen((word & kBlockMDualFlag) != 0u, rows_large, rows_all);
        if (lane == 0) pair_of[r] = pair ? 1u : 0u;
        uint32_t sum = 0, tsum = 0, ssum = 0;
        for (uint32_t i = 0; i < per_lane; ++i) {
            const uint32_t l = lane * per_lane + i;
            if (l < EL) {
                const uint32_t n = total[base + l], tn = routed_tile_rows(bm, n, tile_ordered, pair);
                sum += (n + bm - 1) / bm;
                tsum += (n + tn - 1) / tn;
                ssum += (n + tn - 1) / tn * round_up_u32(tn, 128);
            }
        }
        uint32_t incl = sum, tincl = tsum, sincl = ssum;
        for (uint32_t d = 1; d < 32; d <<= 1) {
            const uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
            const uint32_t tv = __shfl_up_sync(0xffffffffu, tincl, d);
            const uint32_t sv = __shfl_up_sync(0xffffffffu, sincl, d);
            if (lane >= d) { incl += v; tincl += tv; sincl += sv; }
        }
        uint32_t run = incl - sum, trun = tincl - tsum, srun = sincl - ssum;
        for (uint32_t i = 0; i < per_lane; ++i) {
            const uint32_t l = lane * per_lane + i;
            if (l < EL) {
                const uint32_t n = total[base + l], tn = routed_tile_rows(bm, n, tile_ordered, pair);
                first_block[base + l] = run;
                first_tile[base + l] = trun;
                first_sf[base + l] = srun;
                run += (n + bm - 1) / bm;
                trun += (n + tn - 1) / tn;
                srun += (n + tn - 1) / tn * round_up_u32(tn, 128);
            }
        }
        if (r == p.rank && lane == 31) { misc[1] = incl; misc[3] = tincl; }   // pool blocks, GEMM tiles of this rank
    }
    if (blockIdx.x == 0) {
        uint32_t mine = 0;
        for (uint32_t e = tid; e < E; e += kDispatchThreads) mine += own[e];
        for (uint32_t d = 16; d > 0; d >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, d);
        if (lane == 0) atomicAdd(&misc[2], mine);            // valid routes of this rank
    }
    __syncthreads();

    const uint32_t first_local = p.rank * EL;
    if (blockIdx.x == 0) {
        // Tile counters of this call's row tiles start from zero.
        for (uint32_t i = tid; i <= misc[3]; i += kDispatchThreads) p.done_routed[i] = 0;
        if (p.done_shared != nullptr)
            for (uint32_t i = tid; i <= (p.num_tokens + p.block_m - 1) / p.block_m; i += kDispatchThreads)
                p.done_shared[i] = 0;
        // ---- what this rank receives: the reference's count products and the
        // tables the GEMM kernels schedule from
        unsigned long long* recv = reinterpret_cast<unsigned long long*>(my_arena + p.off_recv_count) +
            static_cast<size_t>(gen) * P * EL;
        unsigned long long* recv_sum = reinterpret_cast<unsigned long long*>(my_arena + p.off_recv_count_sum) +
            static_cast<size_t>(gen) * EL;
        const uint32_t* const counts = reinterpret_cast<const uint32_t*>(my_arena + p.off_exchange + exchange::kCounts) +
            static_cast<size_t>(gen) * P * E;
        for (uint32_t l = tid; l < EL; l += kDispatchThreads) {
            const uint32_t n = total[first_local + l];
            p.expert_count[l] = static_cast<int>(n);
            p.expert_block_start[l] = static_cast<int>(first_block[first_local + l]);
            p.expert_tile_start[l] = static_cast<int>(first_tile[first_local + l]);
            p.expert_row_start[l] = static_cast<int>(first_block[first_local + l] * p.block_m);
            // tiles that are the pool blocks read the scale words where the reference layout has them
            p.expert_sf_start[l] = static_cast<int>(tile_ordered ? first_sf[first_local + l]
                                                                 : first_block[first_local + l] * round_up_u32(p.block_m, 128));
            for (uint32_t s = 0; s < P; ++s)
                recv[static_cast<size_t>(s) * EL + l] = P > 1 ? counts[static_cast<size_t>(s) * E + first_local + l] : n;
            // high word: number of source ranks that have reported
            recv_sum[l] = (static_cast<unsigned long long>(P) << 32) | n;
            if (p.stats != nullptr) p.stats[l] += static_cast<int>(n);
        }
        {
            // Counters of the NEXT call's generation start from zero; nobody can be
            // adding to them yet (a peer reaches its next call only after this
            // rank has finished the current one).  The last call of that generation
            // left as many row-tile counters dirty as it had row tiles.
            uint8_t* const ex = my_arena + p.off_exchange;
            uint32_t* const used = reinterpret_cast<uint32_t*>(ex + exchange::kTilesUsed);
            uint32_t* const arrived_next = reinterpret_cast<uint32_t*>(ex + exchange::kTileArrived) + (gen ^ 1u) * exchange::kMaxRowTiles;
            const uint32_t dirty = used[gen ^ 1u];
            for (uint32_t i = tid; i < dirty; i += kDispatchThreads) arrived_next[i] = 0;
            if (tid == 0) {
                used[gen] = misc[3];
                *reinterpret_cast<uint32_t*>(ex + exchange::kCombineArrived + (gen ^ 1u) * 128) = 0;
            }
        }
        if (tid == 0) {
            p.expert_block_start[EL] = static_cast<int>(misc[1]);
            p.expert_tile_start[EL] = static_cast<int>(misc[3]);
            *reinterpret_cast<uint32_t*>(my_arena + p.off_routed_pool_blocks) = misc[1];
            p.call_info[kCallGeneration] = gen;
            p.call_info[kCallCombineRows] = misc[2];
            p.call_info[kCallEpoch] = epoch;
            p.call_info[kCallPairRegime] = pair_of[p.rank];
            if (p.shared_table != nullptr) {
                p.shared_table[0] = static_cast<int>(p.num_tokens);
                p.shared_table[1] = 0;
                p.shared_table[2] = static_cast<int>((p.num_tokens + p.block_m - 1) / p.block_m);
                p.shared_table[3] = 0;     // the shared expert's rows start at token 0
                p.shared_table[4] = 0;     // ... and so do its scale chunks
            }
        }
        // The GEMM launch of this call is already running (it was allowed to start when
        // this kernel did): hand it the tables.  The barrier orders every thread's
        // writes above before the release.
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.call_info + kCallTablesReady), "r"(epoch + 1u)
                         : "memory");
        }
    }

    // Destination of every route in this CTA's slice.
    for (uint32_t a = lo + tid; a < hi; a += kDispatchThreads) {
        const unsigned long long e64 = static_cast<unsigned long long>(p.topk_idx[a]);
        slice_expert[a - lo] = e64 < E ? static_cast<int>(e64) : -1;
    }
    __syncthreads();
    for (uint32_t a = lo + tid; a < hi; a += kDispatchThreads) {
        const int e = slice_expert[a - lo];
        uint32_t row = 0xFFFFFFFFu;
        if (e >= 0) {
            uint32_t i = before[e];                       // position among this source's routes to e
            for (uint32_t j = 0; j < a - lo; ++j) i += (slice_expert[j] == e);
            const uint32_t owner = static_cast<uint32_t>(e) / EL;
            const uint32_t l = static_cast<uint32_t>(e) - owner * EL;
            // Position inside the expert's rows: sources one after the other up to
            // 8 ranks; above that the sources are interleaved (round j takes the j-th
            // route of every source that has more than j, sources ascending), the
            // reference's order for large groups (impls/sm100_fp8_fp4_gc_moe.py:954-986).
            uint32_t pos = lower[e] + i;
            if (P > 8) {
                const uint32_t* const counts = reinterpret_cast<const uint32_t*>(my_arena + p.off_exchange + exchange::kCounts) +
                                               static_cast<size_t>(gen) * P * E + e;
                pos = 0;
                for (uint32_t s = 0; s < P; ++s) {
                    const uint32_t c = counts[static_cast<size_t>(s) * E];
                    pos += min(c, i) + ((s < p.rank && c > i) ? 1u : 0u);
                }
            }
            row = first_block[e] * bm_of[owner] + pos;
            uint8_t* const dst_arena = reinterpret_cast<uint8_t*>(p.arena_base[owner]);
            if (i < p.capacity)
                reinterpret_cast<uint32_t*>(dst_arena + p.off_index_table)[
                    (static_cast<size_t>(l) * P + p.rank) * p.capacity + i] = a;
            uint32_t* meta = reinterpret_cast<uint32_t*>(dst_arena + p.off_metadata) + static_cast<size_t>(row) * 3;
            meta[0] = p.rank;
            meta[1] = a / p.topk;
            meta[2] = a % p.topk;
            reinterpret_cast<float*>(dst_arena + p.off_l1_weights)[row] = p.topk_weights[a];
        }
        slice_row[a - lo] = row;
        slice_pos[a - lo] = row == 0xFFFFFFFFu ? 0u : row - first_block[e >= 0 ? e : 0] * bm_of[(e >= 0 ? e : 0) / EL];
    }
    __syncthreads();

    // One warp per route: copy the FP8 row (16 bytes per lane and load), scatter
    // its packed scale words into the owner's MN-major scale ring, then tell the
    // owner one more row of that expert has landed.
    const uint32_t row_vecs = p.hidden / 16, sf_words = p.hidden / 128;
    // Arrivals leave in batches of up to kArrivalBatch rows per warp: lane j keeps the counter of
    // the j-th row of the batch, and one fence per lane covers the stores of all of them, so
    // a warp with several rows waits for the round trip of its stores once per batch instead
    // of once per row.
    constexpr uint32_t kArrivalBatch = 4;
    uint32_t* pending = nullptr;
    uint32_t num_pending = 0;
    auto flush_arrivals = [&]() {
        __syncwarp();
        if (lane < num_pending) {
            if (P > 1) asm volatile("fence.acq_rel.sys;\n\tred.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(pending), "r"(1u) : "memory");
            else asm volatile("fence.acq_rel.gpu;\n\tred.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(pending), "r"(1u) : "memory");
        }
        num_pending = 0;
    };
    for (uint32_t a = lo + warp; a < hi; a += kDispatchThreads / 32) {
        const uint32_t row = slice_row[a - lo];
        if (row == 0xFFFFFFFFu) continue;
        const uint32_t e = static_cast<uint32_t>(slice_expert[a - lo]);
        const uint32_t owner = e / EL;
        const uint32_t bm = bm_of[owner], sf_block = round_up_u32(bm, 128);
        uint8_t* const dst_arena = reinterpret_cast<uint8_t*>(p.arena_base[owner]);
        const uint32_t t = a / p.topk;
        const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(t) * p.hidden);
        uint4* dst = reinterpret_cast<uint4*>(dst_arena + p.off_l1_acts + static_cast<size_t>(row) * p.hidden);
        // The row's first 64 scale words and sixteen 16-byte loads per lane are in flight
        // before the first store: one memory latency per 8 KiB of row.
        uint32_t sf_first[2];
#pragma unroll
        for (uint32_t j = 0; j < 2; ++j)
            if (lane + j * 32 < sf_words) sf_first[j] = p.x_sf[static_cast<size_t>(t) * sf_words + lane + j * 32];
        for (uint32_t v0 = lane; v0 < row_vecs; v0 += 512) {
            uint4 part[16];
#pragma unroll
            for (uint32_t j = 0; j < 16; ++j)
                if (v0 + j * 32 < row_vecs) part[j] = src[v0 + j * 32];
#pragma unroll
            for (uint32_t j = 0; j < 16; ++j)
                if (v0 + j * 32 < row_vecs) dst[v0 + j * 32] = part[j];
        }
        const uint32_t block = row / bm, u = row - block * bm;
        const uint32_t sf_row = block * sf_block + sf_row_in_block(u);
        uint32_t* sf_dst = reinterpret_cast<uint32_t*>(dst_arena + p.off_l1_acts_sf);
        // second copy, ordered by GEMM tile: the one the owner's GEMM launch reads
        const uint32_t tn = routed_tile_rows(bm, total[e], tile_ordered, pair_of[owner] != 0u);
        const uint32_t pos = slice_pos[a - lo];
        const uint32_t tile_row = p.private_sf_row + first_sf[e] + (pos / tn) * round_up_u32(tn, 128) +
                                  sf_row_in_block(pos % tn);
        for (uint32_t w = lane, j = 0; w < sf_words; w += 32, ++j) {
            const uint32_t word = j == 0 ? sf_first[0] : j == 1 ? sf_first[1] : p.x_sf[static_cast<size_t>(t) * sf_words + w];
            sf_dst[static_cast<size_t>(w) * p.sf_ring + sf_row] = word;
            if (tile_ordered) sf_dst[static_cast<size_t>(w) * p.sf_ring + tile_row] = word;
        }
        // Tell the owner's GEMM launch (which may already be running, on this GPU too)
        // that one more row of this GEMM row tile has landed: fence + relaxed add, a release
        // cumulative over the warp's stores ordered by __syncwarp.
        if (lane == num_pending)
            pending = reinterpret_cast<uint32_t*>(dst_arena + p.off_exchange + exchange::kTileArrived) +
                      gen * exchange::kMaxRowTiles + first_tile[e] + pos / tn;
        if (++num_pending == kArrivalBatch) flush_arrivals();
    }
    flush_arrivals();
}

}  // namespace gcmoe
