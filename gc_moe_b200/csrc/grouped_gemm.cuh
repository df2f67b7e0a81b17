// Persistent grouped block-scaled GEMM over the receive pool, one CTA per SM.
//
//   out[weight_row, token] = sum_k W[e][weight_row, k] * X[token, k]
//
// per row tile (consecutive tokens of one local expert) and 256-row weight
// tile.  Weights are the MMA's A operand, tokens its B operand (N = the tile's
// rows rounded up to 16), so decode-sized token counts waste no tensor rows and
// the HBM stream is the weight stream.  Two instantiations (device_common.cuh,
// pair_mode):
//
//  * kPair = false, decode: one CTA per tile, two M = 128 halves, cta_group::1.
//  * kPair = true, large-token: the two CTAs of a cluster share a tile.  Each CTA
//    loads its own 128 weight rows and its own half of the token rows (per-CTA TMA
//    loads that report to the leader CTA's stage barrier; no cluster multicast),
//    one thread of the leader issues tcgen05.mma.cta_group::2 for both, and each
//    CTA's TMEM holds the accumulator of its 128 weight rows x all tokens, which
//    its own epilogue warps drain.  Both CTAs' barriers are signalled by two plain
//    tcgen05.commit (local, then the peer's shared::cluster address).  A pipeline
//    stage of a pair holds two K128 blocks: the TMA unit of an SM spends about
//    65 ns per request whatever its size (measured: four requests per stage bound
//    the stage at 0.3 us in both regimes, independent of the MMA work), and a
//    CTA of a pair fetches only half a weight tile per request.
//
// Roles (288 threads per CTA):
//   warp 0    weight producer: per K128 stage one TMA tile (packed FP4, unpacked to
//             8-bit containers on the fly; FP8 for the shared expert) + its scale words
//   warp 2    activation producer: the stage's token tile + scale words
//   warp 1,3  MMA issuers.  Decode: one per 128-row half of the tile, each with its
//             own TMEM accumulator and scale columns (with decode-sized N a
//             tcgen05.mma does so little work that instruction issue bounds the
//             kernel, so the halves are issued in parallel).  Pair: warp 1 of the
//             leader CTA alone.  Warp 1 owns the TMEM allocation.
//   warp 4-7  epilogue: read the FP32 accumulators from TMEM (each warp its own
//             32-lane quarter), fuse the layer's element-wise tail, store
//   warp 8    tile scheduler: claims the next tile from a cursor all CTAs share,
//             one tile ahead of the weight producer (pair: the leader's, which
//             publishes to both CTAs)
// Every async instruction is issued under elect.sync by a converged warp: the
// compiler then feeds TMA / tcgen05 operands from uniform registers, which
// measured 1.5x faster than the same code under `lane == 0`.
// Two accumulator stages let the epilogue of tile i overlap the main loop of
// tile i+1.  The work list is tile t = row_tile * n_tiles + n_tile over the
// segments [shared up | routed up | shared down | routed down]; CTA (pair) c
// starts on tile c and then takes whatever tile is next, so the CTAs that share
// a row tile run at about the same time and its activation tile is served from L2.
//
// The launch starts while the dispatch kernel of the same call is still running
// (programmatic dependent launch, no griddepcontrol.wait in front): it waits for
// the call's tables (a release by dispatch CTA 0), then per row tile for the rows
// pushed into the pool (arrival counters, this GPU's own dispatch included), so
// the weight stream and the first tiles of every expert overlap the exchange.
//
// Replaces the reference's role-2 compute kernel
// (gc_moe/impls/sm100_fp8_fp4_gc_moe.py:1108-1905) and its device scheduler
// (gc_moe/scheduler/gc_moe.py:284-328) without ring flow control (the pool is
// not reused inside a call).
#pragma once

#include <cuda_bf16.h>

#include "device_common.cuh"

namespace gcmoe {

constexpr int kGemmThreads = 288;           // eight role warps and the tile scheduler warp
constexpr int kHalfRows = 128;             // MMA M per CTA: rows of one accumulator
constexpr int kTileRows = 256;             // weight rows per tile (two halves)
constexpr int kTileK = 128;                // K per pipeline stage = 4 MMAs of K32
constexpr int kHalfStageBytes = 128 * 128;   // FP4 is unpacked to 8-bit containers by the TMA
constexpr int kSfChunkBytes = 512;         // 128 rows x one packed int32 of four UE8M0 bytes
constexpr int kMaxStages = 16;
constexpr int kSmemLimit = 232448;         // opt-in dynamic shared memory per CTA on sm_100
constexpr int kMaxActMaps = 8;             // activation boxes of different heights per segment

// What a segment's tiles compute after the K loop.
enum SegmentKind : uint32_t {
    kSegUp = 0,     // gate/up projection: SwiGLU, route weight, FP8 requantisation -> intermediate
    kSegDown = 1    // down projection: BF16 rows scattered to the source rank's combine slots
};
constexpr uint32_t kFeedSlots = 32;   // ring of claimed tiles per CTA; the roles are never more than ~8 tiles apart
constexpr int kMaxSegments = 4;   // shared up, routed up, shared down, routed down

// One grouped problem of a launch: the up or the down projection of the routed
// experts of this rank, or of the fused shared expert (one "expert" whose rows
// are this rank's own tokens, FP8 weights).  One launch runs all of them as one
// work list -- shared up, routed up, shared down, routed down -- so that a CTA
// that runs out of up tiles continues with down tiles instead of idling at a
// kernel boundary.  The shared tiles come first because they depend on nothing
// another GPU sends and so hide the dispatch exchange.  A down tile needs every
// up tile of its row tile: up epilogues count finished tiles per row tile in
// `block_done` and the down tile's activation producer waits for the count.
// All up tiles precede all down tiles in every CTA's order and every CTA of the
// grid is resident (grid <= SMs, one CTA per SM), so the wait cannot deadlock.
struct GemmSegment {
    CUtensorMap tm_act[kMaxActMaps];   // u8 [rows][K], box 128 x act_box_rows[i], 128-byte swizzle
                                       // (pair: viewed as [K/128][rows][128], box 128 x rows x 2 K blocks)
    CUtensorMap tm_w;       // FP4: 16U4_ALIGN16B [E][K/128][rows][128]; FP8: u8 [K/128][rows][128];
                            // box 128 x 256 (pair: 128 x 128 x 2 K blocks, one half per CTA)
    CUtensorMap tm_act_sf;  // pair only: u32 [K/128][act_sf_stride], box 128 x 2 K blocks
    CUtensorMap tm_w_sf;    // pair only: u32 [experts x planes][w_sf_stride], box 128 x 2 planes
    uint32_t act_box_rows[kMaxActMaps];   // ascending; a tile fetches the smallest box that holds its rows
    uint32_t num_act_maps;
    const uint32_t* act_sf;  // packed scale words, MN-major: word (kb, r) at kb * act_sf_stride + r
    const uint32_t* w_sf;    // word (e, plane, row) at (e * planes + plane) * w_sf_stride + row
    const int* tile_start;   // [experts + 1] prefix of the experts' tile counts
    const int* count;        // [experts] rows per expert
    const int* row_start;    // [experts] first row of the expert in the activation tensor
    const int* sf_start;     // [experts] first scale row of the expert's tiles in act_sf (and out_sf_private)
    uint32_t tile_rows;      // rows per tile of every expert, or 0: expert_tile_rows(regime, rows of the expert)
    uint32_t act_sf_stride;  // words between consecutive K128 planes of act_sf
    uint32_t w_sf_stride;    // words between consecutive planes of w_sf
    uint32_t w_sf_kblocks;   // K128 blocks one w_sf word covers: 1 (K32 scales) or 4 (K128 scales)
    uint32_t w_rows;         // weight rows per expert (2I for the gate/up GEMM, H for the down GEMM)
    uint32_t k_blocks;       // K / 128
    uint32_t n_tiles;        // w_rows / 256
    uint32_t experts;
    uint32_t weight_format;  // 5 = e2m1 (FP4), 0 = e4m3
    uint32_t weight_tx_bytes;  // bytes the TMA of 256 weight rows reports to the stage barrier
    uint32_t shared;         // rows are own tokens: no route weight, no arrival wait, output slot = topk
    uint32_t kind;           // SegmentKind
    uint32_t* block_done;    // [row tiles] up: tiles finished; down: what to wait for
    uint32_t done_target;    // down: up-tile completions per row tile (0 = do not wait)
    // ---- gate/up epilogue
    uint8_t* out_acts;        // e4m3 [rows][I]
    uint8_t* out_sf;          // bytes of the MN-major packed scale ring
    const float* route_weight;  // [rows], unused for the shared segment
    uint32_t out_sf_stride;   // words between K128 planes of out_sf
    uint32_t ref_block_m;     // block-M of the pool layout: where out_sf rows go in the reference layout
    uint32_t out_sf_private;  // row offset, inside each plane, of the tile-ordered copy the down tiles
                              // read (0 = tiles coincide with pool blocks, no second copy)
    uint32_t inter;           // row length of out_acts
    // ---- down epilogue
    const uint32_t* metadata;  // (src_rank, src_token, slot) per pool row, unused for the shared segment
};

struct GemmParams {
    GemmSegment seg[kMaxSegments];
    uint32_t num_segments;
    uint32_t* status;
    uint64_t timeout_ns;
    uint32_t block_m;        // largest tile of the launch: accumulator stride in TMEM columns
    uint32_t sf_block_m;     // that, rounded up to 128: scale rows of an activation stage
    uint32_t stages;
    uint32_t acc_stages;     // 2, or 1 when two accumulator stages exceed TMEM
    uint32_t table_words;    // shared-memory words for the segments' tables
    uint32_t tmem_cols;
    float clamp;
    uint32_t has_clamp;
    uint32_t fast_math;
    // ---- down epilogue
    uint64_t combine_base[kMaxRanks];  // address of combine_tokens on each rank
    uint32_t capacity;
    uint32_t hidden;
    uint32_t topk;
    uint32_t rank;
    // ---- raw epilogue (test hook): FP32 accumulators of segment 0, [rows][w_rows]
    float* raw_out;
    // ---- hand-over from the dispatch kernel and arrival counters
    const uint32_t* call_info;        // [kCallInfoWords] written by the dispatch kernel
    const uint32_t* epoch_word;       // the workspace's call counter (recv_parity)
    uint32_t wait_tables;             // 1: launched with the call's dispatch kernel, wait for its tables
    uint32_t dual_regime;             // 1: both regimes' launches are enqueued, call_info says which one works
    const uint32_t* tile_arrived;     // this rank's exchange::kTileArrived, [2][kMaxRowTiles]: rows landed per row tile
    uint32_t* failed;                 // this rank's exchange::kFailed
    uint64_t combine_arrived[kMaxRanks];  // address of exchange::kCombineArrived on each rank
    uint32_t num_ranks;
    uint32_t* tile_cursor;   // claims made so far by this launch's CTAs beyond their first tile (zero between launches)
};

struct GemmSmemLayout {
    uint32_t w, a, sfw, sfa, bars, tables, amax, arrive, feed, rows, out, total;
    uint32_t w_stage, a_stage, sfw_stage, sfa_stage;   // bytes per pipeline stage
};
constexpr uint32_t kPairStageBlocks = 2;   // K128 blocks per pipeline stage of a CTA pair

// `block_m`: largest tile of the launch.  A CTA of a pair holds half of the
// weight tile and half of the token tile, and the scale words of all tokens.
__host__ __device__ inline GemmSmemLayout gemm_smem_layout(uint32_t stages, uint32_t block_m,
                                                           uint32_t sf_block_m,
                                                           uint32_t table_words, bool pair) {
    GemmSmemLayout l;
    // single CTA: both 128-row halves of one K128 block; CTA of a pair: its half, two K128 blocks
    l.w_stage = 2 * kHalfStageBytes;
    l.a_stage = pair ? 2 * round_up_u32(block_m / 2 * kTileK, 1024) : round_up_u32(block_m * kTileK, 1024);
    l.sfw_stage = 2 * kSfChunkBytes;
    l.sfa_stage = (pair ? 2 : 1) * sf_block_m * 4;
    l.w = 0;
    l.a = l.w + stages * l.w_stage;
    l.sfw = l.a + stages * l.a_stage;
    l.sfa = l.sfw + stages * l.sfw_stage;
    l.bars = l.sfa + stages * l.sfa_stage;
    // full[stages], empty[stages], acc_full[2], acc_empty[2], drain[2], then the
    // TMEM base slot and the abort word
    l.tables = l.bars + (2 * stages + 6) * 8 + 16;
    l.amax = l.tables + round_up_u32((table_words + 16) * 4, 16);   // tables + per-segment offsets and tile prefix
    l.arrive = l.amax + 2 * 4 * 16 * 4;               // amax exchange [2][4][16] floats
    l.feed = l.arrive + kMaxRanks * 4;                // rows x halves written per source rank by this CTA
    l.rows = l.feed + (kFeedSlots + 2) * 8;           // ring of claimed tiles {sequence number, tile}, producer position
    l.out = round_up_u32(l.rows + 2 * block_m * 16, 16);   // per-tile row info, double buffered
    l.total = l.out + 2 * 16 * kHalfRows * 2;          // output transpose: [2][16 tokens][128 channels] bf16
    return l;
}

__host__ inline uint32_t gemm_pick_stages(uint32_t block_m, uint32_t sf_block_m,
                                          uint32_t table_words, bool pair) {
    for (uint32_t s = kMaxStages; s >= 2; --s) {
        if (gemm_smem_layout(s, block_m, sf_block_m, table_words, pair).total + 1024 <= kSmemLimit)
            return s;
    }
    return 0;
}

// TMEM columns of a CTA: per accumulator stage one FP32 accumulator of block_m
// columns per 128-row half it computes (two halves for a single CTA, one for a
// CTA of a pair), then per half 4 columns of weight scales and sf_block_m / 32
// columns of activation scales.
__host__ __device__ inline uint32_t gemm_tmem_columns(uint32_t block_m, uint32_t sf_block_m,
                                                      uint32_t acc_stages, bool pair) {
    const uint32_t halves = pair ? 1u : 2u;
    return acc_stages * halves * block_m + halves * (4 + sf_block_m / 32);
}

// SwiGLU in the reference's op order (impls:122-171): BF16-round the two
// accumulators, clamp in BF16, FP32 sigmoid, x up, x route weight.
__device__ __forceinline__ float swiglu_weighted(float gate_acc, float up_acc, float route_w,
                                                 float clamp_bf16, bool has_clamp,
                                                 bool fast_math) {
    float g = __bfloat162float(__float2bfloat16_rn(gate_acc));
    float u = __bfloat162float(__float2bfloat16_rn(up_acc));
    if (has_clamp) {
        g = fminf(g, clamp_bf16);
        u = fminf(fmaxf(u, -clamp_bf16), clamp_bf16);
    }
    float gate;
    if (fast_math) {
        const float e = ptx::ex2_approx(__fmul_rn(g, -1.44269502162933349609375f));
        gate = __fmul_rn(g, ptx::rcp_approx_ftz(__fadd_rn(1.0f, e)));
    } else {
        gate = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
    }
    return __fmul_rn(__fmul_rn(gate, u), route_w);
}

// Biased exponent of 2^ceil(log2(amax / 448)), floored at 2^-22
// (gc_moe/common/math.py:146-154).
__device__ __forceinline__ uint32_t ue8m0_scale_byte(float amax) {
    uint32_t e = (__float_as_uint(amax) + 0x7FFFFFu - 0x600000u) >> 23;
    return (e > 113u ? e : 113u) - 8u;
}

// AND of a predicate over the 128 epilogue threads (named barrier 2).
__device__ __forceinline__ bool all_epilogue_threads(bool pred) {
    uint32_t all;
    asm volatile(
        "{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.and.pred p, 2, 128, q; "
        "selp.u32 %0, 1, 0, p; }"
        : "=r"(all)
        : "r"(static_cast<uint32_t>(pred))
        : "memory");
    return all != 0;
}
__device__ __forceinline__ void epilogue_barrier() {
    asm volatile("bar.sync 1, 128;" ::: "memory");
}

// Position in the stage ring after `steps` more stages.
struct StageCursor {
    uint32_t stage = 0, phase = 0;
    __device__ __forceinline__ void advance(uint32_t steps, uint32_t stages) {
        stage += steps;
        while (stage >= stages) { stage -= stages; phase ^= 1u; }
    }
};

// Where a tile of the launch's work list lives: which segment, which row tile
// of which expert, which 256-row slice of the expert's weights.
struct TileCoord {
    uint32_t seg, block, n_tile, expert, valid, row0, sf_row, tiles_of_expert;   // block: tile index inside the segment
};

template <bool kRaw, bool kPair>
__global__ void __launch_bounds__(kGemmThreads, 1)
grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;   // swizzled tiles need 1024-byte alignment
    uint8_t* const gbase = smem_raw + (base - raw_addr);

    const GemmSmemLayout L = gemm_smem_layout(p.stages, p.block_m, p.sf_block_m, p.table_words, kPair);
    const uint32_t bar_full = base + L.bars;
    const uint32_t bar_empty = bar_full + p.stages * 8;
    const uint32_t bar_acc_full = bar_empty + p.stages * 8;
    const uint32_t bar_acc_empty = bar_acc_full + 16;
    const uint32_t bar_drain = bar_acc_empty + 16;
    volatile uint32_t* const tmem_slot = reinterpret_cast<volatile uint32_t*>(gbase + L.bars + (2 * p.stages + 6) * 8);
    volatile uint32_t* const abort_word = tmem_slot + 1;
    int* const tables = reinterpret_cast<int*>(gbase + L.tables);
    float* const amax_x = reinterpret_cast<float*>(gbase + L.amax);       // [2][4][16]
    uint32_t* const arrive = reinterpret_cast<uint32_t*>(gbase + L.arrive);  // [kMaxRanks]
    // Slot n % kFeedSlots holds {n + 1, n-th tile of this CTA} as one 8-byte word.
    volatile unsigned long long* const feed_ring = reinterpret_cast<volatile unsigned long long*>(gbase + L.feed);   // [kFeedSlots]
    volatile uint32_t* const feed_pos = reinterpret_cast<volatile uint32_t*>(gbase + L.feed + kFeedSlots * 8);   // tiles the weight producer has started
    uint32_t* const row_info = reinterpret_cast<uint32_t*>(gbase + L.rows);  // [2][BM][4]
    __nv_bfloat16* const out_stage = reinterpret_cast<__nv_bfloat16*>(gbase + L.out);  // [2][16][128]

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    // A pair is a cluster of two CTAs: rank 0 leads (issues the MMAs, owns the stage
    // barriers the producers report to, claims tiles), rank 1 follows.
    const uint32_t cta = kPair ? ptx::cluster_ctarank() : 0u;
    const uint32_t unit = kPair ? blockIdx.x >> 1 : blockIdx.x;          // index of this CTA (pair) among the grid's
    const uint32_t units = kPair ? gridDim.x >> 1 : gridDim.x;

    WaitCtl ctl;
    ctl.status = p.status;
    ctl.failed = p.failed;
    ctl.abort = abort_word;
    ctl.timeout_ns = p.timeout_ns;
    ctl.kernel = kKernelGemmL1;
    if constexpr (kPair) ctl.peer_abort = ptx::mapa(ptx::smem_u32(const_cast<uint32_t*>(abort_word)), cta ^ 1u);

    if constexpr (!kPair) {
        // Both regimes' launches are enqueued, the pair one first.  When the dispatch kernel has
        // already published its choice and it is the pair regime, this launch has nothing to do:
        // leave before setting anything up.  (The pair launch cannot take this shortcut CTA by
        // CTA -- the two CTAs of a cluster must take the same path -- and does not need to: its
        // set-up overlaps the dispatch kernel.)
        if (p.dual_regime != 0u) {
            volatile uint32_t& not_mine = *reinterpret_cast<volatile uint32_t*>(smem_raw);   // stage memory, not in use yet
            if (threadIdx.x == 0) {
                uint32_t ready = 1;
                if (p.wait_tables != 0u) {
                    uint32_t v;
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.call_info + kCallTablesReady) : "memory");
                    ready = v == *reinterpret_cast<const volatile uint32_t*>(p.epoch_word) + 1u;
                }
                not_mine = ready != 0u && *reinterpret_cast<const volatile uint32_t*>(p.call_info + kCallPairRegime) != 0u;
            }
            __syncthreads();
            if (not_mine != 0u) {
                if (threadIdx.x == 0) ptx::grid_dependency_wait();   // retire after the launches before this one
                return;
            }
            __syncthreads();      // everyone has read the word before the set-up below reuses the memory
        }
    }
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; ++s) {
            // stage filled: both producers (of both CTAs of a pair); stage free: the
            // commits of the two MMA warps (pair: one commit per stage)
            ptx::mbar_init(bar_full + 8 * s, kPair ? 4 : 2);
            ptx::mbar_init(bar_empty + 8 * s, kPair ? 1 : 2);
        }
        for (uint32_t i = 0; i < 2; ++i) {
            ptx::mbar_init(bar_acc_full + 8 * i, kPair ? 1 : 2);
            ptx::mbar_init(bar_acc_empty + 8 * i, kPair ? 8 : 4);   // one arrival per epilogue warp (of both CTAs)
            ptx::mbar_init(bar_drain + 8 * i, 1);
        }
        *abort_word = 0;
        for (uint32_t i = 0; i < kFeedSlots; ++i) feed_ring[i] = 0ull;
        *feed_pos = 0;
        ptx::fence_mbar_init();
        for (uint32_t g = 0; g < p.num_segments; ++g) {
            for (uint32_t i = 0; i < p.seg[g].num_act_maps; ++i) ptx::prefetch_tensormap(&p.seg[g].tm_act[i]);
            ptx::prefetch_tensormap(&p.seg[g].tm_w);
            if constexpr (kPair) {
                ptx::prefetch_tensormap(&p.seg[g].tm_act_sf);
                ptx::prefetch_tensormap(&p.seg[g].tm_w_sf);
            }
        }
    }
    if (warp == 1) {
        ptx::tmem_alloc<kPair>(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), p.tmem_cols);
        ptx::tmem_relinquish<kPair>();
    }
    // Everything above reads only kernel parameters.  Let the combine kernel start
    // its prologue, then wait for the tables of this call: the dispatch kernel is
    // still running and hands them over with a release by its CTA 0.
    ptx::launch_dependents();
    if (threadIdx.x == 0 && p.wait_tables != 0u) {
        const uint32_t want = *reinterpret_cast<const volatile uint32_t*>(p.epoch_word) + 1u;
        const uint32_t* const flag = p.call_info + kCallTablesReady;
        const uint64_t t0 = ptx::globaltimer_ns();
        uint32_t spins = 0, v;
        for (;;) {
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v == want) break;
            if ((++spins & 15u) == 0u) {
                // the dispatch kernel returns without tables when the workspace has failed
                if (*reinterpret_cast<const volatile uint32_t*>(p.failed) != 0u) break;
                if (ptx::globaltimer_ns() - t0 > ctl.timeout_ns) {
                    report_failure(ctl, kWaitTimeout, 9, v, want);
                    break;
                }
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    // Tables of every segment: [start (experts + 1) | count | row start | scale start (experts each)],
    // then per segment the table offset and the prefix of tile counts.
    uint32_t* const seg_meta = reinterpret_cast<uint32_t*>(tables + p.table_words);   // [4] offsets, [5] tile prefix
    if (threadIdx.x == 0) {
        uint32_t off = 0;
        for (uint32_t g = 0; g < p.num_segments; ++g) {
            seg_meta[g] = off;
            off += 4 * p.seg[g].experts + 1;
        }
    }
    __syncthreads();
    for (uint32_t g = 0; g < p.num_segments; ++g) {
        const uint32_t ne = p.seg[g].experts;
        int* const start = tables + seg_meta[g];
        for (uint32_t i = threadIdx.x; i <= ne; i += kGemmThreads) start[i] = p.seg[g].tile_start[i];
        for (uint32_t i = threadIdx.x; i < ne; i += kGemmThreads) {
            start[ne + 1 + i] = p.seg[g].count[i];
            start[2 * ne + 1 + i] = p.seg[g].row_start[i];
            start[3 * ne + 1 + i] = p.seg[g].sf_start[i];
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (uint32_t g = 0; g < p.num_segments; ++g) {
            seg_meta[4 + g] = run;
            run += static_cast<uint32_t>(tables[seg_meta[g] + p.seg[g].experts]) * p.seg[g].n_tiles;
        }
        for (uint32_t g = p.num_segments; g <= kMaxSegments; ++g) seg_meta[4 + g] = run;
    }
    __syncthreads();
    // Barriers and abort words of both CTAs are initialised before either touches the other's.
    if constexpr (kPair) ptx::cluster_sync();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t bm = p.block_m;
    // nothing to do once a wait on this workspace has given up
    // ... and nothing when the dispatch kernel chose the other regime for this call
    const bool mine = !p.dual_regime || (p.call_info[kCallPairRegime] != 0u) == kPair;
    const uint32_t total_tiles = (!mine || *reinterpret_cast<const volatile uint32_t*>(p.failed) != 0u || *abort_word != 0u)
                                     ? 0u : seg_meta[4 + kMaxSegments];
    const uint32_t generation = p.call_info[kCallGeneration];

    // Decode a tile index: segment, row tile, 256-row weight slice, owning
    // expert (last e with start[e] <= block) and the tile's valid rows.
    auto locate = [&](uint32_t tile) -> TileCoord {
        TileCoord c;
        c.seg = 0;
#pragma unroll
        for (uint32_t g = 1; g < kMaxSegments; ++g) c.seg += tile >= seg_meta[4 + g] ? 1u : 0u;
        const uint32_t local = tile - seg_meta[4 + c.seg];
        const uint32_t nt = p.seg[c.seg].n_tiles, ne = p.seg[c.seg].experts;
        c.block = local / nt;
        c.n_tile = local - c.block * nt;
        const int* const start = tables + seg_meta[c.seg];
        uint32_t lo = 0, hi = ne;   // start[lo] <= block < start[hi]
        while (hi - lo > 1) {
            const uint32_t mid = (lo + hi) >> 1;
            if (static_cast<uint32_t>(start[mid]) <= c.block) lo = mid; else hi = mid;
        }
        c.expert = lo;
        const uint32_t rows = static_cast<uint32_t>(start[ne + 1 + lo]);
        const uint32_t tn = p.seg[c.seg].tile_rows != 0u ? p.seg[c.seg].tile_rows
                                                         : expert_tile_rows(kPair, rows);
        const uint32_t t = c.block - static_cast<uint32_t>(start[lo]);
        const uint32_t left = rows - t * tn;
        c.valid = left < tn ? left : tn;
        c.row0 = static_cast<uint32_t>(start[2 * ne + 1 + lo]) + t * tn;
        c.sf_row = static_cast<uint32_t>(start[3 * ne + 1 + lo]) + t * round_up_u32(tn, 128);
        c.tiles_of_expert = static_cast<uint32_t>(start[lo + 1] - start[lo]);
        return c;
    };
    auto rows_of_expert = [&](uint32_t seg, uint32_t e) -> uint32_t {
        return static_cast<uint32_t>(tables[seg_meta[seg] + p.seg[seg].experts + 1 + e]);
    };

    // ---- tile feed.  The first tile of CTA (pair) c is tile c; the rest of the work
    // list is claimed tile by tile from a counter all of them share (tiles cost
    // different times: gate/up tiles have 2-3.5x the K of down tiles, and row counts
    // differ).  The scheduler warp claims one tile ahead of the weight producer --
    // so that the counter's round trip is on nobody's critical path, and nobody
    // hoards tiles -- and publishes the claims in a small ring in shared memory
    // (of both CTAs of a pair) that the roles follow.  Claims ascend, and every
    // gate/up tile comes before every down tile in the list, so when a down tile is
    // claimed all the gate/up tiles it waits for are already claimed by running CTAs.
    // The n-th tile of this CTA, for a whole warp (lane 0 polls): the tile index,
    // total_tiles after the last one, 0xFFFFFFFF if the CTA is aborting.  Sequence
    // number and tile travel in one 8-byte shared-memory word, so no fence is needed.
    auto feed_take = [&](uint32_t n) -> uint32_t {
        uint32_t t = 0xFFFFFFFFu;
        if (lane == 0) {
            volatile unsigned long long* const slot = feed_ring + n % kFeedSlots;
            unsigned long long word = *slot;
            if (static_cast<uint32_t>(word) != n + 1) {
                const uint64_t t0 = ptx::globaltimer_ns();
                uint32_t spins = 0;
                for (;;) {
                    word = *slot;
                    if (static_cast<uint32_t>(word) == n + 1) break;
                    if ((++spins & 63u) == 0u) {
                        if (*ctl.abort) break;
                        if (ptx::globaltimer_ns() - t0 > ctl.timeout_ns) {
                            report_failure(ctl, kWaitTimeout, 7, static_cast<uint32_t>(word), n + 1);
                            break;
                        }
                    }
                }
            }
            if (static_cast<uint32_t>(word) == n + 1) t = static_cast<uint32_t>(word >> 32);
        }
        return __shfl_sync(0xffffffffu, t, 0);
    };

    // Barriers the roles use.  In a pair the stage-full and accumulator-free barriers
    // are the leader's (its MMA thread waits on them); stage-free and accumulator-full
    // are local to each CTA and the leader's MMA thread commits to both.
    const uint32_t lead_full = kPair ? ptx::mapa(bar_full, 0) : bar_full;
    const uint32_t lead_acc_empty = kPair ? ptx::mapa(bar_acc_empty, 0) : bar_acc_empty;
    const uint32_t peer_empty = kPair ? ptx::mapa(bar_empty, 1) : 0u;
    const uint32_t peer_acc_full = kPair ? ptx::mapa(bar_acc_full, 1) : 0u;

    if (warp == 0 || warp == 2) {
        // ------------------------------------------------------------ producers
        const bool weights = warp == 0;
        StageCursor cur;
        uint32_t armed = 0, armed_parity = 0, ntiles = 0, ready_block = 0xFFFFFFFFu;
        bool ok = true;
        for (; ok; ++ntiles) {
            if (weights && lane == 0) *feed_pos = ntiles + 1;     // lets the scheduler claim the tile after this one
            const uint32_t tile = feed_take(ntiles);
            if (tile == 0xFFFFFFFFu) ok = false;
            if (tile >= total_tiles) break;
            const TileCoord tc = locate(tile);
            const GemmSegment& sg = p.seg[tc.seg];
            const uint32_t nt = tc.n_tile, e = tc.expert;
            // w_sf_kblocks is 1 or 4: use mask and shift in the per-stage loop
            const uint32_t kmask = sg.w_sf_kblocks - 1, kshift = sg.w_sf_kblocks == 4 ? 2u : 0u;
            const uint32_t k_blocks = sg.k_blocks, w_sf_stride = sg.w_sf_stride;
            const uint32_t w_tx = kPair ? sg.weight_tx_bytes / 2 : sg.weight_tx_bytes;
            const uint32_t act_sf_stride = sg.act_sf_stride;
            const bool fp4 = sg.weight_format == 5u;
            const uint32_t sf_planes = (k_blocks + kmask) >> kshift;
            const uint32_t w_row0 = nt * kTileRows + (kPair ? cta * kHalfRows : 0u);   // first weight row this CTA loads
            const uint32_t* wsf = sg.w_sf + static_cast<size_t>(e) * sf_planes * sg.w_sf_stride + w_row0;
            const uint32_t n_cols = round_up_u32(tc.valid, 16);
            const uint32_t sf_chunk = round_up_u32(n_cols, 128);          // scale rows of the tile: 128 or 256
            const uint32_t* asf = sg.act_sf + tc.sf_row;
            // The token rows this CTA stages: all of the tile, or its half of them; the
            // smallest box that holds them (rows beyond are fetched and ignored).
            const uint32_t need = kPair ? n_cols / 2 : tc.valid;
            uint32_t mi = 0;
            while (mi + 1 < sg.num_act_maps && sg.act_box_rows[mi] < need) ++mi;
            const uint32_t act_rows = sg.act_box_rows[mi];
            const CUtensorMap* const act_map = &sg.tm_act[mi];
            const uint32_t act_row0 = tc.row0 + (kPair ? cta * (n_cols / 2) : 0u);
            // An expert with several row tiles streams its weights once per tile: keep them in L2.
            const uint64_t w_hint = tc.tiles_of_expert >= 2u ? ptx::kEvictNormal : ptx::kEvictFirst;
            if (!weights && sg.kind == kSegUp && !sg.shared && tc.block != ready_block) {
                // The rows of this tile are pushed by the dispatch kernels (of this and the
                // other GPUs), which count them per row tile: wait until all of them have
                // landed, then order the TMA (async proxy) after the acquire.
                uint32_t landed = 1;
                if (lane == 0)
                    landed = flag_wait_eq(p.tile_arrived + generation * exchange::kMaxRowTiles + tc.block, tc.valid, ctl, 5);
                if (!__shfl_sync(0xffffffffu, landed, 0)) { ok = false; break; }
                ptx::fence_proxy_async_global();
                ready_block = tc.block;
            }
            if (!weights && sg.kind == kSegDown && sg.done_target != 0) {
                // The tile's intermediate rows are written by the up tiles of this same
                // launch, possibly on other SMs: wait for all of them.
                uint32_t done = 1;
                if (lane == 0) done = flag_wait_ge_gpu(sg.block_done + tc.block, sg.done_target, ctl, 7);
                if (!__shfl_sync(0xffffffffu, done, 0)) { ok = false; break; }
                ptx::fence_proxy_async_global();
            }
            for (uint32_t kb = 0; kb < k_blocks; kb += kPair ? kPairStageBlocks : 1u) {
                const bool got = mbar_wait(bar_empty + 8 * cur.stage, cur.phase ^ 1u, ctl, 1);
                if (!got) { ok = false; break; }
                const uint32_t full = lead_full + 8 * cur.stage;
                armed |= 1u << cur.stage;
                armed_parity = (armed_parity & ~(1u << cur.stage)) | (cur.phase << cur.stage);
                if (ptx::elect_one()) {
                    if (weights) {
                        // K128-granular scales: one packed word serves four K128 blocks
                        const bool load_sf = (kb & kmask) == 0;
                        const uint32_t dst = base + L.w + cur.stage * L.w_stage;
                        const uint32_t sf_dst = base + L.sfw + cur.stage * L.sfw_stage;
                        if constexpr (kPair) {
                            // two K128 blocks of this CTA's 128 rows per request (a block beyond K reads zeros)
                            ptx::mbar_arrive_expect_tx_cluster(full, 2 * w_tx + (load_sf ? L.sfw_stage : 0));
                            if (fp4) ptx::tma_pair_load_4d(dst, &sg.tm_w, full, 0, w_row0, kb, e, w_hint);
                            else ptx::tma_pair_load_3d(dst, &sg.tm_w, full, 0, w_row0, kb, w_hint);
                            if (load_sf)
                                ptx::tma_pair_load_2d(sf_dst, &sg.tm_w_sf, full, w_row0, e * sf_planes + (kb >> kshift), w_hint);
                        } else {
                            ptx::mbar_arrive_expect_tx(full, w_tx + (load_sf ? L.sfw_stage : 0));
                            if (fp4) ptx::tma_load_4d(dst, &sg.tm_w, full, 0, w_row0, kb, e, w_hint);
                            else ptx::tma_load_3d(dst, &sg.tm_w, full, 0, w_row0, kb, w_hint);
                            if (load_sf)
                                ptx::bulk_load_1d(sf_dst, wsf + static_cast<size_t>(kb >> kshift) * w_sf_stride,
                                                  L.sfw_stage, full, w_hint);
                        }
                    } else {
                        const uint32_t dst = base + L.a + cur.stage * L.a_stage;
                        const uint32_t sf_dst = base + L.sfa + cur.stage * L.sfa_stage;
                        if constexpr (kPair) {
                            // token rows [2 K blocks][rows][128 B]; scale words [128-row chunk][2 K blocks][128]
                            ptx::mbar_arrive_expect_tx_cluster(full, 2 * (act_rows * kTileK + sf_chunk * 4));
                            ptx::tma_pair_load_3d(dst, act_map, full, 0, act_row0, kb, ptx::kEvictLast);
                            ptx::tma_pair_load_2d(sf_dst, &sg.tm_act_sf, full, tc.sf_row, kb, ptx::kEvictLast);
                            if (sf_chunk > 128)
                                ptx::tma_pair_load_2d(sf_dst + 2 * kSfChunkBytes, &sg.tm_act_sf, full, tc.sf_row + 128, kb,
                                                      ptx::kEvictLast);
                        } else {
                            ptx::mbar_arrive_expect_tx(full, act_rows * kTileK + sf_chunk * 4);
                            ptx::tma_load_2d(dst, act_map, full, kb * kTileK, act_row0, ptx::kEvictLast);
                            ptx::bulk_load_1d(sf_dst, asf + static_cast<size_t>(kb) * act_sf_stride, sf_chunk * 4, full,
                                              ptx::kEvictLast);
                        }
                    }
                }
                __syncwarp();
                cur.advance(1, p.stages);
            }
        }
        if (!ok && lane == 0 && !kPair) {
            // Another role gave up.  Let the copies already in flight land (they
            // depend on nothing) before the CTA releases its shared memory.  (A pair
            // cannot watch the leader's barrier from the follower; both CTAs instead
            // meet at the cluster barrier below after the leader has drained.)
            const uint64_t t0 = ptx::globaltimer_ns();
            for (uint32_t s = 0; s < p.stages; ++s) {
                if (!(armed >> s & 1u)) continue;
                while (!ptx::mbar_try_wait(bar_full + 8 * s, (armed_parity >> s) & 1u) &&
                       ptx::globaltimer_ns() - t0 < 2000000ull) {}
            }
        }
        if (!ok && lane == 0 && kPair) {
            // copies in flight complete within microseconds; give them that time
            const uint64_t t0 = ptx::globaltimer_ns();
            while (ptx::globaltimer_ns() - t0 < 20000ull) __nanosleep(1000);
        }
    } else if ((warp == 1 || warp == 3) && (!kPair || (warp == 1 && cta == 0))) {
        // ------------------------------------------------------------ MMA issue
        const uint32_t m = kPair ? 0u : warp >> 1;            // single CTA: which 128-row half of the tile
        const uint32_t halves = kPair ? 1u : 2u;
        {
            const uint32_t sf_cols = 4 + p.sf_block_m / 32;
            const uint32_t sfw_tmem = tmem_base + p.acc_stages * halves * bm + m * sf_cols;   // 4 columns
            const uint32_t sfa_tmem = sfw_tmem + 4;                            // sf_block_m / 32 columns
            const uint64_t wdesc0 = ptx::smem_desc(base + L.w + m * kHalfStageBytes, 1024, true);
            const uint64_t adesc0 = ptx::smem_desc(base + L.a, 1024, true);
            const uint64_t sfw_desc0 = ptx::smem_desc(base + L.sfw + m * kSfChunkBytes, 128, false);
            const uint64_t sfa_desc0 = ptx::smem_desc(base + L.sfa, 128, false);
            StageCursor cur;
            uint32_t it = 0;
            bool ok = true;
            for (; ok; ++it) {
                const uint32_t tile = feed_take(it);
                if (tile == 0xFFFFFFFFu) ok = false;
                if (tile >= total_tiles) break;
                const TileCoord tc = locate(tile);
                const GemmSegment& sg = p.seg[tc.seg];
                const uint32_t n = round_up_u32(tc.valid, 16);
                const uint32_t idesc = ptx::instr_desc(n, sg.weight_format, kPair);
                const uint32_t kmask = sg.w_sf_kblocks - 1, k_blocks = sg.k_blocks;   // w_sf_kblocks is 1 or 4
                const bool wide_sf = n > 128;
                const uint32_t as = p.acc_stages == 2 ? (it & 1u) : 0u;
                const uint32_t acc_phase = p.acc_stages == 2 ? ((it >> 1) & 1u) : (it & 1u);
                const bool acc_free = mbar_wait(bar_acc_empty + 8 * as, acc_phase ^ 1u, ctl, 2);
                if (!acc_free) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (as * halves + m) * bm;
                // rows of token operand staged per K block (pair: this CTA's box, see the producer)
                uint32_t a_block_bytes = 0;
                if constexpr (kPair) {
                    uint32_t mi = 0;
                    while (mi + 1 < sg.num_act_maps && sg.act_box_rows[mi] < n / 2) ++mi;
                    a_block_bytes = sg.act_box_rows[mi] * kTileK;
                }
                for (uint32_t kb = 0; kb < k_blocks; kb += kPair ? kPairStageBlocks : 1u) {
                    const bool got = mbar_wait(bar_full + 8 * cur.stage, cur.phase, ctl, 3);
                    if (!got) { ok = false; break; }
                    ptx::tc_fence_after();
                    if (ptx::elect_one()) {
                        // Descriptors of this stage: the per-warp base plus the stage's offset in
                        // 16-byte units (all shared-memory addresses fit the 14-bit field).
                        const uint64_t sfw_desc = sfw_desc0 + cur.stage * (L.sfw_stage >> 4);
                        const uint64_t sfa_desc = sfa_desc0 + cur.stage * (L.sfa_stage >> 4);
                        const uint64_t wdesc = wdesc0 + cur.stage * (L.w_stage >> 4);
                        const uint64_t adesc = adesc0 + cur.stage * (L.a_stage >> 4);
                        const uint32_t step = kmask ? (1u << 4) : ((1u << 29) | (1u << 4));
                        if constexpr (kPair) {
#pragma unroll
                            for (uint32_t j = 0; j < kPairStageBlocks; ++j) {
                                const uint32_t k = kb + j;
                                if (k < k_blocks) {
                                    // weight scales of K128 granularity: one word per four K blocks
                                    if ((k & kmask) == 0) ptx::tmem_cp_sf<kPair>(sfw_tmem, sfw_desc + (kmask ? 0u : j * (kSfChunkBytes >> 4)));
                                    ptx::tmem_cp_sf<kPair>(sfa_tmem, sfa_desc + j * (kSfChunkBytes >> 4));
                                    if (wide_sf) ptx::tmem_cp_sf<kPair>(sfa_tmem + 4, sfa_desc + (2 + j) * (kSfChunkBytes >> 4));
                                    const uint32_t first = kmask ? (idesc | ((k & 3u) << 29)) : idesc;
                                    ptx::mma_mxf8f6f4_k128<kPair>(d_tmem, wdesc + j * (kHalfStageBytes >> 4),
                                                                  adesc + j * (a_block_bytes >> 4), first, step, sfw_tmem,
                                                                  sfa_tmem, k != 0u ? 1u : 0u);
                                }
                            }
                        } else {
                            // Weight scales of K128 granularity arrive with every fourth stage and
                            // stay in TMEM for the three stages that follow.
                            if ((kb & kmask) == 0) ptx::tmem_cp_sf<kPair>(sfw_tmem, sfw_desc);
                            ptx::tmem_cp_sf<kPair>(sfa_tmem, sfa_desc);
                            if (wide_sf) ptx::tmem_cp_sf<kPair>(sfa_tmem + 4, sfa_desc + (kSfChunkBytes >> 4));
                            // Scale byte of MMA k: k-th byte of the stage's packed words (K32 scales);
                            // for K128 weight scales the weight byte is kb % 4 for all four.
                            const uint32_t first = kmask ? (idesc | ((kb & 3u) << 29)) : idesc;
                            ptx::mma_mxf8f6f4_k128<kPair>(d_tmem, wdesc, adesc, first, step, sfw_tmem, sfa_tmem,
                                                          kb != 0u ? 1u : 0u);
                        }
                        ptx::tc_commit<kPair>(bar_empty + 8 * cur.stage);
                        if constexpr (kPair) ptx::tc_commit<kPair>(peer_empty + 8 * cur.stage);
                        if (kb + (kPair ? kPairStageBlocks : 1u) >= k_blocks) {
                            ptx::tc_commit<kPair>(bar_acc_full + 8 * as);
                            if constexpr (kPair) ptx::tc_commit<kPair>(peer_acc_full + 8 * as);
                        }
                    }
                    __syncwarp();
                    cur.advance(1, p.stages);
                }
            }
            if (!ok && lane == 0) {
                // Do not free TMEM (or let the other CTA of a pair go) under MMAs that may
                // still be running.
                ptx::tc_commit<kPair>(bar_drain + 8 * m);
                const uint64_t t0 = ptx::globaltimer_ns();
                while (!ptx::mbar_try_wait(bar_drain + 8 * m, 0) && ptx::globaltimer_ns() - t0 < 2000000ull) {}
            }
        }
    } else if (warp == 8) {
        // ------------------------------------------------------------ tile scheduler
        if (lane == 0 && cta == 0) {
            const uint32_t peer_ring = kPair ? ptx::mapa(ptx::smem_u32(const_cast<unsigned long long*>(feed_ring)), 1) : 0u;
            for (uint32_t n = 0;; ++n) {
                // stay one tile ahead of the weight producer, not more
                bool go = true;
                if (n > *feed_pos) {
                    const uint64_t t0 = ptx::globaltimer_ns();
                    while (n > *feed_pos) {
                        __nanosleep(200);
                        if (*ctl.abort) { go = false; break; }
                        if (ptx::globaltimer_ns() - t0 > ctl.timeout_ns) {
                            report_failure(ctl, kWaitTimeout, 8, *feed_pos, n);
                            go = false;
                            break;
                        }
                    }
                }
                if (!go) break;
                uint32_t tile;
                if (n == 0 && unit < total_tiles) {
                    tile = unit;
                } else {
                    // Every CTA (pair) ends with exactly one claim beyond the list, so the
                    // launch makes max(total - units, 0) + units claims; whoever draws the
                    // last one knows all others are done claiming and puts the cursor back to
                    // zero for the next launch.
                    const uint32_t v = atomicAdd(p.tile_cursor, 1u);
                    tile = min(units + v, total_tiles);
                    const uint32_t inside = total_tiles > units ? total_tiles - units : 0u;
                    if (v == inside + units - 1u) *p.tile_cursor = 0;
                }
                const unsigned long long word = (static_cast<unsigned long long>(tile) << 32) | (n + 1);
                feed_ring[n % kFeedSlots] = word;
                if constexpr (kPair) ptx::st_cluster_u64(peer_ring + (n % kFeedSlots) * 8, word);
                if (tile >= total_tiles) break;
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------------------------------------ epilogue
        const uint32_t q = warp & 3u;           // the TMEM lane quarter this warp can read
        const uint32_t r = q * 32 + lane;       // weight row inside the 128-row half
        const uint32_t lane_base = (q * 32) << 16;
        const uint32_t etid = threadIdx.x - 128;
        const uint32_t halves = kPair ? 1u : 2u;
        uint32_t it = 0;
        uint32_t xbuf = 0;
        bool ok = true;
        const float clamp_bf16 = __bfloat162float(__float2bfloat16_rn(p.clamp));
        uint32_t rows_ready = 0xFFFFFFFFu;   // routed row tile whose pushed rows, weights and metadata are known to have landed
        for (uint32_t i = etid; i < kMaxRanks; i += 128) arrive[i] = 0;
        epilogue_barrier();
        for (; ok; ++it) {
            // The four warps read the same ring entry; they vote so that all of them
            // leave together if one saw the CTA aborting (the named barriers below
            // count 128 threads).
            const uint32_t tile = feed_take(it);
            if (!all_epilogue_threads(tile != 0xFFFFFFFFu)) { ok = false; break; }
            if (tile >= total_tiles) break;
            const TileCoord tc = locate(tile);
            const GemmSegment& sg = p.seg[tc.seg];
            const uint32_t b = tc.block, nt = tc.n_tile, valid = tc.valid;
            const uint32_t ncols = round_up_u32(valid, 16);
            const uint32_t as = p.acc_stages == 2 ? (it & 1u) : 0u;
            const uint32_t acc_phase = p.acc_stages == 2 ? ((it >> 1) & 1u) : (it & 1u);
            const uint32_t row0 = tc.row0;      // activation row of accumulator column 0
            // Stage what the stores need to know about the tile's rows while the
            // main loop is still running: route weight (gate/up) or destination.
            uint32_t* const info = row_info + (it & 1u) * bm * 4;
            if (!kRaw && !sg.shared && b != rows_ready) {
                // Route weights and source metadata are pushed together with the rows by
                // the dispatch kernels; wait until the tile's rows have all landed (a down
                // tile can be reached before its gate/up tiles were waited for by this CTA).
                bool landed = true;
                if (etid == 0)
                    landed = flag_wait_eq(p.tile_arrived + generation * exchange::kMaxRowTiles + b, valid, ctl, 6);
                if (!all_epilogue_threads(landed)) { ok = false; break; }
                rows_ready = b;
            }
            if (kRaw) {
            } else if (sg.kind == kSegUp) {
                // the shared expert's rows carry no route weight
                for (uint32_t i = etid; i < valid; i += 128)
                    info[i] = sg.shared ? __float_as_uint(1.0f) : __float_as_uint(sg.route_weight[row0 + i]);
            } else {
                if (sg.shared) {
                    // own tokens: row t goes to this rank's combine slot `topk`
                    for (uint32_t i = etid; i < valid; i += 128) {
                        info[i * 3] = p.rank;
                        info[i * 3 + 1] = row0 + i;
                        info[i * 3 + 2] = p.topk;
                    }
                } else {
                    for (uint32_t i = etid; i < valid * 3; i += 128)
                        info[i] = sg.metadata[static_cast<size_t>(row0) * 3 + i];
                }
            }
            // Every epilogue thread must take the same exit, or the named barriers
            // below would wait for threads that have left: vote on the outcome.
            const bool acc_ready = all_epilogue_threads(mbar_wait(bar_acc_full + 8 * as, acc_phase, ctl, 4));
            if (!acc_ready) {
                ok = false;
                break;
            }
            ptx::tc_fence_after();
            if (!kRaw && sg.kind == kSegDown && p.num_ranks > 1 && !sg.shared) {
                // Rows x 128-channel halves this tile writes to each source rank; reported
                // once, after the CTA's last tile (the vote above made `info` visible to
                // all threads).
                for (uint32_t i = etid; i < valid; i += 128) atomicAdd(arrive + info[i * 3], halves);
            }
            for (uint32_t hh = 0; hh < halves; ++hh)
            for (uint32_t c0 = 0; c0 < ncols; c0 += 16) {
                const uint32_t half = kPair ? cta : hh;   // which 128 rows of the weight tile
                const uint32_t nh = nt * 2 + half;      // index of the 128-row half among the expert's rows
                uint32_t vi[16];
                ptx::tmem_ld16(tmem_base + lane_base + (as * halves + hh) * bm + c0, vi);
                ptx::tmem_ld_wait();
                if (hh + 1 == halves && c0 + 16 >= ncols) {
                    // Last read of this accumulator stage: hand it back to the MMA warps.
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (kPair) ptx::mbar_arrive_cluster(lead_acc_empty + 8 * as);
                        else ptx::mbar_arrive(bar_acc_empty + 8 * as);
                    }
                }
                if constexpr (kRaw) {
#pragma unroll
                    for (uint32_t c = 0; c < 16; ++c) {
                        const uint32_t col = c0 + c;
                        if (col < valid)
                            p.raw_out[static_cast<size_t>(row0 + col) * sg.w_rows + nh * kHalfRows + r] =
                                __uint_as_float(vi[c]);
                    }
                } else if (sg.kind == kSegDown) {
                    // Transpose through shared memory so that a token's 128 channels leave
                    // as 16-byte vectors: 256 contiguous bytes per half-warp, which is what
                    // NVLink (and HBM) want, instead of 2-byte elements per lane.
                    __nv_bfloat16* const tile = out_stage + xbuf * 16 * kHalfRows;
#pragma unroll
                    for (uint32_t c = 0; c < 16; ++c)
                        tile[c * kHalfRows + r] = __float2bfloat16_rn(__uint_as_float(vi[c]));
                    epilogue_barrier();
#pragma unroll
                    for (uint32_t v = 0; v < 2; ++v) {
                        const uint32_t c = (etid >> 4) + v * 8, seg = etid & 15u;
                        const uint32_t col = c0 + c;
                        if (col < valid) {
                            const uint32_t src_rank = info[col * 3], src_token = info[col * 3 + 1], slot = info[col * 3 + 2];
                            uint4* dst = reinterpret_cast<uint4*>(
                                reinterpret_cast<__nv_bfloat16*>(p.combine_base[src_rank]) +
                                (static_cast<size_t>(slot) * p.capacity + src_token) * p.hidden + nh * kHalfRows) + seg;
                            *dst = *reinterpret_cast<const uint4*>(tile + c * kHalfRows + seg * 8);
                        }
                    }
                    xbuf ^= 1u;
                } else {
                    // Rows come in groups of 16: 8 gate rows then the 8 up rows of the
                    // same channels, so lane l and lane l^8 hold a channel's pair.  The
                    // gate lane finishes the even columns, the up lane the odd ones.
                    const uint32_t is_up = (r >> 3) & 1u;
                    float res[8], amax[8];
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        const float even = __uint_as_float(vi[2 * j]), odd = __uint_as_float(vi[2 * j + 1]);
                        const float recv = __shfl_xor_sync(0xffffffffu, is_up ? even : odd, 8);
                        const float g = is_up ? recv : even;
                        const float u = is_up ? odd : recv;
                        const uint32_t col = c0 + 2 * j + is_up;
                        const float w = col < valid ? __uint_as_float(info[col]) : 0.0f;
                        res[j] = swiglu_weighted(g, u, w, clamp_bf16, p.has_clamp != 0, p.fast_math != 0);
                        float a = fabsf(res[j]);
                        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 1));
                        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 2));
                        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 4));
                        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, 16));
                        amax[j] = a;     // max over this warp's 16 channels of column `col`
                    }
                    // A scale covers 32 channels = this warp and its neighbour (q ^ 1).
                    float* const mine = amax_x + (xbuf * 4 + q) * 16;
                    const float* const other = amax_x + (xbuf * 4 + (q ^ 1u)) * 16;
                    if ((lane & 0x17u) == 0u) {
#pragma unroll
                        for (uint32_t j = 0; j < 8; ++j) mine[2 * j + is_up] = amax[j];
                    }
                    epilogue_barrier();
                    // Quantise into a [16 tokens][64 channels] byte tile in shared memory, then
                    // store it as 16-byte vectors (64 contiguous bytes per token) and let one
                    // thread per (token, 32-channel group) write the scale byte.
                    uint8_t* const otile = reinterpret_cast<uint8_t*>(out_stage) + xbuf * 4096;
                    const uint32_t c64 = (r >> 4) * 8 + (r & 7u);        // channel inside this half's 64
#pragma unroll
                    for (uint32_t j = 0; j < 8; ++j) {
                        const uint32_t col16 = 2 * j + is_up;
                        const float mx = fmaxf(amax[j], other[col16]);
                        const uint32_t code = ue8m0_scale_byte(mx);
                        const float inv = __uint_as_float((254u - code) << 23);
                        otile[col16 * 64 + c64] = static_cast<uint8_t>(ptx::cvt_e4m3x2(__fmul_rn(res[j], inv), 0.0f) & 0xFFu);
                        if ((q & 1u) == 0u && (lane & 0x17u) == 0u) otile[1024 + col16 * 2 + (q >> 1)] = static_cast<uint8_t>(code);
                    }
                    epilogue_barrier();
                    if (etid < 64) {
                        const uint32_t col16 = etid >> 2, seg16 = etid & 3u, col = c0 + col16;
                        if (col < valid)
                            *reinterpret_cast<uint4*>(sg.out_acts + static_cast<size_t>(row0 + col) * sg.inter + nh * 64 + seg16 * 16) =
                                *reinterpret_cast<const uint4*>(otile + col16 * 64 + seg16 * 16);
                    } else if (etid < 96) {
                        const uint32_t col16 = (etid - 64) >> 1, grp = etid & 1u, col = c0 + col16;
                        if (col < valid) {
                            const uint8_t code = otile[1024 + col16 * 2 + grp];
                            const uint32_t k32 = nh * 2 + grp;           // index of the 32-channel group
                            // reference layout: position of the pool row inside its block-M block
                            const uint32_t row = row0 + col, rb = row / sg.ref_block_m;
                            const size_t plane = static_cast<size_t>(k32 >> 2) * sg.out_sf_stride;
                            const size_t word = plane + static_cast<size_t>(rb) * round_up_u32(sg.ref_block_m, 128) +
                                                sf_row_in_block(row - rb * sg.ref_block_m);
                            sg.out_sf[word * 4 + (k32 & 3u)] = code;
                            if (sg.out_sf_private != 0u) {
                                // tile-ordered copy for the down tiles of this launch
                                const size_t mine = plane + sg.out_sf_private + tc.sf_row + sf_row_in_block(col);
                                sg.out_sf[mine * 4 + (k32 & 3u)] = code;
                            }
                        }
                    }
                    xbuf ^= 1u;
                }
            }
            if (!kRaw && sg.kind == kSegUp) {
                // Publish the tile: make the intermediate rows visible to the TMA reads of
                // the down tiles (other SMs), then count it for its row tile.
                ptx::fence_proxy_async_global();
                epilogue_barrier();
                if (etid == 0) {
                    __threadfence();
                    atomicAdd(sg.block_done + b, 1u);
                }
            }
        }
        if (!kRaw && ok && p.num_ranks > 1) {
            // Tell each source rank how many rows x halves this CTA has written into its
            // combine slots: one release per rank and CTA, after the last tile.  A
            // release per tile would make the epilogue wait for the NVLink round trip of
            // its stores every time (measured: a third of the GEMM time on 4 GPUs).  The
            // barrier orders every epilogue thread's stores before the releases.
            epilogue_barrier();
            if (etid < p.num_ranks) {
                const uint32_t n = arrive[etid];
                if (n != 0u)
                    ptx::red_release_sys_add(reinterpret_cast<uint32_t*>(p.combine_arrived[etid] + generation * 128), n);
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    // Neither CTA of a pair leaves (or frees TMEM) while the other may still address
    // its shared memory or run MMAs that read it.
    if constexpr (kPair) ptx::cluster_sync();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after();
        ptx::tmem_dealloc<kPair>(tmem_base, p.tmem_cols);
    }
    // The launch never waited for the dispatch kernel as a whole; do it before the
    // grid retires, so that whatever is ordered after this launch is ordered after
    // the dispatch kernel too.
    if (threadIdx.x == 0) ptx::grid_dependency_wait();
}

}  // namespace gcmoe
