// Host side of libgcmoe_sm100.so: argument checks, TMA descriptor encoding,
// launch configuration and the extern "C" entry points of include/gcmoe.h.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "../../include/gcmoe.h"
#include "combine.cuh"
#include "stage_inputs.cuh"
#include "transform_weights.cuh"
#include "dispatch.cuh"
#include "grouped_gemm.cuh"

namespace gcmoe {

thread_local char g_error[512] = "";

static int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

#define GCMOE_CUDA(expr)                                                              \
    do {                                                                              \
        cudaError_t err__ = (expr);                                                   \
        if (err__ != cudaSuccess)                                                     \
            return fail(GCMOE_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__)); \
    } while (0)

// cuTensorMapEncodeTiled is a driver entry point; resolve it through the
// runtime so the library does not link against libcuda directly.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int get_encoder(EncodeTiledFn* fn) {
    static EncodeTiledFn cached = nullptr;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (cached == nullptr) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        GCMOE_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q));
        if (q != cudaDriverEntryPointSuccess || sym == nullptr)
            return fail(GCMOE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        cached = reinterpret_cast<EncodeTiledFn>(sym);
    }
    *fn = cached;
    return GCMOE_OK;
}

static int encode_map(CUtensorMap* map, CUtensorMapDataType type, uint32_t rank, uint64_t address,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      const char* what, bool swizzle128 = true) {
    EncodeTiledFn encode;
    if (int rc = get_encoder(&encode)) return rc;
    cuuint64_t gdims[5], gstrides[4];
    cuuint32_t gbox[5], estr[5];
    for (uint32_t i = 0; i < rank; ++i) { gdims[i] = dims[i]; gbox[i] = box[i]; estr[i] = 1; }
    for (uint32_t i = 0; i + 1 < rank; ++i) gstrides[i] = strides_bytes[i];
    CUresult r = encode(map, type, rank, reinterpret_cast<void*>(address), gdims, gstrides, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(GCMOE_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, int(r));
    return GCMOE_OK;
}

static uint32_t pow2_at_least(uint32_t v) {
    uint32_t r = 32;
    while (r < v) r <<= 1;
    return r;
}

struct Plan {
    gcmoe_problem prob;
    gcmoe_buffers buf;
    int device = 0;
    int num_sms = 0;
    uint32_t* status = nullptr;
    DispatchParams dispatch;
    // Launch set of one GEMM regime: up tiles only, down tiles only, the layer's single GEMM launch.
    struct Regime {
        GemmParams up, down, fused;
        uint32_t grid = 0, smem = 0;      // grid 0: this regime is never launched for this plan
    };
    Regime single, pairs;         // one CTA per tile (cta_group::1); CTA pairs (clusters of two, cta_group::2)
    CombineParams combine;
    uint32_t dispatch_grid = 1, dispatch_smem = 0;
    uint32_t combine_grid = 1;
};

}  // namespace gcmoe

struct gcmoe_plan : gcmoe::Plan {};

using namespace gcmoe;

static int check_problem(const gcmoe_problem& q) {
    if (q.num_ranks <= 0 || q.num_ranks > GCMOE_MAX_RANKS || q.rank < 0 || q.rank >= q.num_ranks)
        return fail(GCMOE_ERR_INVALID, "invalid rank %d of %d", q.rank, q.num_ranks);
    if (q.num_experts <= 0 || q.num_experts > kMaxExperts || q.num_experts % q.num_ranks ||
        q.num_experts / q.num_ranks > kMaxLocalExperts)
        return fail(GCMOE_ERR_INVALID, "invalid rank/expert configuration");
    if (q.topk <= 0 || q.topk + (q.num_shared_experts > 0) > 32)
        return fail(GCMOE_ERR_INVALID, "invalid topk/shared configuration");
    if (q.hidden <= 0 || q.hidden % 256 || q.intermediate <= 0 || q.intermediate % 128 ||
        q.intermediate > 4096)
        return fail(GCMOE_ERR_UNSUPPORTED, "hidden must be a multiple of 256 and intermediate a multiple of 128 up to 4096");
    if (q.capacity <= 0 || q.num_tokens < 0 || q.num_tokens > q.capacity)
        return fail(GCMOE_ERR_INVALID, "token count %d outside capacity %d", q.num_tokens, q.capacity);
    const int bm = q.block_m;
    if (!(bm == 16 || bm == 32 || bm == 64 || bm == 96 || bm == 128 || bm == 192 || bm == 240))
        return fail(GCMOE_ERR_INVALID, "block_m %d is not a block-M candidate", bm);
    if (q.ring_tokens <= 0 || q.ring_tokens % 1920 || q.sf_ring_tokens % 4 ||
        q.sf_ring_tokens < (q.ring_tokens / bm) * int(round_up_u32(bm, 128)))
        return fail(GCMOE_ERR_INVALID, "invalid ring geometry");
    // The kernels address the pool without wrap-around: the ring must hold the
    // largest pool this call can produce.
    const long long local = q.num_experts / q.num_ranks;
    const long long routes = 1ll * q.num_ranks * q.capacity * (q.topk < local ? q.topk : local);
    if (q.ring_tokens < routes + local * (bm - 1))
        return fail(GCMOE_ERR_UNSUPPORTED, "ring of %d rows cannot hold the whole receive pool", q.ring_tokens);
    if (q.dispatch_sms < 0) return fail(GCMOE_ERR_INVALID, "invalid dispatch SM request");
    if (q.num_shared_experts < 0 || (q.num_shared_experts > 0 && q.shared_gran_k != 32 && q.shared_gran_k != 128))
        return fail(GCMOE_ERR_INVALID, "invalid shared expert configuration");
    if (1ll * q.num_shared_experts * q.intermediate > 65536)
        return fail(GCMOE_ERR_UNSUPPORTED, "shared intermediate size too large");
    return GCMOE_OK;
}

extern "C" int gcmoe_version(void) { return 100; }

extern "C" const char* gcmoe_last_error(void) { return g_error; }

extern "C" size_t gcmoe_scratch_bytes(const gcmoe_problem* problem) {
    if (problem == nullptr || problem->num_ranks <= 0) return 0;
    const size_t local = size_t(problem->num_experts / problem->num_ranks);
    // status | count | block prefix | tile prefix | row start | scale start | call info | shared table | tile counters
    const size_t counters = size_t(problem->ring_tokens) / 16 + local + size_t(problem->capacity) / 16 + 4;
    return round_up_u32(uint32_t(kStatusWords * 4 + (5 * local + 2) * 4 + kCallInfoWords * 4 + 8 * 4 + counters * 4), 256);
}

extern "C" int gcmoe_plan_create(const gcmoe_problem* problem, const gcmoe_buffers* buffers,
                                 gcmoe_plan** out) {
    if (problem == nullptr || buffers == nullptr || out == nullptr)
        return fail(GCMOE_ERR_INVALID, "null argument");
    *out = nullptr;
    if (int rc = check_problem(*problem)) return rc;
    const gcmoe_problem& q = *problem;
    const gcmoe_buffers& b = *buffers;
    if (b.arena_base[q.rank] == 0 || b.arena_base[q.rank] % 16)
        return fail(GCMOE_ERR_INVALID, "arena base must be a 16-byte aligned device address");
    if (b.y % 16) return fail(GCMOE_ERR_INVALID, "y must be 16-byte aligned");
    if (q.num_tokens > 0 && b.y == 0) return fail(GCMOE_ERR_INVALID, "y is null");
    if (b.w1 == 0 || b.w2 == 0 || b.w1_sf == 0 || b.w2_sf == 0 || b.w1 % 32 || b.w2 % 32 ||
        b.w1_sf % 16 || b.w2_sf % 16)
        return fail(GCMOE_ERR_INVALID, "weights must be 32-byte and scales 16-byte aligned device addresses");
    if (b.w1_sf_stride < uint64_t(2 * q.intermediate) || b.w1_sf_stride % 4 ||
        b.w2_sf_stride < uint64_t(q.hidden) || b.w2_sf_stride % 4)
        return fail(GCMOE_ERR_INVALID, "weight scales must be MN-major with a 4-aligned K stride");
    if (b.scratch == 0 || b.scratch % 16 || b.scratch_bytes < gcmoe_scratch_bytes(problem))
        return fail(GCMOE_ERR_INVALID, "scratch block missing or too small");
    if (q.num_shared_experts > 0) {
        if (b.sw1 == 0 || b.sw2 == 0 || b.sw1_sf == 0 || b.sw2_sf == 0 || b.sw1 % 16 || b.sw2 % 16 ||
            b.sw1_sf % 16 || b.sw2_sf % 16 || b.sw1_sf_stride % 4 || b.sw2_sf_stride % 4 ||
            b.sw1_sf_stride < uint64_t(2) * q.num_shared_experts * q.intermediate ||
            b.sw2_sf_stride < uint64_t(q.hidden) || b.shared_sf_rows == 0)
            return fail(GCMOE_ERR_INVALID, "shared expert weights, scales or scale views missing or misaligned");
    }
    for (int r = 0; r < q.num_ranks; ++r)
        if (b.arena_base[r] == 0 || b.arena_base[r] % 16)
            return fail(GCMOE_ERR_INVALID, "arena of rank %d is not mapped", r);
    if (b.off_exchange == 0 || b.off_exchange % 128)
        return fail(GCMOE_ERR_INVALID, "exchange block missing or misaligned");
    if (uint64_t(q.ring_tokens) / 16 + uint64_t(q.num_experts / q.num_ranks) + 1 > exchange::kMaxRowTiles)
        return fail(GCMOE_ERR_UNSUPPORTED, "ring of %d rows has more row tiles than the arrival counters hold", q.ring_tokens);

    GCMOE_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    GCMOE_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    GCMOE_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    GCMOE_CUDA(cudaFuncSetAttribute(grouped_gemm_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));
    GCMOE_CUDA(cudaFuncSetAttribute(dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit));

    gcmoe_plan* plan = new (std::nothrow) gcmoe_plan();
    if (plan == nullptr) return fail(GCMOE_ERR_INVALID, "out of host memory");
    plan->prob = q;
    plan->buf = b;
    auto bail = [&](int rc) { delete plan; return rc; };

    cudaError_t ce = cudaGetDevice(&plan->device);
    if (ce != cudaSuccess) return bail(fail(GCMOE_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(ce)));
    int sms = 0, cc_major = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, plan->device);
    cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, plan->device);
    if (cc_major != 10)
        return bail(fail(GCMOE_ERR_UNSUPPORTED, "device compute capability %d.x is not sm_100", cc_major));
    plan->num_sms = (q.num_sms > 0 && q.num_sms < sms) ? q.num_sms : sms;

    const uint32_t P = q.num_ranks, E = q.num_experts, EL = E / P, H = q.hidden, I = q.intermediate;
    const uint32_t bm = q.block_m, sfbm = round_up_u32(bm, 128);
    const uint64_t arena = b.arena_base[q.rank];
    const uint64_t timeout_ns = uint64_t(q.timeout_ms > 0 ? q.timeout_ms : 2000) * 1000000ull;

    // ---- scratch: status | expert_count[EL] | block prefix[EL + 1] | tile prefix[EL + 1] | row start[EL] |
    //      scale start[EL] | call info | shared table | tile counters
    plan->status = reinterpret_cast<uint32_t*>(b.scratch);
    int* expert_count = reinterpret_cast<int*>(b.scratch + kStatusWords * 4);
    int* expert_block_start = expert_count + EL;
    int* expert_tile_start = expert_block_start + EL + 1;
    int* expert_row_start = expert_tile_start + EL + 1;
    int* expert_sf_start = expert_row_start + EL;
    uint32_t* call_info = reinterpret_cast<uint32_t*>(expert_sf_start + EL);

    // GEMM tiles need not be pool blocks (expert_tile_rows); the scale words of the tiles are kept a
    // second time, in tile order, in the upper half of every plane of the scale rings, which the
    // reference layout never touches for block-M >= 16.  Every rank must take the same decision: it
    // depends on the buffer geometry only.  Worst case of the copy: every tile of 121+ rows (or every
    // single-tile expert) takes a 256-row chunk.
    const uint32_t half_sf = (uint32_t(q.sf_ring_tokens) / 2) & ~127u;
    const uint32_t private_sf_row =
        (uint64_t(q.ring_tokens) / 120 + EL + 1) * 256 <= uint64_t(half_sf) ? half_sf : 0u;
    const bool tile_ordered = private_sf_row != 0u;

    // ---- dispatch
    DispatchParams& d = plan->dispatch;
    memset(&d, 0, sizeof(d));
    d.x = reinterpret_cast<const uint8_t*>(arena + b.off_x);
    d.x_sf = reinterpret_cast<const uint32_t*>(arena + b.off_x_sf);
    d.topk_idx = reinterpret_cast<const long long*>(arena + b.off_topk_idx);
    d.topk_weights = reinterpret_cast<const float*>(arena + b.off_topk_weights);
    for (uint32_t r = 0; r < P; ++r) d.arena_base[r] = b.arena_base[r];
    d.off_recv_count = b.off_recv_count;
    d.off_recv_count_sum = b.off_recv_count_sum;
    d.off_routed_pool_blocks = b.off_routed_pool_blocks;
    d.off_recv_parity = b.off_recv_parity;
    d.off_index_table = b.off_index_table;
    d.off_metadata = b.off_metadata;
    d.off_l1_acts = b.off_l1_acts;
    d.off_l1_acts_sf = b.off_l1_acts_sf;
    d.off_l1_weights = b.off_l1_topk_weights;
    d.off_exchange = b.off_exchange;
    d.call_info = call_info;
    d.expert_count = expert_count;
    d.expert_block_start = expert_block_start;
    d.expert_tile_start = expert_tile_start;
    d.expert_row_start = expert_row_start;
    d.expert_sf_start = expert_sf_start;
    d.private_sf_row = private_sf_row;
    d.stats = reinterpret_cast<int*>(b.stats);
    d.status = plan->status;
    d.timeout_ns = timeout_ns;
    d.num_ranks = P; d.rank = q.rank; d.num_experts = E; d.local_experts = EL;
    d.num_tokens = q.num_tokens; d.topk = q.topk; d.hidden = H; d.capacity = q.capacity;
    d.block_m = bm; d.sf_ring = q.sf_ring_tokens;
    const uint32_t routes = uint32_t(q.num_tokens) * q.topk;
    const uint32_t warps = kDispatchThreads / 32;
    // One warp pushes one route at a time.  The grid is kept small (32 CTAs unless the caller
    // says otherwise): the expert GEMMs start while this kernel runs and need the other SMs
    // (a GEMM CTA fills an SM's shared memory, so it cannot share an SM with a dispatch CTA),
    // and the pushes are bound by NVLink, not by the number of warps.  With several ranks at
    // least one CTA per peer, so that the counts reach all peers at the same time.
    // (beyond 16 routes per warp the grid grows again: 32768 routes on 32 CTAs took 370 us)
    const uint32_t dcap = q.dispatch_sms > 0 ? uint32_t(q.dispatch_sms) : (routes / 256 > 32u ? routes / 256 : 32u);
    uint32_t dgrid = (routes + warps - 1) / warps;
    if (P > 1 && dgrid < P) dgrid = P;
    if (dgrid > dcap) dgrid = dcap;
    dgrid = dgrid < 1 ? 1 : (dgrid > uint32_t(plan->num_sms) ? plan->num_sms : dgrid);
    plan->dispatch_grid = dgrid;
    plan->dispatch_smem = dispatch_smem_bytes(E, P, (routes + dgrid - 1) / dgrid);
    if (plan->dispatch_smem > uint32_t(kSmemLimit))
        return bail(fail(GCMOE_ERR_UNSUPPORTED, "dispatch slice does not fit shared memory"));

    // ---- the two grouped GEMMs (each: shared-expert segment first, then routed), once per regime
    const uint32_t S = q.num_shared_experts, IS = S * I;
    int* shared_table = reinterpret_cast<int*>(call_info + kCallInfoWords);   // count, start[0], start[1], row start, scale start
    // Per-row-tile counters of finished up tiles (zeroed by the dispatch kernel).
    uint32_t* done_routed = reinterpret_cast<uint32_t*>(shared_table + 8);
    uint32_t* done_shared = done_routed + q.ring_tokens / 16 + EL + 1;
    d.done_routed = done_routed;
    d.done_shared = S ? done_shared : nullptr;
    d.shared_table = S ? shared_table : nullptr;
    // Small calls only ever run the single regime; for the others the dispatch kernel chooses
    // per call and both launches are enqueued.
    const bool dual = dual_regime_call(bm, uint64_t(P) * q.num_tokens * q.topk);
    d.dual = dual ? 1u : 0u;
    auto build_regime = [&](const bool pair, Plan::Regime& out) -> int {
    // largest tile of the launch: accumulator stride, rows of an activation stage
    const uint32_t widest = pair ? kPairTileRows : kSingleTileRows;
    const uint32_t tn = tile_ordered ? (S && bm > widest ? bm : widest) : bm;
    const uint32_t sftn = round_up_u32(tn, 128);
    const uint32_t table_words = 2 * ((4 * EL + 1) + (S ? 5 : 0));   // up and down segments each hold a copy
    const uint32_t stages = gemm_pick_stages(tn, sftn, table_words, pair);
    if (stages < 2) return fail(GCMOE_ERR_UNSUPPORTED, "block_m %u leaves no room for two pipeline stages", bm);
    out.smem = gemm_smem_layout(stages, tn, sftn, table_words, pair).total + 1024;
    // Two accumulator stages (epilogue overlaps the next tile) while they fit TMEM.
    const uint32_t acc_stages = gemm_tmem_columns(tn, sftn, 2, pair) <= 512 ? 2u : 1u;
    if (gemm_tmem_columns(tn, sftn, acc_stages, pair) > 512)
        return fail(GCMOE_ERR_UNSUPPORTED, "TMEM budget exceeded");

    auto fill_common = [&](GemmParams& g) {
        memset(&g, 0, sizeof(g));
        g.status = plan->status;
        g.timeout_ns = timeout_ns;
        g.block_m = tn;
        g.sf_block_m = sftn;
        g.stages = stages;
        g.acc_stages = acc_stages;
        g.table_words = table_words;
        g.tmem_cols = pow2_at_least(gemm_tmem_columns(tn, sftn, acc_stages, pair));
        g.clamp = q.clamp;
        g.has_clamp = q.has_clamp != 0;
        g.fast_math = q.fast_math != 0;
        g.capacity = q.capacity;
        g.hidden = H;
        g.topk = q.topk;
        g.rank = q.rank;
        g.num_ranks = P;
        g.call_info = call_info;
        g.dual_regime = dual ? 1u : 0u;
        g.epoch_word = reinterpret_cast<const uint32_t*>(arena + b.off_recv_parity);
        g.tile_cursor = call_info + (pair ? kCallTileCursorPair : kCallTileCursor);
        g.tile_arrived = reinterpret_cast<const uint32_t*>(arena + b.off_exchange + exchange::kTileArrived);
        g.failed = reinterpret_cast<uint32_t*>(arena + b.off_exchange + exchange::kFailed);
        for (uint32_t r = 0; r < P; ++r) {
            g.combine_arrived[r] = b.arena_base[r] + b.off_exchange + exchange::kCombineArrived;
            g.combine_base[r] = b.arena_base[r] + b.off_combine_tokens;
        }
    };
    // Activation boxes of a few heights: a tile fetches the smallest one that holds its rows
    // (a CTA of a pair stages half of the tile's rows).
    auto activation_maps = [&](GemmSegment& sg, uint64_t acts, uint32_t k, uint64_t rows, uint32_t max_rows,
                               const char* what) -> int {
        const uint32_t top = pair ? max_rows / 2 : max_rows;
        const uint32_t heights[kMaxActMaps] = {8, 16, 32, 48, 64, 96, 112, 120};
        sg.num_act_maps = 0;
        for (int i = 0; i < kMaxActMaps; ++i) {
            uint32_t h = heights[i];
            if (!pair && h < 16) continue;
            if (h >= top || i == kMaxActMaps - 1) h = top;
            int rc;
            if (pair) {
                // [K/128][rows][128 B] view of the row-major tensor: one request stages two K blocks
                const uint64_t adims[3] = {128, rows, k / 128};
                const uint64_t astr[2] = {k, 128};
                const uint32_t abox[3] = {128, h, kPairStageBlocks};
                rc = encode_map(&sg.tm_act[sg.num_act_maps], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, acts, adims, astr, abox, what);
            } else {
                const uint64_t adims[2] = {k, rows};
                const uint64_t astr[1] = {k};
                const uint32_t abox[2] = {128, h};
                rc = encode_map(&sg.tm_act[sg.num_act_maps], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, acts, adims, astr, abox, what);
            }
            if (rc) return rc;
            sg.act_box_rows[sg.num_act_maps++] = h;
            if (h == top) break;
        }
        return GCMOE_OK;
    };
    // Scale words through tensor maps (CTA pairs only: their loads report to the leader's barrier).
    auto scale_maps = [&](GemmSegment& sg, uint64_t acts_sf, uint64_t act_sf_rows, uint64_t act_sf_stride,
                          uint32_t k_blocks, uint64_t w_sf, uint64_t w_sf_stride, uint64_t w_sf_planes,
                          const char* what) -> int {
        if (!pair) return GCMOE_OK;
        const uint32_t box[2] = {128, kPairStageBlocks};
        const uint64_t adims[2] = {act_sf_rows, k_blocks}, astr[1] = {act_sf_stride * 4};
        if (int rc = encode_map(&sg.tm_act_sf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, acts_sf, adims, astr, box, what, false))
            return rc;
        const uint64_t wdims[2] = {w_sf_stride, w_sf_planes}, wstr[1] = {w_sf_stride * 4};
        return encode_map(&sg.tm_w_sf, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, w_sf, wdims, wstr, box, what, false);
    };
    // Routed experts: FP4 weights [EL][K/128][rows][64 B], pool rows as activations.
    auto routed_segment = [&](GemmSegment& sg, uint64_t acts, uint64_t acts_sf, uint32_t k, uint64_t weights,
                              uint64_t w_sf, uint64_t w_sf_stride, uint32_t w_rows, const char* what) -> int {
        sg.tile_start = expert_tile_start;
        sg.count = expert_count;
        sg.row_start = expert_row_start;
        sg.sf_start = expert_sf_start;
        sg.experts = EL;
        sg.tile_rows = tile_ordered ? 0u : bm;      // 0: per expert, from its row count
        sg.ref_block_m = bm;
        sg.out_sf_private = private_sf_row;
        sg.w_rows = w_rows;
        sg.k_blocks = k / 128;
        sg.n_tiles = w_rows / kTileRows;
        sg.weight_format = 5;
        sg.weight_tx_bytes = kTileRows * 128 / 2;
        sg.w_sf_kblocks = 1;
        // the tile-ordered scale copy when there is one, else the reference layout (tiles = pool blocks)
        sg.act_sf = reinterpret_cast<const uint32_t*>(acts_sf) + private_sf_row;
        sg.act_sf_stride = q.sf_ring_tokens;
        sg.w_sf = reinterpret_cast<const uint32_t*>(w_sf);
        sg.w_sf_stride = uint32_t(w_sf_stride);
        if (int rc = activation_maps(sg, acts, k, uint64_t(q.ring_tokens), tn, what)) return rc;
        if (int rc = scale_maps(sg, acts_sf + uint64_t(private_sf_row) * 4, uint64_t(q.sf_ring_tokens) - private_sf_row,
                                uint64_t(q.sf_ring_tokens), k / 128, w_sf, w_sf_stride, uint64_t(EL) * (k / 128), what))
            return rc;
        // 128-element (64-byte) rows of one K128 tile are adjacent, so a 128 x 256
        // box is one contiguous 16 KiB range in HBM.
        const uint64_t wdims[4] = {128, w_rows, k / 128, EL};
        const uint64_t wstr[3] = {64, uint64_t(w_rows) * 64, uint64_t(w_rows) * 64 * (k / 128)};
        const uint32_t wbox[4] = {128, uint32_t(pair ? kHalfRows : kTileRows), pair ? kPairStageBlocks : 1u, 1};
        return encode_map(&sg.tm_w, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 4, weights, wdims, wstr, wbox, what);
    };
    // Shared expert: FP8 weights [K/128][rows][128 B], this rank's own tokens as rows.
    auto shared_segment = [&](GemmSegment& sg, uint64_t acts, uint64_t acts_sf, uint32_t k, uint64_t weights,
                              uint64_t w_sf, uint64_t w_sf_stride, uint32_t w_rows, const char* what) -> int {
        sg.shared = 1;
        sg.count = shared_table;
        sg.tile_start = shared_table + 1;
        sg.row_start = shared_table + 3;
        sg.sf_start = shared_table + 4;
        sg.experts = 1;
        sg.tile_rows = bm;            // the caller stages the scales in block-M order
        sg.ref_block_m = bm;
        sg.w_rows = w_rows;
        sg.k_blocks = k / 128;
        sg.n_tiles = w_rows / kTileRows;
        sg.weight_format = 0;
        sg.weight_tx_bytes = kTileRows * 128;
        sg.w_sf_kblocks = q.shared_gran_k == 128 ? 4 : 1;
        sg.act_sf = reinterpret_cast<const uint32_t*>(acts_sf);
        sg.act_sf_stride = uint32_t(b.shared_sf_rows);
        sg.w_sf = reinterpret_cast<const uint32_t*>(w_sf);
        sg.w_sf_stride = uint32_t(w_sf_stride);
        if (int rc = activation_maps(sg, acts, k, uint64_t(q.capacity), bm, what)) return rc;
        const uint32_t planes = (k / 128 + sg.w_sf_kblocks - 1) / sg.w_sf_kblocks;
        if (int rc = scale_maps(sg, acts_sf, b.shared_sf_rows, b.shared_sf_rows, k / 128, w_sf, w_sf_stride, planes, what))
            return rc;
        const uint64_t wdims[3] = {128, w_rows, k / 128};
        const uint64_t wstr[2] = {128, uint64_t(w_rows) * 128};
        const uint32_t wbox[3] = {128, uint32_t(pair ? kHalfRows : kTileRows), pair ? kPairStageBlocks : 1u};
        return encode_map(&sg.tm_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, weights, wdims, wstr, wbox, what);
    };

    // a CTA of a pair finishes one half of an up tile
    const uint32_t done_per_tile = pair ? 2u : 1u;

    GemmSegment shared_up, shared_down, routed_up, routed_down;
    memset(&shared_up, 0, sizeof(GemmSegment));
    memset(&shared_down, 0, sizeof(GemmSegment));
    memset(&routed_up, 0, sizeof(GemmSegment));
    memset(&routed_down, 0, sizeof(GemmSegment));
    if (S) {
        if (int rc = shared_segment(shared_up, arena + b.off_x, arena + b.off_shared_l1_acts_sf, H, b.sw1, b.sw1_sf,
                                    b.sw1_sf_stride, 2 * IS, "shared gate/up GEMM")) return rc;
        shared_up.kind = kSegUp;
        shared_up.out_acts = reinterpret_cast<uint8_t*>(arena + b.off_shared_l2_acts);
        shared_up.out_sf = reinterpret_cast<uint8_t*>(arena + b.off_shared_l2_acts_sf);
        shared_up.out_sf_stride = uint32_t(b.shared_sf_rows);
        shared_up.inter = IS;
        shared_up.block_done = done_shared;
        if (int rc = shared_segment(shared_down, arena + b.off_shared_l2_acts, arena + b.off_shared_l2_acts_sf, IS,
                                    b.sw2, b.sw2_sf, b.sw2_sf_stride, H, "shared down GEMM")) return rc;
        shared_down.kind = kSegDown;
        shared_down.block_done = done_shared;
        shared_down.done_target = shared_up.n_tiles * done_per_tile;
    }
    if (int rc = routed_segment(routed_up, arena + b.off_l1_acts, arena + b.off_l1_acts_sf, H, b.w1, b.w1_sf,
                                b.w1_sf_stride, 2 * I, "gate/up GEMM")) return rc;
    routed_up.kind = kSegUp;
    routed_up.out_acts = reinterpret_cast<uint8_t*>(arena + b.off_l2_acts);
    routed_up.out_sf = reinterpret_cast<uint8_t*>(arena + b.off_l2_acts_sf);
    routed_up.out_sf_stride = q.sf_ring_tokens;
    routed_up.inter = I;
    routed_up.route_weight = reinterpret_cast<const float*>(arena + b.off_l1_topk_weights);
    routed_up.block_done = done_routed;
    if (int rc = routed_segment(routed_down, arena + b.off_l2_acts, arena + b.off_l2_acts_sf, I, b.w2, b.w2_sf,
                                b.w2_sf_stride, H, "down GEMM")) return rc;
    routed_down.kind = kSegDown;
    routed_down.metadata = reinterpret_cast<const uint32_t*>(arena + b.off_metadata);
    routed_down.block_done = done_routed;
    routed_down.done_target = routed_up.n_tiles * done_per_tile;

    fill_common(out.up);
    fill_common(out.down);
    fill_common(out.fused);
    auto push = [](GemmParams& g, const GemmSegment& sg) { g.seg[g.num_segments++] = sg; };
    if (S) { push(out.up, shared_up); push(out.fused, shared_up); }
    push(out.up, routed_up);
    push(out.fused, routed_up);
    if (S) { push(out.fused, shared_down); shared_down.done_target = 0; push(out.down, shared_down); }
    push(out.fused, routed_down);
    routed_down.done_target = 0;          // launched on its own, the up tiles finished in an earlier kernel
    push(out.down, routed_down);

    // Upper bound of pool blocks this call can produce: one partial block per
    // expert that can be hit, plus the full blocks.
    const uint64_t all_routes = uint64_t(P) * routes;   // collective calls bring the same order of T
    uint64_t max_blocks = (all_routes < EL ? all_routes : EL) + all_routes / bm;
    if (max_blocks < 1) max_blocks = 1;
    const uint64_t shared_blocks = S ? (uint64_t(q.num_tokens) + bm - 1) / bm : 0;
    {
        // With several ranks the pool depends on what the other ranks send.
        uint64_t tiles = P > 1 ? uint64_t(plan->num_sms)
            : max_blocks * routed_up.n_tiles + (S ? shared_blocks * shared_up.n_tiles : 0);
        if (pair) tiles *= 2;        // two CTAs per tile
        uint32_t grid = uint32_t(tiles < uint64_t(plan->num_sms) ? tiles : uint64_t(plan->num_sms));
        if (pair) {
            // Every CTA of the launch must be resident (down tiles wait for up tiles of running
            // CTAs): no more clusters than the device can hold at once.
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(plan->num_sms & ~1);
            cfg.blockDim = dim3(kGemmThreads);
            cfg.dynamicSmemBytes = out.smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            cudaError_t oe = cudaOccupancyMaxActiveClusters(&clusters, grouped_gemm_kernel<false, true>, &cfg);
            if (oe != cudaSuccess || clusters < 1)
                return fail(GCMOE_ERR_CUDA, "cudaOccupancyMaxActiveClusters: %s (%d clusters)",
                            cudaGetErrorString(oe), clusters);
            grid &= ~1u;
            if (grid < 2) grid = 2;
            if (grid > uint32_t(clusters) * 2) grid = uint32_t(clusters) * 2;
        }
        out.grid = grid;
    }
    return GCMOE_OK;
    };   // build_regime
    if (int rc = build_regime(false, plan->single)) return bail(rc);
    if (dual)
        if (int rc = build_regime(true, plan->pairs)) return bail(rc);

    // ---- combine
    CombineParams& c = plan->combine;
    memset(&c, 0, sizeof(c));
    c.slots = reinterpret_cast<const __nv_bfloat16*>(arena + b.off_combine_tokens);
    c.topk_idx = reinterpret_cast<const long long*>(arena + b.off_topk_idx);
    c.y = reinterpret_cast<__nv_bfloat16*>(b.y);
    c.epoch_word = reinterpret_cast<uint32_t*>(arena + b.off_recv_parity);
    c.num_tokens = q.num_tokens; c.topk = q.topk; c.hidden = H; c.capacity = q.capacity;
    c.num_experts = E; c.has_shared = S ? 1 : 0;
    c.num_ranks = P;
    c.call_info = call_info;
    c.combine_arrived = reinterpret_cast<const uint32_t*>(arena + b.off_exchange + exchange::kCombineArrived);
    c.failed = reinterpret_cast<uint32_t*>(arena + b.off_exchange + exchange::kFailed);
    c.status = plan->status;
    c.timeout_ns = timeout_ns;
    c.halves_per_row = H / kHalfRows;
    const uint64_t cvecs = uint64_t(q.num_tokens) * (H / 8);
    uint64_t cgrid = (cvecs + kCombineThreads - 1) / kCombineThreads;
    const uint64_t cmax = uint64_t(plan->num_sms) * 8;
    plan->combine_grid = uint32_t(cgrid < 1 ? 1 : (cgrid > cmax ? cmax : cgrid));

    *out = plan;
    return GCMOE_OK;
}

extern "C" int gcmoe_plan_destroy(gcmoe_plan* plan) {
    delete plan;
    return GCMOE_OK;
}

// Launch with programmatic stream serialization: the kernel may start while
// its predecessor in the stream is still running and orders itself with
// griddepcontrol.wait (or, for the GEMM launch, with the flags the dispatch
// kernel raises), so it overlaps the predecessor.  `cluster` > 1 launches
// thread-block clusters of that many CTAs.
template <typename Params>
static cudaError_t launch_dependent(void (*kernel)(Params), uint32_t grid, uint32_t block, uint32_t smem,
                                    cudaStream_t stream, const Params& params, bool dependent,
                                    uint32_t cluster = 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    unsigned n = 0;
    if (dependent) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, params);
}

// The GEMM launch(es) of a plan: the pair regime first when the plan has one, then the
// single regime; the dispatch kernel's choice decides which of the two does the work.
// `pick` selects the parameter set of a regime (up, down or fused tiles).
template <bool kRaw, typename Pick>
static cudaError_t launch_gemms(const gcmoe::Plan* plan, Pick pick, cudaStream_t s, bool dependent, bool wait_tables,
                                float* raw_out) {
    auto prepare = [&](const gcmoe::Plan::Regime& regime) {
        GemmParams g = pick(regime);
        // Launched together with the call's dispatch kernel the GEMMs start while it runs and
        // wait for its tables; launched alone they find the tables of the last call in place.
        g.wait_tables = wait_tables ? 1u : 0u;
        if (kRaw) {
            g.seg[0] = g.seg[g.num_segments - 1];   // the routed gate/up segment alone
            g.num_segments = 1;
            g.raw_out = raw_out;
        }
        return g;
    };
    if (plan->pairs.grid != 0) {
        const GemmParams g = prepare(plan->pairs);
        cudaError_t err = launch_dependent(grouped_gemm_kernel<kRaw, true>, plan->pairs.grid, kGemmThreads,
                                           plan->pairs.smem, s, g, dependent, 2);
        if (err != cudaSuccess) return err;
        dependent = true;
    }
    const GemmParams g = prepare(plan->single);
    return launch_dependent(grouped_gemm_kernel<kRaw, false>, plan->single.grid, kGemmThreads, plan->single.smem, s, g,
                            dependent);
}

extern "C" int gcmoe_kernels_per_launch(const gcmoe_plan* plan) {
    return plan == nullptr ? 0 : (plan->pairs.grid != 0 ? 4 : 3);
}

extern "C" int gcmoe_launch_kernels(gcmoe_plan* plan, unsigned mask, void* cuda_stream) {
    if (plan == nullptr) return fail(GCMOE_ERR_INVALID, "null plan");
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    // Only a kernel launched together with its predecessor may overlap it.
    bool chained = false;
    if (mask & 1u) {
        GCMOE_CUDA(launch_dependent(dispatch_kernel, plan->dispatch_grid, kDispatchThreads, plan->dispatch_smem, s,
                                    plan->dispatch, false));
        chained = true;
    }
    if (mask & 6u) {
        // both GEMMs of the layer are one launch (per regime); either one alone is for tests and timing
        const unsigned which = mask & 6u;
        auto pick = [which](const gcmoe::Plan::Regime& r) -> const GemmParams& {
            return which == 6u ? r.fused : which == 2u ? r.up : r.down;
        };
        GCMOE_CUDA(launch_gemms<false>(plan, pick, s, chained, chained, nullptr));
        chained = true;
    } else chained = false;
    if (mask & 8u)
        GCMOE_CUDA(launch_dependent(combine_kernel, plan->combine_grid, kCombineThreads, 0, s, plan->combine, chained));
    GCMOE_CUDA(cudaGetLastError());
    return GCMOE_OK;
}

extern "C" int gcmoe_launch(gcmoe_plan* plan, void* cuda_stream) {
    return gcmoe_launch_kernels(plan, 15u, cuda_stream);
}

extern "C" int gcmoe_status_read(gcmoe_plan* plan, void* cuda_stream, uint32_t* words) {
    if (plan == nullptr || words == nullptr) return fail(GCMOE_ERR_INVALID, "null argument");
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    GCMOE_CUDA(cudaMemcpyAsync(words, plan->status, kStatusWords * 4, cudaMemcpyDeviceToHost, s));
    GCMOE_CUDA(cudaStreamSynchronize(s));
    if (words[kStatusCode] != 0)
        return fail(GCMOE_ERR_DEVICE,
                    "device wait gave up: code %u kernel %u site %u block %u observed %u expected %u",
                    words[kStatusCode], words[kStatusKernel], words[kStatusSite], words[kStatusBlock],
                    words[kStatusObserved], words[kStatusExpected]);
    return GCMOE_OK;
}

// A wait on a word nothing ever sets, with a short limit: exercises the timeout
// path (status block, sticky word, clean return) without any real failure.
__global__ void expire_wait_kernel(const uint32_t* never_set, uint32_t* status, uint32_t* failed,
                                   uint64_t timeout_ns) {
    __shared__ uint32_t abort_word;
    abort_word = 0;
    WaitCtl ctl;
    ctl.status = status;
    ctl.failed = failed;
    ctl.abort = &abort_word;
    ctl.timeout_ns = timeout_ns;
    ctl.kernel = kKernelDispatch;
    flag_wait_eq(never_set, 0xFFFFFFFFu, ctl, 99);
}

extern "C" int gcmoe_debug_expire_wait(gcmoe_plan* plan, unsigned timeout_us, void* cuda_stream) {
    if (plan == nullptr) return fail(GCMOE_ERR_INVALID, "null plan");
    const uint64_t arena = plan->buf.arena_base[plan->prob.rank];
    // word 7 of the status block is never written by any kernel and starts at zero
    expire_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        plan->status + 7, plan->status,
        reinterpret_cast<uint32_t*>(arena + plan->buf.off_exchange + exchange::kFailed), uint64_t(timeout_us) * 1000ull);
    GCMOE_CUDA(cudaGetLastError());
    return GCMOE_OK;
}

extern "C" int gcmoe_stage_inputs(const gcmoe_stage_args* args, void* cuda_stream) {
    if (args == nullptr) return fail(GCMOE_ERR_INVALID, "null argument");
    const gcmoe_stage_args& a = *args;
    if (a.num_tokens == 0) return GCMOE_OK;
    if (a.hidden == 0 || a.hidden % 256) return fail(GCMOE_ERR_INVALID, "hidden must be a positive multiple of 256");
    if (a.topk == 0 || a.topk > 32) return fail(GCMOE_ERR_INVALID, "topk must be in 1..32");
    if (a.x == 0 || a.x % 16 || a.x_q == 0 || a.x_q % 8 || a.x_sf == 0 || a.x_sf % 4 || a.topk_idx == 0 ||
        a.topk_idx % 8 || a.topk_weights == 0 || a.topk_weights % 4)
        return fail(GCMOE_ERR_INVALID, "activation or output address missing or misaligned");
    if (a.router_logits != 0) {
        if (a.router_logits % 4 || a.num_experts < a.topk || a.num_experts > 2048)
            return fail(GCMOE_ERR_INVALID, "router logits need topk <= num_experts <= 2048");
    } else if (a.topk_idx_in == 0 || a.topk_idx_in % 8 || a.topk_weights_in == 0 || a.topk_weights_in % 4) {
        return fail(GCMOE_ERR_INVALID, "neither router logits nor top-k arrays given");
    }
    if (a.shared_sf != 0 && (a.shared_sf % 4 || a.block_m == 0 || a.block_m % 16 ||
                             uint64_t((a.num_tokens + a.block_m - 1) / a.block_m) * round_up_u32(a.block_m, 128) >
                                 a.shared_sf_rows))
        return fail(GCMOE_ERR_INVALID, "shared scale view too small for %u tokens in blocks of %u", a.num_tokens,
                    a.block_m);
    StageParams p;
    p.x = reinterpret_cast<const uint4*>(a.x);
    p.logits = reinterpret_cast<const float*>(a.router_logits);
    p.idx_in = reinterpret_cast<const long long*>(a.topk_idx_in);
    p.weights_in = reinterpret_cast<const float*>(a.topk_weights_in);
    p.x_q = reinterpret_cast<uint2*>(a.x_q);
    p.x_sf = reinterpret_cast<uint32_t*>(a.x_sf);
    p.topk_idx = reinterpret_cast<long long*>(a.topk_idx);
    p.topk_weights = reinterpret_cast<float*>(a.topk_weights);
    p.shared_sf = reinterpret_cast<uint32_t*>(a.shared_sf);
    p.shared_sf_rows = a.shared_sf_rows;
    p.block_m = a.block_m;
    p.hidden = a.hidden; p.num_experts = a.num_experts; p.topk = a.topk;
    const size_t smem = a.router_logits != 0 ? size_t(a.num_experts) * 4 : 0;
    stage_inputs_kernel<<<a.num_tokens, kStageThreads, smem, static_cast<cudaStream_t>(cuda_stream)>>>(p);
    GCMOE_CUDA(cudaGetLastError());
    return GCMOE_OK;
}

extern "C" int gcmoe_transform_weights(const gcmoe_transform_args* args, void* cuda_stream) {
    if (args == nullptr) return fail(GCMOE_ERR_INVALID, "null argument");
    const gcmoe_transform_args& a = *args;
    if (a.groups == 0 || a.rows == 0 || a.row_bytes == 0) return GCMOE_OK;
    if ((a.segment_bytes != 64 && a.segment_bytes != 128) || a.row_bytes % a.segment_bytes)
        return fail(GCMOE_ERR_INVALID, "weight rows must hold whole K128 segments of 64 (FP4) or 128 (FP8) bytes");
    if (a.payload_in == 0 || a.payload_out == 0 || a.payload_in % 16 || a.payload_out % 16)
        return fail(GCMOE_ERR_INVALID, "weight payload missing or not 16-byte aligned");
    if (a.interleave_gate_up && a.rows % 16) return fail(GCMOE_ERR_INVALID, "W1 rows must be a multiple of 16");
    if (a.sf_out != 0) {
        if (a.rows % 128 || a.sf_packs == 0 || a.sf_out % 4)
            return fail(GCMOE_ERR_INVALID, "scale rows must be a multiple of 128 and the words 4-byte aligned");
        if (a.block_codes == 0 && (a.sf_in == 0 || a.sf_in % 4))
            return fail(GCMOE_ERR_INVALID, "neither scale words nor block codes given");
        if (a.block_codes != 0 && (a.groups != 1 || a.k_blocks == 0 || a.sf_packs != (a.k_blocks + 3) / 4))
            return fail(GCMOE_ERR_INVALID, "block codes need one matrix and ceil(k_blocks / 4) words per row");
    }
    TransformParams p = {};
    p.payload_in = reinterpret_cast<const uint4*>(a.payload_in);
    p.payload_out = reinterpret_cast<uint4*>(a.payload_out);
    p.sf_in = reinterpret_cast<const uint32_t*>(a.sf_in);
    p.sf_out = reinterpret_cast<uint32_t*>(a.sf_out);
    p.block_codes = reinterpret_cast<const uint8_t*>(a.block_codes);
    p.groups = a.groups; p.rows = a.rows; p.row_vecs = a.row_bytes / 16; p.seg_vecs = a.segment_bytes / 16;
    p.sf_packs = a.sf_packs; p.k_blocks = a.k_blocks;
    p.in_stride_g = a.sf_in_stride_g; p.in_stride_r = a.sf_in_stride_r; p.in_stride_p = a.sf_in_stride_p;
    p.out_stride_g = a.sf_out_stride_g; p.out_stride_r = a.sf_out_stride_r; p.out_stride_p = a.sf_out_stride_p;
    p.interleave = a.interleave_gate_up;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    auto blocks = [](uint64_t items) {
        const uint64_t b = (items + kTransformThreads - 1) / kTransformThreads;
        return unsigned(b < 1 ? 1 : (b > 148ull * 16 ? 148ull * 16 : b));
    };
    transform_payload_kernel<<<blocks(uint64_t(a.groups) * a.rows * p.row_vecs), kTransformThreads, 0, s>>>(p);
    if (a.sf_out != 0)
        transform_scales_kernel<<<blocks(uint64_t(a.groups) * a.rows * a.sf_packs), kTransformThreads, 0, s>>>(p);
    GCMOE_CUDA(cudaGetLastError());
    return GCMOE_OK;
}

extern "C" int gcmoe_debug_gemm_l1_raw(gcmoe_plan* plan, uint64_t out, void* cuda_stream) {
    if (plan == nullptr || out == 0) return fail(GCMOE_ERR_INVALID, "null argument");
    auto pick = [](const gcmoe::Plan::Regime& r) -> const GemmParams& { return r.up; };
    GCMOE_CUDA(launch_gemms<true>(plan, pick, static_cast<cudaStream_t>(cuda_stream), false, false,
                                  reinterpret_cast<float*>(out)));
    GCMOE_CUDA(cudaGetLastError());
    return GCMOE_OK;
}

// ---------------------------------------------------------------------------
// Layer call for callers that must not allocate device memory.
//
// Some hosts of this operator run with a frozen device heap: a serving loop
// whose memory pool was sized at start-up, or a worker that is already inside
// a region where cudaMalloc would synchronise or fail.  They cannot provide
// the plan-private scratch block the other entry points expect.  For them the
// scratch (status words, per-expert token counts, pool-block prefix) lives in
// the fixed device array below, which every GPU that loads the library
// holds until the process exits.
// ---------------------------------------------------------------------------
namespace gcmoe {

constexpr int kStaticMaxLocalExperts = 128;
constexpr size_t kStaticScratchBytes = 65536;  // status, counts, prefix for 128 local experts, tile counters of ~16000 row blocks
static_assert(kStaticScratchBytes >= kStatusWords * 4 + (5 * kStaticMaxLocalExperts + 2) * 4 + kCallInfoWords * 4 + 32, "static scratch too small");

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_static_scratch_address[kMaxDevices] = {};
static const uint32_t* g_static_last_failed_word[kMaxDevices] = {};   // sticky failure word of the last call's workspace
static std::mutex g_static_scratch_mutex;

// Device address of g_static_scratch on the current device.  In host code the
// array's name is only a handle; the address has to be asked for, once per
// device, while that device is current.
static int static_scratch_address(void** out) {
    int device = 0;
    GCMOE_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices)
        return fail(GCMOE_ERR_UNSUPPORTED, "device ordinal %d is outside the static scratch table", device);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_address[device] == nullptr) {
        void* ptr = nullptr;
        GCMOE_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch));
        g_static_scratch_address[device] = ptr;
    }
    *out = g_static_scratch_address[device];
    return GCMOE_OK;
}

}  // namespace gcmoe

extern "C" int gcmoe_launch_static_scratch(const gcmoe_problem* problem, const gcmoe_buffers* buffers,
                                           void* cuda_stream) {
    if (problem == nullptr || buffers == nullptr) return fail(GCMOE_ERR_INVALID, "null argument");
    if (problem->num_ranks <= 0 || problem->num_experts <= 0)
        return fail(GCMOE_ERR_INVALID, "invalid rank/expert configuration");
    const int local = problem->num_experts / problem->num_ranks;
    if (local > kStaticMaxLocalExperts)
        return fail(GCMOE_ERR_UNSUPPORTED,
                    "%d local experts exceed the %d the built-in scratch holds; use gcmoe_plan_create "
                    "with caller-provided scratch", local, kStaticMaxLocalExperts);
    if (gcmoe_scratch_bytes(problem) > kStaticScratchBytes)
        return fail(GCMOE_ERR_UNSUPPORTED,
                    "the tile counters of a ring of %d rows and a capacity of %d tokens need %zu bytes of scratch, "
                    "more than the %zu the built-in scratch holds; use gcmoe_plan_create with caller-provided scratch",
                    problem->ring_tokens, problem->capacity, gcmoe_scratch_bytes(problem), kStaticScratchBytes);
    void* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    gcmoe_buffers with_scratch = *buffers;
    with_scratch.scratch = reinterpret_cast<uint64_t>(scratch);
    with_scratch.scratch_bytes = kStaticScratchBytes;
    gcmoe_plan* plan = nullptr;
    if (int rc = gcmoe_plan_create(problem, &with_scratch, &plan)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    // The array keeps what the previous call left: the status words must start at zero, and so
    // must the call-info words (the tables-ready word the GEMM launch waits for, its tile
    // cursor), whose place depends on the geometry.  The rest is rewritten by the dispatch kernel.
    cudaError_t err = cudaMemsetAsync(scratch, 0, kStatusWords * 4, s);
    if (err == cudaSuccess)
        err = cudaMemsetAsync(const_cast<uint32_t*>(plan->single.fused.call_info), 0, kCallInfoWords * sizeof(uint32_t), s);
    int rc = err == cudaSuccess ? gcmoe_launch(plan, cuda_stream)
                                : fail(GCMOE_ERR_CUDA, "cudaMemsetAsync failed: %s", cudaGetErrorString(err));
    if (rc == GCMOE_OK) {
        // A workspace on which a wait has given up stays failed: its kernels return at once and write
        // nothing.  Remember where its sticky word lives so that the status query reports that too.
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        int device = 0;
        if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < kMaxDevices)
            g_static_last_failed_word[device] = plan->single.fused.failed;
    }
    gcmoe_plan_destroy(plan);   // host object only; the enqueued kernels carry their parameters by value
    return rc;
}

extern "C" int gcmoe_static_scratch_status(void* cuda_stream, uint32_t* words) {
    if (words == nullptr) return fail(GCMOE_ERR_INVALID, "null argument");
    void* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
    GCMOE_CUDA(cudaMemcpyAsync(words, scratch, kStatusWords * 4, cudaMemcpyDeviceToHost, s));
    const uint32_t* failed_word = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        int device = 0;
        if (cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < kMaxDevices)
            failed_word = g_static_last_failed_word[device];
    }
    uint32_t workspace_failed = 0;
    if (failed_word != nullptr)
        GCMOE_CUDA(cudaMemcpyAsync(&workspace_failed, failed_word, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    GCMOE_CUDA(cudaStreamSynchronize(s));
    if (words[kStatusCode] != 0)
        return fail(GCMOE_ERR_DEVICE, "device wait gave up: code %u kernel %u site %u block %u",
                    words[kStatusCode], words[kStatusKernel], words[kStatusSite], words[kStatusBlock]);
    if (workspace_failed != 0)
        return fail(GCMOE_ERR_DEVICE, "device wait gave up in an earlier call on this workspace: its kernels "
                                      "return at once until the workspace is re-created");
    return GCMOE_OK;
}
