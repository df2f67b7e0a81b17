/*
 * C ABI of libgcmoe_sm100.so: the B200 (sm_100a) implementation of the
 * fp8 x fp4 MoE layer behind the reference operator's Python API.
 *
 * The library replaces everything below the reference's launch seam
 *   launch_gc_moe(config, y, l1_weights, l2_weights, call_buffer, shared_l1,
 *                 shared_l2, stats)
 *   (gc_moe/jit_kernels/impls/sm100_fp8_fp4_gc_moe.py:721-727)
 * i.e. its JIT (gc_moe/runtime/jit.py), its launch runtime
 * (gc_moe/runtime/gc_moe.py:369-418) and its role kernels
 * (gc_moe/impls/sm100_fp8_fp4_gc_moe.py).  Plain C types only: pointers are
 * device addresses passed as integers, sizes are element counts, and every
 * function returns 0 on success or a negative gcmoe_error; the message of the
 * last failure on the calling thread is available from gcmoe_last_error().
 *
 * Nothing here allocates device memory unless its comment says so: the caller
 * owns the symmetric arena, the weights, the output and the scratch block.
 */
#ifndef GCMOE_H_
#define GCMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GCMOE_MAX_RANKS 72
#define GCMOE_STATUS_WORDS 8

typedef enum gcmoe_error {
    GCMOE_OK = 0,
    GCMOE_ERR_INVALID = -1,     /* contract violation in the arguments          */
    GCMOE_ERR_UNSUPPORTED = -2, /* geometry the kernels do not cover            */
    GCMOE_ERR_CUDA = -3,        /* a CUDA runtime or driver call failed         */
    GCMOE_ERR_DEVICE = -4       /* a kernel's bounded wait ran out (see status) */
} gcmoe_error;

/* Geometry of one call.  Mirrors the reference's ValidatedCall
 * (gc_moe/apis/gc_moe.py:19-31) plus the buffer geometry it reads from
 * GCSymmBuffer (gc_moe/gc/__init__.py:35-58). */
typedef struct gcmoe_problem {
    int32_t num_ranks;          /* P, ranks of the expert-parallel group        */
    int32_t rank;               /* this rank                                    */
    int32_t num_experts;        /* E, routed experts over all ranks             */
    int32_t capacity;           /* token capacity per rank (1920-aligned)       */
    int32_t topk;               /* k                                            */
    int32_t hidden;             /* H                                            */
    int32_t intermediate;       /* I of one routed expert                       */
    int32_t num_tokens;         /* T of this call on this rank (= y.shape[0])   */
    int32_t block_m;            /* get_block_m_for_gc_moe(...) for this call    */
    int32_t ring_tokens;        /* rows of l1_acts / l2_acts                    */
    int32_t sf_ring_tokens;     /* rows of the two scale rings                  */
    int32_t num_shared_experts; /* 0 or the fused shared expert's I / I_routed  */
    int32_t shared_gran_k;      /* 32 or 128: K granularity of shared weight SF */
    int32_t has_clamp;          /* activation_clamp given                       */
    float clamp;                /* its value                                    */
    int32_t fast_math;          /* approx exp2/rcp in the SwiGLU sigmoid        */
    int32_t timeout_ms;         /* limit of every device-side wait (0 = 2000)   */
    int32_t num_sms;            /* SMs to use (0 = all of the device)           */
    int32_t dispatch_sms;       /* upper bound of the dispatch kernel's CTAs, one
                                 * per SM (0 = 32, more for calls with more than 8192 routes).  The expert GEMMs start while
                                 * the dispatch kernel runs and take the other
                                 * SMs at once: the SM split the reference makes
                                 * with green contexts and GC_MOE_DISPATCH_SMS
                                 * (gc_moe/runtime/gc_moe.py:42-49,85-100)       */
} gcmoe_problem;

/* Device addresses.  `arena_base[r]` is rank r's symmetric arena as mapped in
 * THIS process (GCSymmBuffer.peer_addresses, gc_moe/gc/__init__.py:64-69);
 * the off_* members are byte offsets inside an arena, taken from the
 * reference-compatible layout (gc_moe/layout/gc_moe.py:110-251). */
typedef struct gcmoe_buffers {
    uint64_t arena_base[GCMOE_MAX_RANKS];
    uint64_t off_recv_parity, off_routed_pool_blocks;
    uint64_t off_recv_count, off_recv_count_sum;
    uint64_t off_index_table, off_metadata;
    uint64_t off_x, off_x_sf, off_topk_idx, off_topk_weights;
    uint64_t off_l1_acts, off_l1_acts_sf, off_l1_topk_weights;
    uint64_t off_l2_acts, off_l2_acts_sf, off_combine_tokens;
    uint64_t off_shared_l1_acts_sf, off_shared_l2_acts, off_shared_l2_acts_sf;
    uint64_t shared_sf_rows;      /* rows of the two shared scale views          */
    uint64_t y;                   /* bf16 [T, H], 16-byte aligned                */
    uint64_t stats;               /* int32 [E/P] cumulative counter, or 0        */
    uint64_t w1, w1_sf;           /* int8 [E/P, H/128, 2I, 64]; int32 MN-major   */
    uint64_t w2, w2_sf;           /* int8 [E/P, I/128, H, 64];  int32 MN-major   */
    uint64_t w1_sf_stride, w2_sf_stride;   /* words between K128 planes          */
    uint64_t sw1, sw1_sf, sw2, sw2_sf;     /* fused shared expert, or 0          */
    uint64_t sw1_sf_stride, sw2_sf_stride;
    uint64_t scratch;             /* gcmoe_scratch_bytes() bytes, zero-filled    */
    uint64_t scratch_bytes;
    uint64_t off_exchange;        /* required: byte offset of 8 MiB of the arena
                                   * for this library's own cross-rank counters
                                   * and its sticky failure word; the reference
                                   * layout's unused `l2_full_mask` signal region */
} gcmoe_buffers;

typedef struct gcmoe_plan gcmoe_plan;

/* Library version: major * 10000 + minor * 100 + patch. */
int gcmoe_version(void);

/* Message of the last error returned on this thread ("" if none). */
const char* gcmoe_last_error(void);

/* Bytes of plan-private device scratch a plan for `problem` needs (status
 * block, per-expert counts, pool-block prefix, call info, per-block tile
 * counters).  The caller allocates and
 * zero-fills it once. */
size_t gcmoe_scratch_bytes(const gcmoe_problem* problem);

/* Validate the geometry, encode the TMA descriptors and precompute the launch
 * configuration of the layer's kernels.  Replaces prepare_role_binaries
 * (gc_moe/jit_kernels/impls/sm100_fp8_fp4_gc_moe.py:551-719).  No device
 * memory is allocated; the plan stays valid while the addresses in `buffers`
 * do. */
int gcmoe_plan_create(const gcmoe_problem* problem, const gcmoe_buffers* buffers,
                      gcmoe_plan** plan);
int gcmoe_plan_destroy(gcmoe_plan* plan);

/* Enqueue one layer call (dispatch, the expert GEMMs, combine) on
 * `cuda_stream` (a cudaStream_t).  Plain stream launches: a caller that is
 * capturing the stream into a CUDA graph captures the layer.  Replaces
 * GreenContextPair.launch (gc_moe/runtime/gc_moe.py:369-418). */
int gcmoe_launch(gcmoe_plan* plan, void* cuda_stream);

/* Enqueue only the kernels selected by `kernel_mask` (bit 0 dispatch, bit 1
 * gate/up tiles, bit 2 down tiles, bit 3 combine); bits 1 and 2 together are
 * the layer's single GEMM launch, either alone runs only those tiles.  Kernels
 * enqueued by one call may overlap (the GEMM launch starts while the dispatch
 * kernel is still pushing rows); kernels enqueued by separate calls run one
 * after the other, which is how per-kernel times are taken.  A GEMM launch
 * without its dispatch kernel reuses the tables of the last complete call. */
int gcmoe_launch_kernels(gcmoe_plan* plan, unsigned kernel_mask, void* cuda_stream);

/* Number of kernels gcmoe_launch enqueues per call. */
int gcmoe_kernels_per_launch(const gcmoe_plan* plan);

/* Copy the plan's device status block to `words` (GCMOE_STATUS_WORDS values)
 * after synchronising `cuda_stream`.  Returns GCMOE_ERR_DEVICE if a bounded
 * wait ran out; the reference traps the GPU instead
 * (gc_moe/comm/gc_barrier.py:44-80). */
int gcmoe_status_read(gcmoe_plan* plan, void* cuda_stream, uint32_t* words);

/* Raw grouped GEMM over the pool of the last complete call: FP32 accumulators
 * of W1 x pool rows to `out` ([pool rows][2I] floats, row r of the pool at
 * out[r * 2I], weight rows in the transformed (gate/up interleaved) order).
 * Test hook for the MMA, descriptor and scale plumbing of both tile regimes
 * (gc_moe/mma/sm100.py:22-254 is what it stands in for). */
int gcmoe_debug_gemm_l1_raw(gcmoe_plan* plan, uint64_t out, void* cuda_stream);

/* Enqueue a one-thread kernel that waits, for at most `timeout_us`, on a word
 * nothing sets: the wait runs out, the plan's status block and the workspace's
 * sticky failure word are set, and the kernel returns.  Lets a test exercise
 * failure detection on a healthy GPU; the reference's counterpart is the
 * timeout path of comm/gc_barrier.py:44-80, which traps instead. */
int gcmoe_debug_expire_wait(gcmoe_plan* plan, unsigned timeout_us, void* cuda_stream);

/* Inputs of gcmoe_stage_inputs: device addresses and element counts. */
typedef struct gcmoe_stage_args {
    uint64_t x;               /* bf16 [T, H] activations, rows 16-byte aligned     */
    uint64_t router_logits;   /* f32 [T, E], or 0 to copy the two arrays below     */
    uint64_t topk_idx_in;     /* int64 [T, k]  (router_logits == 0)                */
    uint64_t topk_weights_in; /* f32 [T, k]    (router_logits == 0)                */
    uint64_t x_q;             /* out: e4m3 [cap, H]       = GCSymmBuffer.x          */
    uint64_t x_sf;            /* out: int32 [cap, H/128]  = GCSymmBuffer.x_sf       */
    uint64_t topk_idx;        /* out: int64 [cap, k]      = GCSymmBuffer.topk_idx   */
    uint64_t topk_weights;    /* out: f32 [cap, k]        = GCSymmBuffer.topk_weights */
    uint64_t shared_sf;       /* out: MN-major int32 [shared_sf_rows, H/128] =
                               * GCSymmBuffer.shared_l1_acts_sf, or 0             */
    uint32_t shared_sf_rows;
    uint32_t block_m;         /* get_block_m_for_gc_moe(...) of the call (shared_sf) */
    uint32_t num_tokens, hidden, num_experts, topk;
} gcmoe_stage_args;

/* Upstream producer of a layer call, one kernel on `cuda_stream`: picks the k
 * largest router logits per token (descending, ties to the lower expert id)
 * with softmax weights over those k, quantises the BF16 rows to e4m3 with one
 * UE8M0 scale 2^ceil(log2(amax/448)) per 32 channels, and writes both straight
 * into the workspace views, including the shared expert's scale rows at
 * (t / BM) * align(BM,128) + (u & ~127) + (u & 31) * 4 + ((u >> 5) & 3),
 * u = t % BM.  Replaces the four copy_ kernels, the quantise kernel and the
 * index_put the reference leaves to the caller (README.md:234-252, 363-377;
 * "the scale staging can be fused into an upstream producer", README.md:387).
 * Allocates nothing; capturable. */
int gcmoe_stage_inputs(const gcmoe_stage_args* args, void* cuda_stream);

/* One weight matrix (or one stack of per-expert matrices) of
 * gcmoe_transform_weights: device addresses and element counts. */
typedef struct gcmoe_transform_args {
    uint64_t payload_in;      /* [groups][rows][row_bytes]: packed FP4 int8 [E][rows][K/2]
                               * or FP8 [rows][K] (groups = 1)                          */
    uint64_t payload_out;     /* [groups][row_bytes / segment_bytes][rows][segment_bytes] */
    uint64_t sf_in;           /* int32 packed scale words [groups][rows][sf_packs] with the
                               * element strides below, or 0 when block_codes is given */
    uint64_t sf_out;          /* same shape, strides below                             */
    uint64_t block_codes;     /* uint8 [rows / 128][k_blocks]: one UE8M0 byte per
                               * 128 x 128 block, expanded on the fly; or 0           */
    uint64_t sf_in_stride_g, sf_in_stride_r, sf_in_stride_p;     /* in elements */
    uint64_t sf_out_stride_g, sf_out_stride_r, sf_out_stride_p;
    uint32_t groups, rows, row_bytes, segment_bytes;   /* segment: 64 (FP4) or 128 (FP8) */
    uint32_t sf_packs, k_blocks;
    uint32_t interleave_gate_up;   /* 1 for W1: rows [gate ; up] -> groups of 8 + 8   */
    uint32_t reserved;
} gcmoe_transform_args;

/* Re-layout one weight set for the kernels, two launches on `cuda_stream`: the
 * K128 tile repack of the payload, and the scale words' row interleave and 4 x 32
 * transpose (with the block-row expansion of 128 x 128 scales when block_codes is
 * given).  Produces the bytes of transform_weights_for_gc_moe
 * (gc_moe/gc/__init__.py:166-223; gc_moe/jit_kernels/impls/runtime_utils.py:86-118).
 * Allocates nothing; input and output must not overlap. */
int gcmoe_transform_weights(const gcmoe_transform_args* args, void* cuda_stream);

/* One layer call for callers that cannot allocate device memory (no
 * counterpart in the reference, whose launch path allocates through its JIT
 * and graph caches).  Meant for hosts with a frozen device heap -- a serving
 * loop whose pool was sized at start-up, or code running where cudaMalloc
 * would synchronise or is forbidden -- which therefore cannot hand over the
 * scratch block gcmoe_plan_create asks for.  The kernels' scratch (status
 * words, per-expert token counts, pool-block prefix, per-block tile counters)
 * lives in a fixed 64 KiB device array inside the library instead, enough for
 * 128 local experts and about 15000 row-tile counters (ring_tokens / 16 +
 * capacity / 16 of them are reserved); a problem beyond either limit is
 * rejected with GCMOE_ERR_UNSUPPORTED and a message that names the limit.
 * `buffers->scratch` is ignored; the arena, weights and y are still the
 * caller's.  No cudaMalloc / cudaFree or any other allocating device routine
 * is called; one small host object lives for the duration of the call.
 *
 * Host cost: unlike gcmoe_launch, which reuses a plan, every call here checks
 * the geometry again and encodes the layer's tensor maps again on the host
 * (tens of microseconds) before it enqueues anything.
 *
 * The first call on a device looks up the array's device address; make that
 * first call before starting any stream capture on that device.  All calls on
 * a device share the one array: its status words and call-info words (the
 * tables-ready word, the GEMM launch's tile cursor) are cleared on the stream
 * before the kernels, the rest is rewritten by the dispatch kernel, and two
 * calls whose kernels overlap on the GPU (different streams) race on it. */
int gcmoe_launch_static_scratch(const gcmoe_problem* problem, const gcmoe_buffers* buffers,
                                void* cuda_stream);

/* Status words of the built-in scratch after synchronising `cuda_stream`
 * (same meaning as gcmoe_status_read).  Each call clears the status words, so
 * a wait that gave up is in them only until the next call; the failure stays
 * visible all the same, because this query also reads the sticky failure word
 * of the workspace the last call used and returns GCMOE_ERR_DEVICE while it
 * is set (the kernels of such a workspace return at once and leave y alone). */
int gcmoe_static_scratch_status(void* cuda_stream, uint32_t* words);

#ifdef __cplusplus
}
#endif
#endif /* GCMOE_H_ */
