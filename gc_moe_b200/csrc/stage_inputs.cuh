// Upstream producer of one layer call: router top-k + softmax, FP8/UE8M0
// quantisation of the BF16 activations and the shared expert's scale staging,
// written straight into the workspace views the layer reads.
//
// The reference leaves this to the caller as four copy_ kernels, a quantise
// kernel from a third-party package and an index_put for the shared scales
// (README.md:234-252, 363-377; tests/test_gc_moe.py:368-372) and notes that
// "the scale staging can be fused into an upstream producer" (README.md:387).
// This kernel is that producer: one CTA per token, one pass over the row.
//
// Formats (the ones the layer decodes, tests/test_gc_moe_se.py:167-179,193-197):
//   x_q      e4m3 [T][H], value = x / 2^(code-127), round to nearest even, saturating
//   x_sf     int32 [T][H/128], byte j of word w = code of K-block 4w+j,
//            code = biased exponent of the smallest power of two >= amax/448 (min 0)
//   topk_idx int64 [T][k], topk_weights f32 [T][k]: the k largest logits in
//            descending order (ties: lower expert id first), softmax over those k
//   shared scale rows: word (t, w) also at
//            shared_sf[w * shared_sf_rows + (t / BM) * align(BM,128) + sf_row_in_block(t % BM)]
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_common.cuh"
#include "ptx.cuh"

namespace gcmoe {

constexpr int kStageThreads = 256;

struct StageParams {
    const uint4* x;               // bf16 [T][H], 16-byte aligned rows
    const float* logits;          // f32 [T][E] or null
    const long long* idx_in;      // int64 [T][k] (used when logits == null)
    const float* weights_in;      // f32 [T][k]   (used when logits == null)
    uint2* x_q;                   // e4m3 [cap][H]
    uint32_t* x_sf;               // int32 [cap][H/128]
    long long* topk_idx;          // int64 [cap][k]
    float* topk_weights;          // f32 [cap][k]
    uint32_t* shared_sf;          // MN-major int32 [shared_sf_rows][H/128] or null
    uint32_t shared_sf_rows;
    uint32_t block_m;
    uint32_t hidden, num_experts, topk;
};

// Biased exponent of the smallest power of two >= amax / 448 for a finite
// non-negative amax whose mantissa has at most 7 fraction bits (BF16): 448 is
// 1.75 * 2^8, so the exponent goes up by one exactly when the mantissa exceeds
// 1.75 (fraction 0x600000), and the result is floored at code 0 (2^-127).
__device__ __forceinline__ uint32_t ue8m0_code_for_e4m3(float amax) {
    const uint32_t bits = __float_as_uint(amax);
    const uint32_t up = (bits + 0x7fffffu - 0x600000u) >> 23;
    return (up > 8u ? up : 8u) - 8u;
}

__global__ void __launch_bounds__(kStageThreads) stage_inputs_kernel(const StageParams p) {
    extern __shared__ float logit_row[];          // [E] when routing in the kernel
    const uint32_t t = blockIdx.x, tid = threadIdx.x, lane = tid & 31;
    const uint32_t chunks = p.hidden / 8, words = p.hidden / 128;

    // Routing runs in warp 0 after its share of the row; fetch the logits early.
    if (p.logits != nullptr)
        for (uint32_t e = tid; e < p.num_experts; e += kStageThreads)
            logit_row[e] = p.logits[static_cast<size_t>(t) * p.num_experts + e];

    uint32_t shared_row = 0;
    if (p.shared_sf != nullptr) {
        const uint32_t block = t / p.block_m;
        shared_row = block * round_up_u32(p.block_m, 128) + sf_row_in_block(t - block * p.block_m);
    }

    // 8 BF16 per thread and step; the four lanes of a 32-element group are adjacent.
    const uint4* row = p.x + static_cast<size_t>(t) * chunks;
    uint2* out = p.x_q + static_cast<size_t>(t) * chunks;
    for (uint32_t c = tid; c < chunks; c += kStageThreads) {      // chunks % 32 == 0: whole warps
        const uint4 raw = row[c];
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const uint32_t code = ue8m0_code_for_e4m3(amax);
        const float inv = __uint_as_float((254u - code) << 23);    // 2^(127 - code)
        uint32_t q[2];
#pragma unroll
        for (int i = 0; i < 2; ++i)
            q[i] = uint32_t(ptx::cvt_e4m3x2(v[4 * i] * inv, v[4 * i + 1] * inv)) |
                   (uint32_t(ptx::cvt_e4m3x2(v[4 * i + 2] * inv, v[4 * i + 3] * inv)) << 16);
        out[c] = make_uint2(q[0], q[1]);
        // four groups (16 lanes) make one packed scale word
        const uint32_t base = lane & 16u;
        const uint32_t word = __shfl_sync(0xffffffffu, code, base) |
                              (__shfl_sync(0xffffffffu, code, base + 4) << 8) |
                              (__shfl_sync(0xffffffffu, code, base + 8) << 16) |
                              (__shfl_sync(0xffffffffu, code, base + 12) << 24);
        if ((lane & 15u) == 0) {
            const uint32_t wi = c >> 4;
            p.x_sf[static_cast<size_t>(t) * words + wi] = word;
            if (p.shared_sf != nullptr)
                p.shared_sf[static_cast<size_t>(wi) * p.shared_sf_rows + shared_row] = word;
        }
    }

    if (p.logits == nullptr) {
        for (uint32_t j = tid; j < p.topk; j += kStageThreads) {
            p.topk_idx[static_cast<size_t>(t) * p.topk + j] = p.idx_in[static_cast<size_t>(t) * p.topk + j];
            p.topk_weights[static_cast<size_t>(t) * p.topk + j] = p.weights_in[static_cast<size_t>(t) * p.topk + j];
        }
        return;
    }
    __syncthreads();
    if (tid >= 32) return;
    // k rounds of a warp-wide argmax; the winner is struck out of the row.
    float mine = 0.f, top = 0.f;
    uint32_t mine_idx = 0;
    for (uint32_t j = 0; j < p.topk; ++j) {
        float best = -INFINITY;
        uint32_t best_idx = 0xFFFFFFFFu;
        for (uint32_t e = lane; e < p.num_experts; e += 32) {
            const float v = logit_row[e];
            if (v > best || (best_idx == 0xFFFFFFFFu && v == best)) { best = v; best_idx = e; }
        }
#pragma unroll
        for (uint32_t d = 16; d > 0; d >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, d);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, best_idx, d);
            if (ov > best || (ov == best && oi < best_idx)) { best = ov; best_idx = oi; }
        }
        if (j == 0) top = best;
        if (lane == j) { mine = best; mine_idx = best_idx; }
        if (lane == 0 && best_idx != 0xFFFFFFFFu) logit_row[best_idx] = -INFINITY;
        __syncwarp();
    }
    const float ex = lane < p.topk ? expf(mine - top) : 0.f;
    float sum = ex;
#pragma unroll
    for (uint32_t d = 16; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
    if (lane < p.topk) {
        p.topk_idx[static_cast<size_t>(t) * p.topk + lane] = mine_idx == 0xFFFFFFFFu ? -1ll : static_cast<long long>(mine_idx);
        p.topk_weights[static_cast<size_t>(t) * p.topk + lane] = ex / sum;
    }
}

}  // namespace gcmoe
