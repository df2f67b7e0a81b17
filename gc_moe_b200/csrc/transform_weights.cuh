// Weight re-layout on the GPU: what transform_weights_for_gc_moe does once per
// weight set (gc_moe/gc/__init__.py:166-223,
// gc_moe/jit_kernels/impls/runtime_utils.py:86-118), as two byte-permuting
// kernels instead of a chain of torch reshapes and copies:
//   * payload [G][rows][row_bytes] -> [G][row_bytes / seg][rows][seg] (seg = 64
//     bytes of packed FP4 or 128 bytes of FP8 = one K128 block), so that a
//     (K128 block, 128 or 256 rows) weight tile is one contiguous range;
//   * for gate/up weights the rows are interleaved on the way: output rows come in
//     groups of 16, 8 gate rows then the 8 up rows of the same channels;
//   * packed scale words: the same row interleave, then inside every 128 rows
//     row u moves to position (u % 32) * 4 + u / 32, the order tcgen05.cp lays
//     128 scale words across 32 TMEM lanes x 4 columns;
//   * optionally the scale words are first built from one UE8M0 byte per
//     128 x 128 block (block-row scale expansion: every row of a block row gets
//     the block's bytes, four K128 blocks per word, missing bytes = 127).
// HBM-bound: 16-byte vectors, every byte read and written once.
#pragma once

#include "device_common.cuh"

namespace gcmoe {

constexpr int kTransformThreads = 256;

struct TransformParams {
    const uint4* payload_in;
    uint4* payload_out;
    const uint32_t* sf_in;         // packed words, or null when block_codes is given
    uint32_t* sf_out;
    const uint8_t* block_codes;    // [rows / 128][k_blocks] or null
    uint32_t groups, rows, row_vecs, seg_vecs;     // row_vecs = row_bytes / 16, seg_vecs = segment_bytes / 16
    uint32_t sf_packs, k_blocks;
    uint64_t in_stride_g, in_stride_r, in_stride_p;      // elements
    uint64_t out_stride_g, out_stride_r, out_stride_p;
    uint32_t interleave;           // gate/up row interleave
};

// Source row of output row `o`: [gate(0..R/2) ; up(0..R/2)] -> groups of 16 = 8 gate + 8 up.
__device__ __forceinline__ uint32_t transform_source_row(uint32_t o, uint32_t rows, bool interleave) {
    if (!interleave) return o;
    const uint32_t group = o >> 4, j = o & 15u;
    return (j < 8u ? 0u : rows / 2) + group * 8u + (j & 7u);
}

__global__ void __launch_bounds__(kTransformThreads) transform_payload_kernel(const TransformParams p) {
    const uint64_t per_group = static_cast<uint64_t>(p.rows) * p.row_vecs;
    const uint64_t total = per_group * p.groups;
    const uint32_t tiles = p.row_vecs / p.seg_vecs;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kTransformThreads + threadIdx.x; i < total;
         i += static_cast<uint64_t>(gridDim.x) * kTransformThreads) {
        // output index: [g][tile][row][vec inside the segment]
        const uint32_t g = static_cast<uint32_t>(i / per_group);
        uint64_t r = i - g * per_group;
        const uint32_t v = static_cast<uint32_t>(r % p.seg_vecs);
        r /= p.seg_vecs;
        const uint32_t row = static_cast<uint32_t>(r % p.rows), tile = static_cast<uint32_t>(r / p.rows);
        (void)tiles;
        const uint32_t src = transform_source_row(row, p.rows, p.interleave != 0);
        p.payload_out[i] = p.payload_in[g * per_group + static_cast<uint64_t>(src) * p.row_vecs + tile * p.seg_vecs + v];
    }
}

__global__ void __launch_bounds__(kTransformThreads) transform_scales_kernel(const TransformParams p) {
    const uint64_t per_group = static_cast<uint64_t>(p.rows) * p.sf_packs;
    const uint64_t total = per_group * p.groups;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * kTransformThreads + threadIdx.x; i < total;
         i += static_cast<uint64_t>(gridDim.x) * kTransformThreads) {
        // consecutive threads take consecutive output rows of one plane (MN-major: unit stride)
        const uint32_t g = static_cast<uint32_t>(i / per_group);
        const uint64_t r = i - g * per_group;
        const uint32_t pack = static_cast<uint32_t>(r / p.rows), o = static_cast<uint32_t>(r % p.rows);
        const uint32_t pos = o & 127u, u = (pos & 3u) * 32u + (pos >> 2);      // position -> row inside the 128
        const uint32_t src = transform_source_row((o & ~127u) + u, p.rows, p.interleave != 0);
        uint32_t word;
        if (p.block_codes != nullptr) {
            word = 0;
#pragma unroll
            for (uint32_t b = 0; b < 4; ++b) {
                const uint32_t kb = pack * 4 + b;
                const uint32_t code = kb < p.k_blocks ? p.block_codes[static_cast<size_t>(src / 128) * p.k_blocks + kb] : 127u;
                word |= code << (8 * b);
            }
        } else {
            word = p.sf_in[g * p.in_stride_g + src * p.in_stride_r + pack * p.in_stride_p];
        }
        p.sf_out[g * p.out_stride_g + o * p.out_stride_r + pack * p.out_stride_p] = word;
    }
}

}  // namespace gcmoe
