"""Shared helpers of the GPU parity tests: build one seeded layer problem,
run it through the public operator API, and fetch the arena data products."""
from __future__ import annotations

import numpy as np
import torch

import gc_moe_b200 as G
from gc_moe_b200.layout import round_up, sf_row_in_block
from oracle import gcmoe_oracle as O

DEV = 'cuda'


class LayerCase:
    """One world-1 problem: quantised weights on the GPU in operator layout,
    a workspace, and the original CPU tensors for the oracle."""

    def __init__(self, group, num_experts, hidden, inter, topk, capacity=1920, seed=0, weight_std=0.02,
                 num_shared_experts=0):
        self.e, self.h, self.i, self.k = num_experts, hidden, inter, topk
        self.capacity = capacity
        # Quantise on the GPU (seconds instead of a minute at benchmark sizes);
        # the oracle gets CPU copies of the very same bytes.
        from gc_moe_b200 import quant
        g = torch.Generator(device=DEV).manual_seed(seed)
        gpu = []
        for rows, k in ((2 * inter, hidden), (hidden, inter)):
            payload = torch.empty((num_experts, rows, k // 2), dtype=torch.int8, device=DEV)
            codes = torch.empty((num_experts, rows, k // 32), dtype=torch.uint8, device=DEV)
            for e in range(num_experts):
                w = torch.randn((rows, k), device=DEV, generator=g) * weight_std
                payload[e], codes[e] = quant.quantize_weights_fp4(w)
            gpu.append((payload, codes))
        (self.q1, self.c1), (self.q2, self.c2) = [(a.cpu(), b.cpu()) for a, b in gpu]
        self.buf = G.get_symm_buffer_for_gc_moe(group, num_experts, capacity, topk, hidden, inter,
                                                num_shared_experts)
        self.l1, self.l2 = G.transform_weights_for_gc_moe(
            (gpu[0][0], quant.weight_scales_mn_major(gpu[0][1])),
            (gpu[1][0], quant.weight_scales_mn_major(gpu[1][1])))

    def block_m(self, tokens):
        return G.get_block_m_for_gc_moe(1, self.e, self.buf.num_max_tokens_per_rank, tokens, self.k)

    def stage(self, xq, xsf, idx, w):
        t = xq.shape[0]
        self.buf.x[:t].copy_(xq.to(DEV))
        self.buf.x_sf[:t].copy_(xsf.to(DEV))
        self.buf.topk_idx[:t].copy_(idx.to(DEV))
        self.buf.topk_weights[:t].copy_(w.to(DEV))

    def run(self, xq, xsf, idx, w, clamp=10.0, fast_math=True, stats=None, y=None, guard=0):
        """Stage the inputs, call the operator, return y on the CPU.  With
        `guard` rows of NaN around y the caller can check nothing else is written."""
        t = xq.shape[0]
        self.stage(xq, xsf, idx, w)
        if y is None:
            full = torch.full((t + 2 * guard, self.h), float('nan'), dtype=torch.bfloat16, device=DEV)
            y = full[guard:guard + t]
            self.full_y = full
        G.fp8_fp4_gc_moe(y, self.l1, self.l2, self.buf, cumulative_local_expert_recv_stats=stats,
                         activation_clamp=clamp, fast_math=fast_math)
        torch.cuda.synchronize()
        self.buf.raise_on_device_error()
        return y.cpu()

    def oracle(self, xq, xsf, idx, w, clamp=10.0):
        return O.moe_layer([xq], [xsf], [idx], [w], self.q1, self.c1, self.q2, self.c2,
                           [self.block_m(xq.shape[0])], clamp=clamp)

    # ---- arena data products of the last call (generation = parity before the call)
    def products(self, tokens, generation):
        lay, bm = self.buf.layout, self.block_m(tokens)
        e = self.e
        out = {}
        out['counts'] = self.buf.region('expert_recv_count').view(torch.int64)[generation * e:(generation + 1) * e].cpu().numpy()
        out['count_sum'] = (self.buf.region('expert_recv_count_sum').view(torch.int64)[generation * e:(generation + 1) * e]
                            .cpu().numpy() & 0xFFFFFFFF)
        out['pool_blocks'] = int(self.buf.region('routed_pool_blocks').view(torch.int32)[0])
        rows = out['pool_blocks'] * bm
        out['metadata'] = self.buf.region('token_src_metadata').view(torch.int32).reshape(-1, 3)[:rows].cpu().numpy()
        out['index_table'] = self.buf.region('src_token_topk_idx').view(torch.int32).reshape(e, 1, lay.capacity).cpu().numpy()
        out['l1_acts'] = self.buf.l1_acts.view(torch.uint8)[:rows].cpu().numpy()
        out['l1_weights'] = self.buf.buffer.narrow(0, lay.views['l1_topk_weights'].offset, rows * 4).view(torch.float32).cpu().numpy()
        sf_rows = out['pool_blocks'] * round_up(bm, 128)
        out['l1_acts_sf'] = self.buf.l1_acts_sf[:sf_rows].cpu().numpy()
        out['l2_acts'] = self.buf.l2_acts.view(torch.uint8)[:rows].cpu().numpy()
        out['l2_acts_sf'] = np.ascontiguousarray(self.buf.l2_acts_sf[:sf_rows].cpu().numpy()).view(np.uint8)
        return out

    def close(self):
        self.buf.destroy()


def sf_rows_of_pool(rows, bm):
    """Scale-ring row of each pool row."""
    return np.array([(r // bm) * round_up(bm, 128) + sf_row_in_block(r % bm) for r in rows], dtype=np.int64)


def check_requantised_intermediate(prod, ref, bm, name, max_fraction=1e-5):
    """The FP8 bytes and UE8M0 scale bytes of the requantised gate/up output against the oracle's,
    every mismatch counted and classified.

    The tensor core adds the products of a K block, and the K blocks of a row, in an order of its
    own; the oracle sums in numpy's.  The FP32 accumulators therefore differ in their last bits,
    and an element that sits on a rounding boundary -- of the BF16 rounding in front of SwiGLU or
    of the FP8 rounding behind it -- may come out one FP8 code away (a BF16 step is 2^-8 of the
    value, an e4m3 step 2^-3, so two flipped BF16 roundings still cross at most one FP8
    boundary).  When the element is the largest of its group of 32 and sits on a power of two,
    the group's scale byte moves by one and the group's payload bytes with it.  Nothing else is
    accepted: scale bytes differ by at most one; where the scale byte agrees a payload byte
    differs by at most one code (the sign only between the two zeros and the smallest
    magnitudes); and each kind stays below ``max_fraction`` of its population (or two, for
    small populations).  Measured on B200: none at 16 tokens of the small configuration and at
    1 and 8 tokens of the single-GPU benchmark geometry, 1, 1 and 4 payload bytes of 0.5, 2.1
    and 4.2 million at 32, 128 and 256 tokens, no scale byte.
    """
    valid = np.nonzero(ref.dispatch[0].metadata[:, 0] >= 0)[0]
    got = prod['l2_acts'][valid]
    want = ref.l2_acts[0].view(torch.uint8).numpy()[valid]
    got_sf = prod['l2_acts_sf'][sf_rows_of_pool(valid, bm)].reshape(len(valid), -1)
    want_sf = ref.l2_sf[0].numpy()[valid]
    assert got.shape == want.shape and got_sf.shape == want_sf.shape
    sf_delta = got_sf.astype(np.int16) - want_sf.astype(np.int16)
    assert np.abs(sf_delta).max(initial=0) <= 1
    moved = sf_delta != 0
    same_scale = ~np.repeat(moved, 32, axis=1)
    differs = (got != want) & same_scale
    got_mag, want_mag = (got & 0x7F).astype(np.int16), (want & 0x7F).astype(np.int16)
    sign_differs = ((got ^ want) & 0x80) != 0
    one_step = (np.abs(got_mag - want_mag) <= 1) & (~sign_differs | (got_mag + want_mag <= 1))
    assert one_step[differs].all()
    print(f'PARITY {name}: requantised intermediate: {int(differs.sum())} of {differs.size} payload bytes '
          f'one code away, {int(moved.sum())} of {moved.size} scale bytes one step away')
    assert moved.sum() <= max(2, max_fraction * moved.size) and differs.sum() <= max(2, max_fraction * differs.size)


def check_dispatch_products(prod, d, bm):
    """Exact comparison of the arena's dispatch data products with the oracle's."""
    assert np.array_equal(prod['counts'], d.counts[0])
    assert np.array_equal(prod['count_sum'], d.counts.sum(0))
    assert prod['pool_blocks'] == d.pool_blocks
    valid = np.nonzero(d.metadata[:, 0] >= 0)[0]
    assert np.array_equal(prod['metadata'][valid], d.metadata[valid])
    assert np.array_equal(prod['l1_acts'][valid], d.rows[valid])
    assert np.array_equal(prod['l1_weights'][valid], d.weights[valid])
    assert np.array_equal(prod['l1_acts_sf'][sf_rows_of_pool(valid, bm)], d.sf_words[valid])
    for (l, s), lst in d.index_lists.items():
        assert np.array_equal(prod['index_table'][l, s, :len(lst)].astype(np.uint32), lst)
