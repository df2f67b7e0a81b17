"""GPU parity of the upstream producer (router top-k, FP8/UE8M0 quantisation,
shared-expert scale staging) against the CPU oracle, through the public
function and so through the C ABI.

Bytes and integers (e4m3 codes, scale words, expert ids, staged scale rows)
must be bit-exact; the softmax weights are floating point: absolute error at
most 2e-6 (a few FP32 ulps of values in [0, 1]).
"""
import numpy as np
import pytest
import torch

import gc_moe_b200 as G
from oracle import gcmoe_oracle as O

from _cases import LayerCase

pytestmark = pytest.mark.gpu

WEIGHT_ATOL = 2e-6


def _inputs(tokens, hidden, experts, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((tokens, hidden), generator=g) * scale).to(torch.bfloat16)
    logits = torch.randn((tokens, experts), generator=g)
    return x, logits


def _check_views(buf, x, logits, topk):
    tokens = x.shape[0]
    xq, xsf = O.quantize_act_fp8(x)
    idx, w = O.route_topk(logits, topk)
    assert np.array_equal(buf.x[:tokens].view(torch.uint8).cpu().numpy(), xq.view(torch.uint8).numpy())
    assert np.array_equal(buf.x_sf[:tokens].cpu().numpy(), xsf.numpy())
    assert np.array_equal(buf.topk_idx[:tokens].cpu().numpy(), idx.numpy())
    got_w = buf.topk_weights[:tokens].cpu()
    assert float((got_w - w).abs().max()) <= WEIGHT_ATOL
    assert float((got_w.sum(-1) - 1).abs().max()) <= 1e-5
    return xq, xsf, idx, w


@pytest.mark.parametrize('tokens,hidden,experts,topk', [
    (1, 1024, 8, 2), (16, 1024, 8, 2), (37, 4096, 64, 8), (256, 7168, 256, 8), (5, 2048, 384, 6)])
def test_quantised_rows_scales_and_routes_match_the_oracle(single_rank_group, tokens, hidden, experts, topk):
    buf = G.get_symm_buffer_for_gc_moe(single_rank_group, experts, 256, topk, hidden, 512)
    try:
        x, logits = _inputs(tokens, hidden, experts, seed=tokens + hidden)
        # rows that exercise the scale rule: zeros, exact powers of two times 448,
        # the largest and smallest BF16 magnitudes that occur in practice, one hot channel
        x[0, :32] = 0
        if tokens > 1:
            x[1, :32] = torch.tensor([448.0 * 2.0 ** (j - 16) for j in range(32)]).to(torch.bfloat16)
            x[1, 32:64] = 1.75
            x[1, 64:96] = 1.7578125          # 1.75 + 2^-7: the next BF16 above the scale boundary
            x[1, 96:128] = 0
            x[1, 100] = 3.0e4
            x[1, 128:160] = 1.0e-30
        buf.x.view(torch.uint8).fill_(0xAA)
        block_m = G.stage_inputs_for_gc_moe(buf, x.cuda(), logits.cuda())
        torch.cuda.synchronize()
        assert block_m == G.get_block_m_for_gc_moe(1, experts, buf.num_max_tokens_per_rank, tokens, topk)
        _check_views(buf, x, logits, topk)
        # rows past T are not written
        assert int(buf.x[tokens:tokens + 1].view(torch.uint8).min()) == 0xAA
    finally:
        buf.destroy()


def test_ties_go_to_the_lower_expert_id(single_rank_group):
    buf = G.get_symm_buffer_for_gc_moe(single_rank_group, 64, 256, 8, 1024, 512)
    try:
        x, logits = _inputs(4, 1024, 64, seed=3)
        logits[0] = 0.0                        # all equal: experts 0..7
        logits[1] = torch.arange(64).float() // 4      # groups of four equal values
        logits[2, 10:20] = 5.0
        G.stage_inputs_for_gc_moe(buf, x.cuda(), logits.cuda())
        torch.cuda.synchronize()
        _, _, idx, _ = _check_views(buf, x, logits, 8)
        assert idx[0].tolist() == list(range(8))
        assert idx[1].tolist() == [60, 61, 62, 63, 56, 57, 58, 59]
    finally:
        buf.destroy()


def test_ready_routes_are_copied(single_rank_group):
    buf = G.get_symm_buffer_for_gc_moe(single_rank_group, 8, 256, 2, 1024, 512)
    try:
        x, _ = _inputs(9, 1024, 8, seed=4)
        idx = torch.tensor([[0, 7], [3, -1], [8, 2], [1, 1], [5, 4], [6, 0], [2, 3], [7, 7], [4, 5]])
        w = torch.rand((9, 2))
        G.stage_inputs_for_gc_moe(buf, x.cuda(), topk_idx=idx.cuda(), topk_weights=w.cuda())
        torch.cuda.synchronize()
        assert torch.equal(buf.topk_idx[:9].cpu(), idx)
        assert torch.equal(buf.topk_weights[:9].cpu(), w)
        xq, xsf = O.quantize_act_fp8(x)
        assert np.array_equal(buf.x[:9].view(torch.uint8).cpu().numpy(), xq.view(torch.uint8).numpy())
        assert np.array_equal(buf.x_sf[:9].cpu().numpy(), xsf.numpy())
    finally:
        buf.destroy()


def test_argument_errors(single_rank_group):
    buf = G.get_symm_buffer_for_gc_moe(single_rank_group, 8, 256, 2, 1024, 512)
    try:
        x, logits = _inputs(4, 1024, 8, seed=5)
        with pytest.raises(ValueError):
            G.stage_inputs_for_gc_moe(buf, x.float().cuda(), logits.cuda())
        with pytest.raises(ValueError):
            G.stage_inputs_for_gc_moe(buf, x.cuda())
        with pytest.raises(ValueError):
            G.stage_inputs_for_gc_moe(buf, x.cuda(), logits[:, :4].contiguous().cuda())
        with pytest.raises(ValueError):
            G.stage_inputs_for_gc_moe(buf, x[:, :512].contiguous().cuda(), logits.cuda())
    finally:
        buf.destroy()


@pytest.mark.parametrize('tokens', [1, 70, 200])
def test_producer_feeds_the_layer_with_a_fused_shared_expert(single_rank_group, tokens):
    """Producer + layer, captured in one CUDA graph, against the oracle run on the
    oracle's own quantised inputs and routes; the staged shared scale rows are
    checked word for word."""
    e, h, i, k, s = 8, 1024, 512, 2, 2
    case = LayerCase(single_rank_group, e, h, i, k, seed=8, num_shared_experts=s)
    try:
        g = torch.Generator().manual_seed(78)
        sw1, sc1 = O.quantize_block_fp8(torch.randn((2 * s * i, h), generator=g) * 0.02)
        sw2, sc2 = O.quantize_block_fp8(torch.randn((h, s * i), generator=g) * 0.02)
        shared = {'w1': sw1, 'w1_codes': sc1, 'w2': sw2, 'w2_codes': sc2}
        sl1, sl2 = G.transform_weights_for_gc_moe(
            (sw1.cuda(), O.expand_block_sf_rows(sc1, 2 * s * i).cuda()),
            (sw2.cuda(), O.expand_block_sf_rows(sc2, h).cuda()))
        x, logits = _inputs(tokens, h, e, seed=90 + tokens)
        xd, ld = x.cuda(), logits.cuda()
        y = torch.full((tokens, h), float('nan'), dtype=torch.bfloat16, device='cuda')

        def call():
            G.stage_inputs_for_gc_moe(case.buf, xd, ld)
            G.fp8_fp4_gc_moe(y, case.l1, case.l2, case.buf, sl1, sl2, activation_clamp=10.0,
                             shared_recipe=(1, 128, 128))
        call()                                   # eager: builds the plan
        torch.cuda.synchronize()
        case.buf.raise_on_device_error()
        xq, xsf, idx, w = _check_views(case.buf, x, logits, k)
        bm = case.block_m(tokens)
        want, rows = O.stage_shared_sf(xsf, bm, case.buf.shared_l1_acts_sf.shape[0])
        got = case.buf.shared_l1_acts_sf.cpu()
        assert torch.equal(got[rows], want[rows])
        ref = O.moe_layer([xq], [xsf], [idx], [case.buf.topk_weights[:tokens].cpu()], case.q1, case.c1,
                          case.q2, case.c2, [bm], clamp=10.0, shared=shared)
        first = y.cpu().clone()
        assert torch.isfinite(first.float()).all()
        assert O.cosine(first, ref.y[0]) >= 0.9999 and O.max_rel_err(first, ref.y[0]) <= 2.0 ** -6
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                call()
        for _ in range(3):
            y.fill_(float('nan'))
            graph.replay()
        torch.cuda.synchronize()
        case.buf.raise_on_device_error()
        assert torch.equal(y.cpu(), first)
    finally:
        case.close()
