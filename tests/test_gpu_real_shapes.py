"""GPU parity at the per-rank shapes the benchmark times (world of one rank, 32
local experts): the expert-parallel decode geometry (hidden 7168), the fused
shared expert geometry (hidden 6144, shared intermediate 4096, 128 x 128
block scales) and the large-token regime (4096 tokens, three of the 32 experts
drawing half of the assignments).  These sizes exercise what the small cases
cannot: 56 K-stages per gate/up tile and 28 down slices per row tile, the
stage ring wrapping many times inside a tile, descriptor offsets near the top
of shared memory, and CTA-pair tiles of 240 tokens.

Tolerance, stated per configuration (y against the CPU oracle; the integer
dispatch products are compared bit for bit):
  decode H7168     cosine >= 0.99999, max |dy| <= 2^-7 of the largest |y|
  shared H6144     cosine >= 0.99999, max |dy| <= 2^-6 of the largest |y|
  large-token      cosine >= 0.99999, max |dy| <= 2^-6 of the largest |y|
(one BF16 ulp of the largest value is 2^-8 of it; the bound covers one flipped
FP8 rounding of an intermediate element propagated through the down projection.
Measured worst cases on B200: decode 1.9e-3, shared 6.0e-3 at 256 tokens -- the
shared branch adds a second FP8-requantised intermediate of twice the width --
large-token 1.7e-3; every case prints its own values).
"""
import pytest
import torch

import gc_moe_b200 as G
from oracle import gcmoe_oracle as O

from _cases import LayerCase, check_dispatch_products

pytestmark = pytest.mark.gpu


def parity(case):
    return int(case.buf.region('recv_parity').view(torch.int32)[0].item()) & 1


def report(name, y, ref):
    cos, err = O.cosine(y, ref), O.max_rel_err(y, ref)
    print(f'PARITY {name}: cosine {cos:.10f} max_rel_err {err:.3e}')
    return cos, err


@pytest.fixture(scope='module')
def decode(single_rank_group):
    case = LayerCase(single_rank_group, num_experts=32, hidden=7168, inter=2048, topk=8, seed=11)
    yield case
    case.close()


@pytest.mark.parametrize('tokens', [1, 16, 64, 256])
def test_decode_geometry_h7168(decode, tokens):
    xq, xsf, idx, w = O.make_tokens(tokens, decode.h, decode.e, decode.k, seed=500 + tokens)
    gen = parity(decode)
    y = decode.run(xq, xsf, idx, w, guard=1)
    ref = decode.oracle(xq, xsf, idx, w)
    check_dispatch_products(decode.products(tokens, gen), ref.dispatch[0], decode.block_m(tokens))
    cos, err = report(f'decode H7168 T={tokens} BM={decode.block_m(tokens)}', y, ref.y[0])
    assert torch.isfinite(y.float()).all() and cos >= 0.99999 and err <= 2.0 ** -7
    guard = decode.full_y.cpu()
    assert torch.isnan(guard[:1].float()).all() and torch.isnan(guard[-1:].float()).all()


@pytest.fixture(scope='module')
def shared_case(single_rank_group):
    e, h, i, k, s = 32, 6144, 2048, 8, 2
    case = LayerCase(single_rank_group, e, h, i, k, seed=12, num_shared_experts=s)
    g = torch.Generator().manual_seed(13)
    sw1, sc1 = O.quantize_block_fp8(torch.randn((2 * s * i, h), generator=g) * 0.02)
    sw2, sc2 = O.quantize_block_fp8(torch.randn((h, s * i), generator=g) * 0.02)
    case.shared = {'w1': sw1, 'w1_codes': sc1, 'w2': sw2, 'w2_codes': sc2}
    case.sl1, case.sl2 = G.transform_weights_for_gc_moe(
        (sw1.cuda(), O.expand_block_sf_rows(sc1, 2 * s * i).cuda()),
        (sw2.cuda(), O.expand_block_sf_rows(sc2, h).cuda()))
    yield case
    case.close()


@pytest.mark.parametrize('tokens', [1, 16, 64, 256])
def test_fused_shared_expert_geometry_h6144(shared_case, tokens):
    case = shared_case
    xq, xsf, idx, w = O.make_tokens(tokens, case.h, case.e, case.k, seed=600 + tokens)
    bm = case.block_m(tokens)
    case.stage(xq, xsf, idx, w)
    t = torch.arange(tokens)
    u = t % bm
    rows = (t // bm) * ((bm + 127) // 128 * 128) + (u // 128) * 128 + (u % 32) * 4 + (u % 128) // 32
    case.buf.shared_l1_acts_sf[rows.cuda()] = xsf.cuda()
    y = torch.full((tokens, case.h), float('nan'), dtype=torch.bfloat16, device='cuda')
    G.fp8_fp4_gc_moe(y, case.l1, case.l2, case.buf, case.sl1, case.sl2, activation_clamp=10.0,
                     shared_recipe=(1, 128, 128))
    torch.cuda.synchronize()
    case.buf.raise_on_device_error()
    ref = O.moe_layer([xq], [xsf], [idx], [w], case.q1, case.c1, case.q2, case.c2, [bm], clamp=10.0,
                      shared=case.shared)
    cos, err = report(f'shared H6144 T={tokens} BM={bm}', y.cpu(), ref.y[0])
    assert torch.isfinite(y.float()).all() and cos >= 0.99999 and err <= 2.0 ** -6


def test_large_token_geometry_h7168_skewed(single_rank_group):
    """4096 tokens x top-8 over 32 experts of hidden 7168, three experts (10 %)
    drawing half of the assignments: block-M 240, hot experts of about 5000 rows
    in 240-token CTA-pair tiles, ragged cold experts."""
    e, h, i, k, tokens = 32, 7168, 2048, 8, 4096
    case = LayerCase(single_rank_group, e, h, i, k, capacity=5760, seed=14)
    try:
        g = torch.Generator().manual_seed(15)
        x = torch.randn((tokens, h), generator=g).to(torch.bfloat16)
        weights = torch.full((e,), 0.5 / (e - 3))
        weights[[4, 17, 29]] = 0.5 / 3
        gumbel = -torch.log(-torch.log(torch.rand((tokens, e), generator=g)))
        top, idx = torch.topk(torch.log(weights) + gumbel, k, dim=-1, sorted=False)
        w = torch.softmax(top, dim=-1).float()
        idx = idx.to(torch.int64)
        xq, xsf = O.quantize_act_fp8(x)
        assert case.block_m(tokens) == 240
        gen = parity(case)
        y = case.run(xq, xsf, idx, w)
        ref = case.oracle(xq, xsf, idx, w)
        check_dispatch_products(case.products(tokens, gen), ref.dispatch[0], 240)
        cos, err = report('large-token H7168 T=4096 BM=240', y, ref.y[0])
        assert torch.isfinite(y.float()).all() and cos >= 0.99999 and err <= 2.0 ** -6
    finally:
        case.close()
