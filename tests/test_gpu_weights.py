"""The GPU weight re-layout (gcmoe_transform_weights behind
transform_weights_for_gc_moe) against the reference transform's golden bytes
and against the torch formulation of the same permutation; the block-row
expansion of 128 x 128 scales against the oracle's."""
import os

import numpy as np
import pytest
import torch

from gc_moe_b200 import weights
from oracle import gcmoe_oracle as O

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden')


def mn_major(t):
    return t.transpose(-1, -2).contiguous().transpose(-1, -2)


def test_gpu_transform_matches_reference_bytes():
    g = np.load(os.path.join(GOLDEN, 'weight_transform.npz'))
    w1, w2 = torch.from_numpy(g['in_w1']).cuda(), torch.from_numpy(g['in_w2']).cuda()
    sf1, sf2 = mn_major(torch.from_numpy(g['in_sf1']).cuda()), mn_major(torch.from_numpy(g['in_sf2']).cuda())
    (a1, s1), (a2, s2) = weights.transform_weights_for_gc_moe((w1, sf1), (w2, sf2))
    torch.cuda.synchronize()
    assert np.array_equal(a1.cpu().numpy(), g['out_w1']) and np.array_equal(a2.cpu().numpy(), g['out_w2'])
    assert np.array_equal(s1.cpu().numpy(), g['out_sf1']) and np.array_equal(s2.cpu().numpy(), g['out_sf2'])
    assert s1.stride(-2) == 1 and s2.stride(-2) == 1            # MN-major kept
    assert a1.data_ptr() != w1.data_ptr() and s1.data_ptr() != sf1.data_ptr()   # independent copies
    fp8 = torch.from_numpy(g['in_fp8']).view(torch.float8_e4m3fn).cuda()
    sfx = torch.zeros((256, 1), dtype=torch.int32, device='cuda')
    (c1, _), _ = weights.transform_weights_for_gc_moe((fp8, sfx), (fp8, sfx))
    assert np.array_equal(c1.cpu().view(torch.uint8).numpy(), g['out_fp8'])


@pytest.mark.parametrize('experts,rows,k', [(3, 256, 512), (2, 4096, 1024)])
def test_gpu_transform_equals_torch_formulation(experts, rows, k):
    gen = torch.Generator().manual_seed(experts * rows)
    w1 = torch.randint(-128, 128, (experts, rows, k // 2), generator=gen, dtype=torch.int8)
    w2 = torch.randint(-128, 128, (experts, k, rows // 2), generator=gen, dtype=torch.int8)
    sf1 = mn_major(torch.randint(0, 2 ** 31 - 1, (experts, rows, k // 128), generator=gen, dtype=torch.int32))
    sf2 = mn_major(torch.randint(0, 2 ** 31 - 1, (experts, k, rows // 128), generator=gen, dtype=torch.int32))
    want = weights.transform_weights_for_gc_moe((w1, sf1), (w2, sf2))                 # CPU tensors: torch ops
    got = weights.transform_weights_for_gc_moe((w1.cuda(), mn_major(sf1.cuda())), (w2.cuda(), mn_major(sf2.cuda())))
    for (gp, gs), (wp, ws) in zip(got, want):
        assert torch.equal(gp.cpu(), wp) and torch.equal(gs.cpu(), ws) and gs.stride() == ws.stride()


def test_block_codes_are_expanded_on_the_fly():
    """Raw 128 x 128 block codes give the same scale rows as expanding them to one
    packed row per output row first (K with a ragged last word: 6 blocks)."""
    gen = torch.Generator().manual_seed(5)
    rows, k = 512, 768
    w, codes = O.quantize_block_fp8(torch.randn((rows, k), generator=gen) * 0.02)
    w2, codes2 = O.quantize_block_fp8(torch.randn((k, rows), generator=gen) * 0.02)
    expanded = weights.transform_weights_for_gc_moe(
        (w.cuda(), O.expand_block_sf_rows(codes, rows).cuda()), (w2.cuda(), O.expand_block_sf_rows(codes2, k).cuda()))
    direct = weights.transform_weights_for_gc_moe((w.cuda(), codes.cuda()), (w2.cuda(), codes2.cuda()))
    for (dp, ds), (ep, es) in zip(direct, expanded):
        assert torch.equal(dp.view(torch.uint8), ep.view(torch.uint8))
        assert torch.equal(ds, es) and ds.stride() == es.stride()


def test_bad_arguments_are_refused():
    w = torch.zeros((2, 256, 64), dtype=torch.int8, device='cuda')
    sf = mn_major(torch.zeros((2, 256, 1), dtype=torch.int32, device='cuda'))
    with pytest.raises(ValueError):
        weights.transform_weights_for_gc_moe((w[:, :, :32], sf), (w, sf))            # not contiguous
    with pytest.raises(ValueError):
        weights.transform_weights_for_gc_moe((w.view(torch.uint8), sf), (w, sf))     # wrong dtype
    with pytest.raises(ValueError):
        weights.transform_weights_for_gc_moe((w, sf[:, :128]), (w, sf))              # SF rows do not match
