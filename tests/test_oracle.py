"""The CPU oracle against the golden fixtures made from the reference's own
CPU code, plus the identities that pin the parts restated from device code."""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from oracle import gcmoe_oracle as O

GOLDEN = os.path.join(os.path.dirname(__file__), 'golden')


def sha(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def _case_inputs(args):
    e, h, i, k, t, clamp, seed, drop = args
    q1, c1, q2, c2 = O.make_weights(e, h, i, seed=seed)
    xq, xsf, idx, w = O.make_tokens(t, h, e, k, seed=seed + 1)
    if drop:
        idx[::3, 0] = -1
    return q1, c1, q2, c2, xq, xsf, idx, w, clamp


@pytest.mark.parametrize('name', ['c0', 'c0_noclamp_invalid'])
def test_layer_matches_reference_processed_forward(name):
    """Bit-exact with reference_processed_moe_forward
    (tests/test_sm120_gc_moe.py:187-213) on the fixture inputs."""
    meta = json.load(open(os.path.join(GOLDEN, 'processed_forward.json')))[name]
    gold = np.load(os.path.join(GOLDEN, 'processed_forward.npz'))[f'{name}_y']
    q1, c1, q2, c2, xq, xsf, idx, w, clamp = _case_inputs(meta['args'])
    got_sha = sha(q1) + sha(c1) + sha(q2) + sha(c2) + sha(xq) + sha(xsf) + sha(idx) + sha(w)
    if got_sha != meta['inputs_sha']:
        pytest.skip('seeded inputs differ from the fixture generator (torch RNG changed)')
    assert sha(O.dequant_fp4(q1[0], c1[0]).to(torch.bfloat16)) == meta['w1_dequant_sha']
    assert sha(O.dequant_fp8(xq, O.sf_bytes(xsf))) == meta['x_dequant_sha']
    res = O.moe_layer([xq], [xsf], [idx], [w], q1, c1, q2, c2, [16], clamp=clamp)
    assert np.array_equal(res.y[0].view(torch.int16).numpy(), gold)


def test_shared_expert_matches_reference_shared_forward():
    """Against reference_shared_forward with 128x128 block scales
    (tests/test_sm120_gc_moe.py:128-142).  The reference divides by the scale
    where the kernel order multiplies by its exact reciprocal: identical for
    powers of two."""
    g = np.load(os.path.join(GOLDEN, 'shared_forward.npz'))
    shared = {'w1': torch.from_numpy(g['sw1']).view(torch.float8_e4m3fn), 'w1_codes': torch.from_numpy(g['sc1']),
              'w2': torch.from_numpy(g['sw2']).view(torch.float8_e4m3fn), 'w2_codes': torch.from_numpy(g['sc2'])}
    xq = torch.from_numpy(g['xq']).view(torch.float8_e4m3fn)
    y = O.shared_expert(xq, torch.from_numpy(g['xsf']), shared, 10.0)
    gold = torch.from_numpy(g['y']).view(torch.bfloat16)
    assert O.cosine(y, gold) > 0.999999
    assert (y == gold).float().mean() > 0.999


def test_weight_transform_matches_reference_bytes():
    g = np.load(os.path.join(GOLDEN, 'weight_transform.npz'))
    w1, w2 = torch.from_numpy(g['in_w1']), torch.from_numpy(g['in_w2'])
    mn = lambda a: torch.from_numpy(a).transpose(1, 2).contiguous().transpose(1, 2)
    sf1, sf2 = mn(g['in_sf1']), mn(g['in_sf2'])
    (a1, s1), (a2, s2) = O.transform_weights((w1, sf1), (w2, sf2))
    assert np.array_equal(a1.numpy(), g['out_w1']) and np.array_equal(a2.numpy(), g['out_w2'])
    assert np.array_equal(s1.numpy(), g['out_sf1']) and np.array_equal(s2.numpy(), g['out_sf2'])
    for t, want in ((s1, g['out_sf1_strides']), (s2, g['out_sf2_strides'])):   # MN-major kept
        assert all(a == b for a, b, n in zip(t.stride(), want, t.shape) if n > 1)
    # the product's transform (host logic) gives the same bytes
    from gc_moe_b200.weights import transform_weights_for_gc_moe
    (b1, t1), (b2, t2) = transform_weights_for_gc_moe((w1, sf1), (w2, sf2))
    assert torch.equal(b1, a1) and torch.equal(b2, a2) and torch.equal(t1, s1) and torch.equal(t2, s2)
    assert t1.stride() == s1.stride() and t1.stride(-2) == 1
    fp8 = torch.from_numpy(g['in_fp8']).view(torch.float8_e4m3fn)
    sfx = torch.zeros((256, 1), dtype=torch.int32)
    (c1, _), _ = transform_weights_for_gc_moe((fp8, sfx), (fp8, sfx))
    assert np.array_equal(c1.view(torch.uint8).numpy(), g['out_fp8'])


def test_scale_byte_rule_is_ceil_log2():
    """The integer-bit rule (gc_moe/common/math.py:146-154) equals
    2^ceil(log2(amax/448)) floored at 2^-22, the formula of the reference's
    torch oracle (tests/test_sm120_gc_moe.py:204)."""
    g = torch.Generator().manual_seed(1)
    amax = torch.rand(200000, generator=g) * torch.exp2(torch.randint(-40, 12, (200000,), generator=g).float())
    edge = torch.tensor([0.0, 448.0, 448.0 * 2, 447.99, 448.01, 1.75, 1.7500001, 2.0 ** -22 * 448, 1e-30])
    amax = torch.cat((amax, edge))
    assert torch.equal(O.ue8m0_fp8_scale_byte(amax), O.ue8m0_ceil_exponent(amax / 448.0, floor_exp=-22))


def test_quantisers_round_trip():
    g = torch.Generator().manual_seed(2)
    x = torch.randn((7, 256), generator=g)
    q, sf = O.quantize_act_fp8(x)
    deq = O.dequant_fp8(q, O.sf_bytes(sf))
    assert (deq - x).abs().max() <= x.abs().max() * 2 ** -3
    assert q.float().abs().max() <= 448
    w = torch.randn((2, 16, 128), generator=g) * 0.02
    p, codes = O.quantize_weight_fp4(w)
    wd = O.dequant_fp4(p, codes)
    assert (wd - w).abs().max() <= w.abs().max() * 0.26
    # every e2m1 code survives a round trip exactly
    vals = torch.tensor([s * m for s in (1, -1) for m in O.FP4_VALUES]).repeat(2)[None, None, :]
    p2, c2 = O.quantize_weight_fp4(vals)
    assert torch.equal(O.dequant_fp4(p2, c2), vals)


def test_dispatch_products_are_consistent():
    p, e, k, h = 2, 8, 3, 256
    idx, wts, xb, xs = [], [], [], []
    for s, t in enumerate((5, 0)):
        xq, xsf, i, w = O.make_tokens(t, h, e, k, seed=20 + s)
        if t:
            i[1, 0] = -1
            i[2, 1] = e + 3
        idx.append(i.numpy()); wts.append(w.numpy()); xb.append(xq.view(torch.uint8).numpy()); xs.append(xsf.numpy())
    d = O.dispatch(idx, wts, xb, xs, e, [16, 16])
    total = sum(int(dr.counts.sum()) for dr in d)
    assert total == 5 * k - 2
    for r, dr in enumerate(d):
        assert dr.pool_blocks == sum(-(-int(n) // 16) for n in dr.counts.sum(0))
        rows = np.nonzero(dr.metadata[:, 0] >= 0)[0]
        assert len(rows) == int(dr.counts.sum())
        for row in rows:
            s, t, j = dr.metadata[row]
            assert idx[s][t, j] // (e // p) == r
            assert np.array_equal(dr.rows[row], xb[s][t]) and dr.weights[row] == wts[s][t, j]
        # inside an expert: source ranks ascending, token*k+slot ascending
        for l in range(e // p):
            r0 = int(dr.expert_block_start[l]) * 16
            n = int(dr.counts[:, l].sum())
            keys = [(m[0], m[1] * k + m[2]) for m in dr.metadata[r0:r0 + n]]
            assert keys == sorted(keys)
    assert O.sf_ring_position(16 + 5, 16, 100) == 128 + 20


def test_combine_order_and_invalid_slots():
    big = 2.0 ** 24          # big + 1 is not representable in fp32
    slots = torch.tensor([[[big, 5.0]], [[1.0, 1.0]], [[-big, 3.0]]], dtype=torch.bfloat16)  # [3, 1, 2]
    every = torch.tensor([[True, True, True]])
    # order 0, 1, 2: (big + 1) rounds back to big, minus big -> 0
    assert O.combine(slots, every, shared_last=False)[0, 0].item() == 0.0
    # last slot first (the shared-expert position): (-big + big) + 1 -> 1
    assert O.combine(slots, every, shared_last=True)[0, 0].item() == 1.0
    skipped = O.combine(slots, torch.tensor([[True, False, True]]), shared_last=False)
    assert skipped[0, 1].item() == 8.0
    none = O.combine(slots, torch.tensor([[False, False, False]]), shared_last=False)
    assert torch.equal(none, torch.zeros_like(none))


def test_package_quantisers_equal_the_oracle_quantisers():
    from gc_moe_b200 import quant
    g = torch.Generator().manual_seed(4)
    w = torch.randn((2, 32, 256), generator=g) * 0.02
    a, b = O.quantize_weight_fp4(w)
    c, d = quant.quantize_weights_fp4(w)
    assert torch.equal(a, c) and torch.equal(b, d)
    x = torch.randn((5, 256), generator=g)
    a, b = O.quantize_act_fp8(x)
    c, d = quant.quantize_activations(x)
    assert torch.equal(a.view(torch.uint8), c.view(torch.uint8)) and torch.equal(b, d)
    assert torch.equal(O.pack_weight_sf_mn_major(d.view(torch.uint8).reshape(1, 5, -1)),
                       quant.weight_scales_mn_major(d.view(torch.uint8).reshape(1, 5, -1)))


def test_route_topk_orders_by_value_then_expert_id():
    logits = torch.tensor([[0.5, 2.0, 2.0, -1.0, 2.0, 0.5], [0.0] * 6])
    idx, w = O.route_topk(logits, 4)
    assert idx.tolist() == [[1, 2, 4, 0], [0, 1, 2, 3]]
    assert torch.allclose(w.sum(-1), torch.ones(2))
    assert torch.allclose(w[1], torch.full((4,), 0.25))
    g = torch.Generator().manual_seed(5)
    logits = torch.randn((50, 64), generator=g)
    idx, w = O.route_topk(logits, 8)
    top, ref_idx = torch.topk(logits, 8, dim=-1)          # distinct values: same selection
    assert torch.equal(idx, ref_idx)
    assert torch.allclose(w, torch.softmax(top, -1))


def test_stage_shared_sf_rows_follow_the_block_order():
    from gc_moe_b200.layout import sf_row_in_block
    x_sf = torch.arange(300 * 8, dtype=torch.int32).reshape(300, 8)
    for bm in (16, 96, 192):
        rows_total = -(-300 // bm) * (-(-bm // 128) * 128)
        staged, where = O.stage_shared_sf(x_sf, bm, rows_total)
        assert len(set(where.tolist())) == 300
        for t in (0, 1, 31, 32, 95, 96, 127, 128, 191, 192, 299):
            row = (t // bm) * (-(-bm // 128) * 128) + sf_row_in_block(t % bm)
            assert int(where[t]) == row
            assert torch.equal(staged[row], x_sf[t])


def test_integer_scale_rule_of_the_producer_kernel_equals_the_oracle_rule_for_every_bf16():
    """The CUDA producer computes the UE8M0 code of amax/448 from the float's bits
    (exponent, plus one when the mantissa exceeds 1.75, minus 8, floored at 0).
    Exhaustive over all finite non-negative BF16 values."""
    import numpy as np
    hi = np.arange(0, 0x7F80, dtype=np.uint32)                 # all finite non-negative BF16 bit patterns
    bits = hi << 16
    amax = torch.from_numpy(bits.view(np.float32).copy())
    up = (bits + 0x7FFFFF - 0x600000) >> 23
    rule = np.maximum(up, 8) - 8
    want = O.ue8m0_ceil_exponent(amax / O.E4M3_MAX).numpy()
    assert np.array_equal(rule.astype(np.uint8), want)


def test_package_weight_front_end_matches_the_oracle():
    """The product-side helpers that bring checkpoint-style tensors into the
    operator's input form produce the oracle's bytes."""
    from gc_moe_b200 import quant
    g = torch.Generator().manual_seed(21)
    w = torch.randn((256, 512), generator=g) * 0.02
    q, codes = quant.quantize_weights_fp8_blocks(w)
    oq, ocodes = O.quantize_block_fp8(w)
    assert torch.equal(q.view(torch.uint8), oq.view(torch.uint8)) and torch.equal(codes, ocodes)
    a, b = quant.expand_block_scales(codes, 256), O.expand_block_sf_rows(ocodes, 256)
    assert torch.equal(a, b) and a.stride() == b.stride() and a.stride(0) == 1
    w4 = torch.randn((3, 64, 256), generator=g) * 0.02
    p, c = quant.quantize_weights_fp4(w4)
    op, oc = O.quantize_weight_fp4(w4)
    assert torch.equal(p, op) and torch.equal(c, oc)
    s, os_ = quant.weight_scales_mn_major(c), O.pack_weight_sf_mn_major(oc)
    assert torch.equal(s, os_) and s.stride() == os_.stride()
    x = (torch.randn((9, 512), generator=g)).to(torch.bfloat16)
    xq, xsf = quant.quantize_activations(x)
    oxq, oxsf = O.quantize_act_fp8(x)
    assert torch.equal(xq.view(torch.uint8), oxq.view(torch.uint8)) and torch.equal(xsf, oxsf)


@pytest.mark.parametrize('ranks', [4, 12])
def test_push_plan_agrees_with_the_pool_order_also_above_eight_ranks(ranks):
    """Every source's own computation of its routes' pool rows lands exactly on the
    rows the world-level dispatch assigns: concatenated sources up to 8 ranks,
    interleaved sources (round j = j-th route of every source that has one) above."""
    import numpy as np
    experts, k, h = 2 * ranks, 3, 256
    g = torch.Generator().manual_seed(ranks)
    tokens = [int(torch.randint(0, 40, (1,), generator=g)) for _ in range(ranks)]
    tokens[1] = 0                                              # an idle rank
    idx = [torch.stack([torch.randperm(experts, generator=g)[:k] for _ in range(t)]) if t else
           torch.zeros((0, k), dtype=torch.int64) for t in tokens]
    idx[0][0, 0] = -1                                          # an invalid route
    xb = [torch.randint(0, 255, (t, h), generator=g, dtype=torch.uint8).numpy() for t in tokens]
    xsf = [torch.randint(0, 1 << 20, (t, h // 128), generator=g, dtype=torch.int32).numpy() for t in tokens]
    w = [torch.rand((t, k), generator=g).numpy() for t in tokens]
    bms = [16 if r % 2 else 32 for r in range(ranks)]
    world = O.dispatch([i.numpy() for i in idx], w, xb, xsf, experts, bms)
    counts = np.zeros((ranks, experts), np.int64)
    for s in range(ranks):
        flat = idx[s].reshape(-1)
        for e in flat[(flat >= 0) & (flat < experts)].tolist():
            counts[s, e] += 1
    covered = [set() for _ in range(ranks)]
    for s in range(ranks):
        for owner, l, row, i, t, slot in O.push_plan(s, idx[s].numpy(), counts, bms, experts):
            assert tuple(world[owner].metadata[row]) == (s, t, slot)
            assert world[owner].index_lists[(l, s)][i] == t * k + slot
            assert row not in covered[owner]
            covered[owner].add(row)
    for r in range(ranks):
        assert covered[r] == set(np.nonzero(world[r].metadata[:, 0] >= 0)[0].tolist())
    if ranks > 8:
        # interleaving: inside an expert with several sources the first rows alternate sources
        d = world[0]
        srcs = d.metadata[:, 0]
        assert any(srcs[i] >= 0 and srcs[i + 1] >= 0 and srcs[i + 1] < srcs[i] for i in range(len(srcs) - 1))
