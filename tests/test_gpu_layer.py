"""GPU parity: the CUDA layer, called through the operator API (and so through
the C ABI), against the CPU oracle on the same seeded inputs.

Integer products (counts, pool layout, index table, metadata, dispatched rows
and scales) must be bit-exact.  BF16 outputs: cosine >= 0.9999 and a maximum
error, relative to the largest output magnitude, of at most 2^-6 (two BF16
ulps of the largest value) -- in practice the outputs are bit-identical except
where a differently ordered FP32 accumulation flips one BF16/FP8 rounding.
"""
import numpy as np
import pytest
import torch

import gc_moe_b200 as G
from oracle import gcmoe_oracle as O

from _cases import LayerCase, check_dispatch_products, check_requantised_intermediate, sf_rows_of_pool

pytestmark = pytest.mark.gpu

COSINE_MIN = 0.9999
MAX_REL_ERR = 2.0 ** -6


def assert_close(y, ref):
    assert torch.isfinite(y.float()).all()
    assert O.cosine(y, ref) >= COSINE_MIN
    assert O.max_rel_err(y, ref) <= MAX_REL_ERR


@pytest.fixture(scope='module')
def small(single_rank_group):
    case = LayerCase(single_rank_group, num_experts=8, hidden=1024, inter=512, topk=2, seed=0)
    yield case
    case.close()


@pytest.fixture(scope='module')
def config1(single_rank_group):
    """Single-GPU benchmark geometry: hidden 4096, 64 experts, top-8, intermediate 2048."""
    case = LayerCase(single_rank_group, num_experts=64, hidden=4096, inter=2048, topk=8, seed=1)
    yield case
    case.close()


def parity(case):
    return int(case.buf.region('recv_parity').view(torch.int32)[0].item())


def test_config0_bit_exact_products_and_output(small):
    xq, xsf, idx, w = O.make_tokens(16, small.h, small.e, small.k, seed=1)
    gen = parity(small) & 1
    stats = torch.zeros(small.e, dtype=torch.int32, device='cuda')
    y = small.run(xq, xsf, idx, w, fast_math=False, stats=stats, guard=2)
    ref = small.oracle(xq, xsf, idx, w)
    bm = small.block_m(16)
    prod = small.products(16, gen)
    check_dispatch_products(prod, ref.dispatch[0], bm)
    assert np.array_equal(stats.cpu().numpy(), ref.stats[0])
    check_requantised_intermediate(prod, ref, bm, 'config 0')
    assert_close(y, ref.y[0])
    # nothing outside y[:T] is written
    guard = small.full_y.cpu()
    assert torch.isnan(guard[:2].float()).all() and torch.isnan(guard[-2:].float()).all()


@pytest.mark.parametrize('tokens', [1, 8, 32, 128, 256])
def test_config1_token_sweep(config1, tokens):
    xq, xsf, idx, w = O.make_tokens(tokens, config1.h, config1.e, config1.k, seed=100 + tokens)
    gen = parity(config1) & 1
    y = config1.run(xq, xsf, idx, w)
    ref = config1.oracle(xq, xsf, idx, w)
    prod = config1.products(tokens, gen)
    check_dispatch_products(prod, ref.dispatch[0], config1.block_m(tokens))
    check_requantised_intermediate(prod, ref, config1.block_m(tokens), f'config 1 T={tokens}')
    assert_close(y, ref.y[0])


@pytest.mark.parametrize('tokens', [0, 3, 79, 81, 193, 450])
def test_block_m_boundaries_and_ragged_counts(small, tokens):
    """Token counts on both sides of the block-M switches (16 -> 32 -> 64 ...)
    with ragged per-expert counts, and the empty call."""
    xq, xsf, idx, w = O.make_tokens(tokens, small.h, small.e, small.k, seed=7 + tokens)
    gen = parity(small) & 1
    y = small.run(xq, xsf, idx, w)
    ref = small.oracle(xq, xsf, idx, w)
    check_dispatch_products(small.products(tokens, gen), ref.dispatch[0], small.block_m(tokens))
    assert y.shape == (tokens, small.h)
    if tokens:
        assert_close(y, ref.y[0])


def test_invalid_routes_are_skipped(small):
    xq, xsf, idx, w = O.make_tokens(40, small.h, small.e, small.k, seed=3)
    idx[::3, 0] = -1                 # "no route"
    idx[1::5, 1] = small.e + 5       # out of range
    idx[7] = -1                      # a token without any valid route
    gen = parity(small) & 1
    y = small.run(xq, xsf, idx, w)
    ref = small.oracle(xq, xsf, idx, w)
    check_dispatch_products(small.products(40, gen), ref.dispatch[0], small.block_m(40))
    assert_close(y, ref.y[0])
    assert torch.equal(y[7], torch.zeros_like(y[7]))


def test_all_routes_invalid_gives_zeros(small):
    xq, xsf, idx, w = O.make_tokens(12, small.h, small.e, small.k, seed=4)
    idx[:] = -1
    y = small.run(xq, xsf, idx, w)
    assert torch.equal(y, torch.zeros_like(y))


def test_hot_expert_spans_many_blocks(small):
    """All routes to two experts: several M-blocks per expert, the others empty."""
    tokens = 300
    xq, xsf, idx, w = O.make_tokens(tokens, small.h, small.e, small.k, seed=5)
    idx[:, 0], idx[:, 1] = 2, 5
    gen = parity(small) & 1
    y = small.run(xq, xsf, idx, w)
    ref = small.oracle(xq, xsf, idx, w)
    check_dispatch_products(small.products(tokens, gen), ref.dispatch[0], small.block_m(tokens))
    assert_close(y, ref.y[0])


def test_zero_route_weights_give_exact_zeros(small):
    xq, xsf, idx, w = O.make_tokens(9, small.h, small.e, small.k, seed=6)
    y = small.run(xq, xsf, idx, torch.zeros_like(w))
    assert torch.equal(y, torch.zeros_like(y))


def test_repeat_is_bitwise_identical_and_stats_accumulate(small):
    xq, xsf, idx, w = O.make_tokens(33, small.h, small.e, small.k, seed=8)
    stats = torch.zeros(small.e, dtype=torch.int32, device='cuda')
    y1 = small.run(xq, xsf, idx, w, stats=stats)
    y2 = small.run(xq, xsf, idx, w, stats=stats)
    assert torch.equal(y1.view(torch.int16), y2.view(torch.int16))
    expect = np.bincount(idx.numpy().reshape(-1), minlength=small.e)
    assert np.array_equal(stats.cpu().numpy(), 2 * expect)


def test_no_clamp_and_exact_math_paths(small):
    xq, xsf, idx, w = O.make_tokens(20, small.h, small.e, small.k, seed=9)
    for clamp, fast in ((None, True), (None, False), (0.5, False)):
        y = small.run(xq, xsf, idx, w, clamp=clamp, fast_math=fast)
        assert_close(y, small.oracle(xq, xsf, idx, w, clamp=clamp).y[0])


def test_graph_replay_alternating_inputs(small):
    """Readiness protocol of the reference (tests/test_gc_moe_readiness.py):
    capture once, then replay with inputs A and B alternating at fixed
    addresses; every replay must reproduce its own eager result."""
    tokens = 24
    a = O.make_tokens(tokens, small.h, small.e, small.k, seed=10)
    b = O.make_tokens(tokens, small.h, small.e, small.k, seed=11)
    y = torch.empty((tokens, small.h), dtype=torch.bfloat16, device='cuda')
    eager = []
    for inp in (a, b):
        eager.append(small.run(*inp, y=y).clone())
    assert not torch.equal(eager[0], eager[1])
    import gc_moe_b200 as G
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        G.fp8_fp4_gc_moe(y, small.l1, small.l2, small.buf, activation_clamp=10.0)   # warm
        with torch.cuda.graph(graph, stream=side):
            G.fp8_fp4_gc_moe(y, small.l1, small.l2, small.buf, activation_clamp=10.0)
    torch.cuda.current_stream().wait_stream(side)
    for it in range(20):
        small.stage(*(a, b)[it & 1])
        y.fill_(float('nan'))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y.cpu().view(torch.int16), eager[it & 1].view(torch.int16)), it
    small.buf.raise_on_device_error()


def test_contract_violations_raise_like_the_reference(small):
    import gc_moe_b200 as G
    y = torch.empty((4, small.h), dtype=torch.bfloat16, device='cuda')
    with pytest.raises(ValueError):       # misaligned output
        odd = torch.empty(4 * small.h + 1, dtype=torch.bfloat16, device='cuda')[1:].view(4, small.h)
        G.fp8_fp4_gc_moe(odd, small.l1, small.l2, small.buf)
    with pytest.raises(ValueError):       # untransformed weights
        G.fp8_fp4_gc_moe(y, (small.q1.to('cuda'), small.l1[1]), small.l2, small.buf)
    with pytest.raises(ValueError):       # wrong dtype
        G.fp8_fp4_gc_moe(y.float(), small.l1, small.l2, small.buf)
    with pytest.raises(ValueError):       # stats of the wrong length
        G.fp8_fp4_gc_moe(y, small.l1, small.l2, small.buf,
                         cumulative_local_expert_recv_stats=torch.zeros(3, dtype=torch.int32, device='cuda'))
    with pytest.raises(ValueError):
        G.fp8_fp4_gc_moe(torch.empty((4000, small.h), dtype=torch.bfloat16, device='cuda'), small.l1, small.l2, small.buf)


@pytest.mark.parametrize('tokens,hot', [(40, False), (300, False), (900, True)])
def test_raw_accumulators_of_both_tile_regimes(small, tokens, hot):
    """The FP32 accumulators of the gate/up GEMM, read straight from TMEM, against
    an FP32 matmul of the dequantised operands: a sharper check of the MMA,
    descriptor and scale plumbing than y.  40 tokens run one CTA per tile
    (cta_group::1, the only launch enqueued); for 300 evenly routed tokens both
    regimes' launches are enqueued and the dispatch kernel chooses one CTA per tile
    again (no expert reaches 128 rows); with 900 tokens all routed to two experts
    it chooses CTA pairs (cta_group::2) and an expert spans several 240-token tiles."""
    import ctypes
    from gc_moe_b200 import _native, operator
    from gc_moe_b200.contract import validate_call
    xq, xsf, idx, w = O.make_tokens(tokens, small.h, small.e, small.k, seed=300 + tokens)
    if hot:
        idx[:, 0], idx[:, 1] = 1, 6
    y = torch.empty((tokens, small.h), dtype=torch.bfloat16, device='cuda')
    small.run(xq, xsf, idx, w, y=y)
    ref = small.oracle(xq, xsf, idx, w)
    d = ref.dispatch[0]
    rows = d.metadata.shape[0]
    out = torch.full((rows, 2 * small.i), float('nan'), dtype=torch.float32, device='cuda')
    cfg = validate_call(y, small.l1, small.l2, small.buf, None, None, None, (1, 1, 32), 'swiglu', 10.0, True,
                        None, None)
    assert (cfg.block_m >= 64) == (tokens >= 300)
    plan = operator.get_plan(cfg, y, small.l1, small.l2, small.buf, None, None, None)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _native.raise_for(_native.library().gcmoe_debug_gemm_l1_raw(plan.handle, out.data_ptr(), stream))
    torch.cuda.synchronize()
    small.buf.raise_on_device_error()
    got = out.cpu()
    for l in range(small.e):
        n = int(d.counts[:, l].sum())
        if n == 0:
            continue
        r0 = int(d.expert_block_start[l]) * d.block_m
        xd = O.dequant_fp8(torch.from_numpy(d.rows[r0:r0 + n]).view(torch.float8_e4m3fn),
                           torch.from_numpy(d.sf_words[r0:r0 + n]).view(torch.uint8))
        wd = O.interleave_gate_up(O.dequant_fp4(small.q1[l], small.c1[l]))
        want = xd @ wd.T
        err = (got[r0:r0 + n] - want).abs().max().item()
        assert err <= 1e-4 * want.abs().max().item(), (l, n, err)


@pytest.fixture(scope='module')
def large(single_rank_group):
    """Geometry for the large-token regime: capacity 5760 tokens, 16 experts."""
    case = LayerCase(single_rank_group, num_experts=16, hidden=1024, inter=512, topk=4,
                     capacity=5760, seed=2)
    yield case
    case.close()


@pytest.mark.parametrize('tokens,expect_bm', [(300, 96), (400, 128), (700, 192), (1600, 240), (4096, 240)])
def test_large_token_regime_with_skewed_routing(large, tokens, expect_bm):
    """Block-M 96..240 (TMEM holds one accumulator stage from 128 up) with the
    benchmark's heavy skew: about 10 % of the experts (2 of 16) receive half of
    the assignments, so hot experts span many blocks and cold ones are ragged."""
    assert large.block_m(tokens) == expect_bm
    g = torch.Generator().manual_seed(40 + tokens)
    x = torch.randn((tokens, large.h), generator=g).to(torch.bfloat16)
    weights = torch.full((large.e,), 0.5 / (large.e - 2))
    weights[[3, 11]] = 0.25
    gumbel = -torch.log(-torch.log(torch.rand((tokens, large.e), generator=g)))
    top, idx = torch.topk(torch.log(weights) + gumbel, large.k, dim=-1, sorted=False)
    w = torch.softmax(top, dim=-1)
    xq, xsf = O.quantize_act_fp8(x)
    gen = parity(large) & 1
    y = large.run(xq, xsf, idx.to(torch.int64), w.float())
    ref = large.oracle(xq, xsf, idx.to(torch.int64), w.float())
    check_dispatch_products(large.products(tokens, gen), ref.dispatch[0], expect_bm)
    assert_close(y, ref.y[0])


def _stage_shared_sf(case, xsf, tokens, bm):
    """Caller-side staging of the shared expert's input scales: row of token t is
    (t // BM) * align(BM, 128) + (u // 128) * 128 + (u % 32) * 4 + (u % 128) // 32, u = t % BM
    (gc_moe/gc/__init__.py:19-23)."""
    view = case.buf.shared_l1_acts_sf
    t = torch.arange(tokens)
    u = t % bm
    rows = (t // bm) * ((bm + 127) // 128 * 128) + (u // 128) * 128 + (u % 32) * 4 + (u % 128) // 32
    view[rows.to('cuda')] = xsf.to('cuda')


@pytest.mark.parametrize('tokens', [1, 16, 64, 200, 1500])
def test_fused_shared_expert_k128(single_rank_group, tokens):
    """Routed experts plus one fused shared expert (two experts' worth of
    intermediate) whose FP8 weights carry one UE8M0 scale per 128 x 128 block,
    expanded to one packed row per output row before the transform.  1500
    tokens give block-M 240: with a shared expert such blocks stay whole GEMM
    tiles (one accumulator stage), a path no other case reaches."""
    import gc_moe_b200 as G
    e, h, i, k, s = 8, 1024, 512, 2, 2
    case = LayerCase(single_rank_group, e, h, i, k, seed=6, num_shared_experts=s)
    try:
        g = torch.Generator().manual_seed(77)
        sw1, sc1 = O.quantize_block_fp8(torch.randn((2 * s * i, h), generator=g) * 0.02)
        sw2, sc2 = O.quantize_block_fp8(torch.randn((h, s * i), generator=g) * 0.02)
        shared = {'w1': sw1, 'w1_codes': sc1, 'w2': sw2, 'w2_codes': sc2}
        sl1, sl2 = G.transform_weights_for_gc_moe(
            (sw1.cuda(), O.expand_block_sf_rows(sc1, 2 * s * i).cuda()),
            (sw2.cuda(), O.expand_block_sf_rows(sc2, h).cuda()))
        xq, xsf, idx, w = O.make_tokens(tokens, h, e, k, seed=60 + tokens)
        bm = case.block_m(tokens)
        case.stage(xq, xsf, idx, w)
        _stage_shared_sf(case, xsf, tokens, bm)
        y = torch.full((tokens, h), float('nan'), dtype=torch.bfloat16, device='cuda')
        G.fp8_fp4_gc_moe(y, case.l1, case.l2, case.buf, sl1, sl2, activation_clamp=10.0,
                         shared_recipe=(1, 128, 128))
        torch.cuda.synchronize()
        case.buf.raise_on_device_error()
        ref = O.moe_layer([xq], [xsf], [idx], [w], case.q1, case.c1, case.q2, case.c2, [bm], clamp=10.0,
                          shared=shared)
        assert_close(y.cpu(), ref.y[0])
        # the shared branch alone: routes all invalid -> y is the shared expert's output
        idx[:] = -1
        case.stage(xq, xsf, idx, w)
        G.fp8_fp4_gc_moe(y, case.l1, case.l2, case.buf, sl1, sl2, activation_clamp=10.0,
                         shared_recipe=(1, 128, 128))
        torch.cuda.synchronize()
        only = O.shared_expert(xq, xsf, shared, 10.0)
        assert_close(y.cpu(), only)
    finally:
        case.close()


def test_fused_shared_expert_k32(single_rank_group):
    """Shared expert whose FP8 weights carry per-row K32 scales (shared recipe (1, 1, 32))."""
    import gc_moe_b200 as G
    e, h, i, k, s, tokens = 8, 1024, 512, 2, 1, 40
    case = LayerCase(single_rank_group, e, h, i, k, seed=7, num_shared_experts=s)
    try:
        g = torch.Generator().manual_seed(78)
        sw1, sf1 = O.quantize_act_fp8(torch.randn((2 * s * i, h), generator=g) * 0.02)
        sw2, sf2 = O.quantize_act_fp8(torch.randn((h, s * i), generator=g) * 0.02)
        shared = {'w1': sw1, 'w1_codes': O.sf_bytes(sf1), 'w2': sw2, 'w2_codes': O.sf_bytes(sf2), 'gran': 32}
        mn = lambda t: t.t().contiguous().t()
        sl1, sl2 = G.transform_weights_for_gc_moe((sw1.cuda(), mn(sf1).cuda()), (sw2.cuda(), mn(sf2).cuda()))
        xq, xsf, idx, w = O.make_tokens(tokens, h, e, k, seed=90)
        bm = case.block_m(tokens)
        case.stage(xq, xsf, idx, w)
        _stage_shared_sf(case, xsf, tokens, bm)
        y = torch.full((tokens, h), float('nan'), dtype=torch.bfloat16, device='cuda')
        G.fp8_fp4_gc_moe(y, case.l1, case.l2, case.buf, sl1, sl2, activation_clamp=10.0)
        torch.cuda.synchronize()
        case.buf.raise_on_device_error()
        ref = O.moe_layer([xq], [xsf], [idx], [w], case.q1, case.c1, case.q2, case.c2, [bm], clamp=10.0,
                          shared=shared)
        assert_close(y.cpu(), ref.y[0])
    finally:
        case.close()


def test_expired_wait_is_reported_and_later_calls_return_at_once(single_rank_group):
    """Failure detection without a failure: a wait on a word nothing sets runs
    out after 200 us, the status block says where, the host raises, and every
    later kernel on the workspace returns immediately instead of waiting again."""
    import ctypes
    import gc_moe_b200 as G
    from gc_moe_b200 import _native, operator
    from gc_moe_b200.contract import validate_call
    case = LayerCase(single_rank_group, num_experts=8, hidden=1024, inter=512, topk=2, seed=9)
    try:
        inputs = O.make_tokens(6, case.h, case.e, case.k, seed=70)
        good = case.run(*inputs)
        assert torch.isfinite(good.float()).all()
        y = torch.full((6, case.h), float('nan'), dtype=torch.bfloat16, device='cuda')
        cfg = validate_call(y, case.l1, case.l2, case.buf, None, None, None, (1, 1, 32), 'swiglu', 10.0, True,
                            None, None)
        plan = operator.get_plan(cfg, y, case.l1, case.l2, case.buf, None, None, None)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _native.raise_for(_native.library().gcmoe_debug_expire_wait(plan.handle, 200, stream))
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match='device wait gave up'):
            case.buf.raise_on_device_error()
        G.fp8_fp4_gc_moe(y, case.l1, case.l2, case.buf, activation_clamp=10.0)   # returns at once, writes nothing
        torch.cuda.synchronize()
        assert torch.isnan(y.float()).all()
    finally:
        case.close()


def test_second_wrapper_over_the_same_allocation(small, single_rank_group):
    """``GCSymmBuffer(..., base=owner)`` wraps the owner's bytes without allocating
    (gc_moe/gc/__init__.py:38,73-93): calls through either wrapper, one after the other,
    give the oracle's output and keep alternating the call parity they share; a wrapper of
    another geometry, of a foreign object or of a destroyed owner is rejected."""
    owner = small.buf
    args = (single_rank_group, small.e, small.capacity, small.k, small.h, small.i)
    twin = G.GCSymmBuffer(*args, base=owner)
    try:
        assert twin.buffer.data_ptr() == owner.buffer.data_ptr() and twin.peer_addresses == owner.peer_addresses
        assert twin.layout == owner.layout and twin.x.data_ptr() == owner.x.data_ptr()
        for step, buf in enumerate((twin, owner, twin, twin, owner)):
            xq, xsf, idx, w = O.make_tokens(12 + step, small.h, small.e, small.k, seed=900 + step)
            before = parity(small)
            small.buf = buf
            try:
                y = small.run(xq, xsf, idx, w)
            finally:
                small.buf = owner
            assert parity(small) == before + 1
            assert_close(y, small.oracle(xq, xsf, idx, w).y[0])
        with pytest.raises(ValueError, match='incompatible base'):
            G.GCSymmBuffer(single_rank_group, small.e, small.capacity, small.k, small.h, 2 * small.i, base=owner)
        with pytest.raises(ValueError, match='base must be'):
            G.GCSymmBuffer(*args, base=owner.buffer)
        dead = G.GCSymmBuffer(*args)
        dead.destroy()
        with pytest.raises(ValueError, match='live allocation'):
            G.GCSymmBuffer(*args, base=dead)
    finally:
        twin.destroy()
    assert owner.buffer is not None      # destroying a wrapper leaves the allocation to its owner
    xq, xsf, idx, w = O.make_tokens(5, small.h, small.e, small.k, seed=950)
    assert_close(small.run(xq, xsf, idx, w), small.oracle(xq, xsf, idx, w).y[0])
