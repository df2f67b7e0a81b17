"""The layer entry point for callers that cannot allocate device memory.

Some hosts of the operator run with a frozen device heap (a serving loop whose
pool was sized at start-up, code running where cudaMalloc would synchronise or
is forbidden), so they cannot hand the library a scratch block.
gcmoe_launch_static_scratch keeps the kernels' scratch in a fixed device array
inside the library.  This test calls it through the C ABI, twice in a row on
different inputs (the array keeps the previous call's contents), and requires
the same bytes in y as the plan-based entry point produces; it also checks the
size limit is enforced.  It is collected last so that a failure here cannot
hide any other test.
"""
import ctypes

import pytest
import torch

from gc_moe_b200 import _native
from gc_moe_b200.contract import validate_call
from gc_moe_b200.layout import SIGNAL_OFFSETS
from oracle import gcmoe_oracle as O

from _cases import LayerCase

pytestmark = pytest.mark.gpu


def describe_call(case, y, clamp, fast_math):
    """gcmoe_problem / gcmoe_buffers of one call, filled from the workspace
    layout the way the operator shim fills them -- minus the scratch block."""
    cfg = validate_call(y, case.l1, case.l2, case.buf, None, None, None, (1, 1, 32), 'swiglu',
                        clamp, fast_math, None, None)
    lay = case.buf.layout
    prob = _native.Problem(
        num_ranks=1, rank=0, num_experts=lay.num_experts, capacity=lay.capacity, topk=lay.topk,
        hidden=lay.hidden, intermediate=lay.intermediate, num_tokens=cfg.tokens,
        block_m=cfg.block_m, ring_tokens=lay.ring_tokens, sf_ring_tokens=lay.sf_ring_tokens,
        num_shared_experts=0, shared_gran_k=32, has_clamp=1, clamp=clamp,
        fast_math=int(fast_math), timeout_ms=2000, num_sms=0)
    buf = _native.Buffers()
    buf.arena_base[0] = case.buf.peer_addresses[0]
    buf.off_recv_parity = SIGNAL_OFFSETS['recv_parity']
    buf.off_routed_pool_blocks = SIGNAL_OFFSETS['routed_pool_blocks']
    buf.off_recv_count = SIGNAL_OFFSETS['expert_recv_count']
    buf.off_recv_count_sum = SIGNAL_OFFSETS['expert_recv_count_sum']
    buf.off_index_table = lay.workspace_offsets['src_token_topk_idx']
    buf.off_metadata = lay.workspace_offsets['token_src_metadata']
    for field, view in (('off_x', 'x'), ('off_x_sf', 'x_sf'), ('off_topk_idx', 'topk_idx'),
                        ('off_topk_weights', 'topk_weights'), ('off_l1_acts', 'l1_acts'),
                        ('off_l1_acts_sf', 'l1_acts_sf'), ('off_l1_topk_weights', 'l1_topk_weights'),
                        ('off_l2_acts', 'l2_acts'), ('off_l2_acts_sf', 'l2_acts_sf'),
                        ('off_combine_tokens', 'combine_tokens')):
        setattr(buf, field, lay.views[view].offset)
    buf.off_exchange = SIGNAL_OFFSETS['l2_full_mask']
    buf.y = y.data_ptr()
    buf.w1, buf.w1_sf = case.l1[0].data_ptr(), case.l1[1].data_ptr()
    buf.w2, buf.w2_sf = case.l2[0].data_ptr(), case.l2[1].data_ptr()
    buf.w1_sf_stride, buf.w2_sf_stride = case.l1[1].stride(-1), case.l2[1].stride(-1)
    return prob, buf          # buf.scratch stays 0: the entry point supplies its own


def test_static_scratch_entry_matches_plan_entry(single_rank_group):
    lib = _native.library()
    case = LayerCase(single_rank_group, num_experts=8, hidden=1024, inter=512, topk=2, seed=21)
    try:
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        words = (ctypes.c_uint32 * _native.STATUS_WORDS)()
        for call, (tokens, seed) in enumerate(((40, 31), (7, 32))):
            inputs = O.make_tokens(tokens, case.h, case.e, case.k, seed=seed)
            expected = case.run(*inputs, clamp=10.0, fast_math=True)        # existing entry point
            y = torch.full((tokens, case.h), float('nan'), dtype=torch.bfloat16, device='cuda')
            case.stage(*inputs)
            prob, buf = describe_call(case, y, 10.0, True)
            _native.raise_for(lib.gcmoe_launch_static_scratch(ctypes.byref(prob), ctypes.byref(buf), stream))
            _native.raise_for(lib.gcmoe_static_scratch_status(stream, words))
            # same kernels, same inputs: the outputs are bit-identical
            assert torch.equal(y.cpu().view(torch.int16), expected.view(torch.int16)), call
            ref = case.oracle(*inputs)
            assert O.cosine(y.cpu(), ref.y[0]) >= 0.9999
    finally:
        case.close()


def test_static_scratch_keeps_an_earlier_failure_visible(single_rank_group):
    """A wait that gave up leaves the workspace failed: its kernels return at once.
    A later static-scratch call clears the status words, runs nothing and leaves y
    alone -- the status query must still say so, not report success."""
    import gc_moe_b200 as G
    from gc_moe_b200 import operator
    lib = _native.library()
    case = LayerCase(single_rank_group, num_experts=8, hidden=1024, inter=512, topk=2, seed=22)
    try:
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        words = (ctypes.c_uint32 * _native.STATUS_WORDS)()
        inputs = O.make_tokens(5, case.h, case.e, case.k, seed=33)
        case.run(*inputs)                                        # a plan to hang the expiring wait on
        y = torch.full((5, case.h), float('nan'), dtype=torch.bfloat16, device='cuda')
        cfg = validate_call(y, case.l1, case.l2, case.buf, None, None, None, (1, 1, 32), 'swiglu', 10.0, True,
                            None, None)
        plan = operator.get_plan(cfg, y, case.l1, case.l2, case.buf, None, None, None)
        _native.raise_for(lib.gcmoe_debug_expire_wait(plan.handle, 200, stream))
        torch.cuda.synchronize()
        case.stage(*inputs)
        prob, buf = describe_call(case, y, 10.0, True)
        _native.raise_for(lib.gcmoe_launch_static_scratch(ctypes.byref(prob), ctypes.byref(buf), stream))
        rc = lib.gcmoe_static_scratch_status(stream, words)
        assert rc == _native.ERR_DEVICE, _native.last_error()
        assert torch.isnan(y.float()).all()
        case.buf._plans.clear()        # the failed plan's status would raise at close otherwise
    finally:
        case.close()


def test_static_scratch_rejects_more_experts_than_it_holds():
    lib = _native.library()
    prob = _native.Problem(num_ranks=1, rank=0, num_experts=256, capacity=1920, topk=8, hidden=1024,
                           intermediate=512, num_tokens=4, block_m=16, ring_tokens=1920 * 40,
                           sf_ring_tokens=1920 * 40 * 8)
    rc = lib.gcmoe_launch_static_scratch(ctypes.byref(prob), ctypes.byref(_native.Buffers()), None)
    assert rc == _native.ERR_UNSUPPORTED
    assert '128' in _native.last_error()
    with pytest.raises(NotImplementedError):
        _native.raise_for(rc)
