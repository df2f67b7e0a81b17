"""Host-side geometry against fixtures generated from the reference's own
Python (tests/golden/make_golden.py): arena offsets, block-M, ring sizing."""
import json
import os

import pytest

from gc_moe_b200.heuristics import (full_pool_ring_tokens, get_block_m_for_gc_moe,
                                    get_ring_tokens)
from gc_moe_b200.layout import GCBufferLayout, SIGNAL_OFFSETS, sf_row_in_block

GOLDEN = os.path.join(os.path.dirname(__file__), 'golden', 'host_geometry.json')


@pytest.fixture(scope='module')
def golden():
    with open(GOLDEN) as f:
        return json.load(f)


def test_signal_offsets_exact(golden):
    assert SIGNAL_OFFSETS == golden['signal_offsets']


def test_layout_offsets_exact(golden):
    for case in golden['layouts']:
        lay = GCBufferLayout(*case['args'])
        assert lay.nbytes == case['nbytes']
        assert lay.num_max_pool_tokens == case['num_max_pool_tokens']
        assert lay.workspace_offsets == case['workspace']
        assert set(lay.views) == set(case['views'])
        for name, (offset, nbytes, shape, dtype, stride) in case['views'].items():
            v = lay.views[name]
            assert (v.offset, v.nbytes, list(v.shape), v.dtype,
                    list(v.stride) if v.stride else None) == (offset, nbytes, shape, dtype, stride), name


def test_block_m_exact(golden):
    for case in golden['block_m']:
        p, e, cap, k = case['args']
        got = [get_block_m_for_gc_moe(p, e, cap, t, k) for t in case['tokens']]
        assert got == case['block_m'], case['args']


def test_ring_tokens_exact(golden):
    for case in golden['ring']:
        assert list(get_ring_tokens(*case['args'])) == case['ring']


def test_block_m_rejects_bad_queries():
    for args in [(0, 8, 16, 1, 2), (2, 9, 16, 1, 2), (1, 8, 16, 17, 2), (1, 8, 16, -1, 2),
                 (1, 8, 16, 1, 0), (1, 8, 16, 1, 33)]:
        with pytest.raises(ValueError):
            get_block_m_for_gc_moe(*args)
    with pytest.raises(ValueError):
        get_block_m_for_gc_moe(1, 8, 16, 1, 2, mma_type='int8')


def test_layout_rejects_bad_geometry():
    ring, sf = full_pool_ring_tokens(1, 8, 1920, 2)
    good = dict(num_ranks=1, num_experts=8, capacity=1920, topk=2, hidden=1024, intermediate=512,
                ring_tokens=ring, sf_ring_tokens=sf)
    GCBufferLayout(**good)
    for bad in (dict(num_ranks=0), dict(num_experts=9, num_ranks=2), dict(topk=0), dict(topk=33),
                dict(hidden=1000), dict(intermediate=100), dict(ring_tokens=ring + 1),
                dict(sf_ring_tokens=4), dict(num_experts=4096)):
        with pytest.raises(ValueError):
            GCBufferLayout(**{**good, **bad})


def test_full_pool_ring_holds_every_pool():
    for p, e, cap, k in [(1, 64, 1920, 8), (8, 256, 1920, 8), (8, 256, 5760, 8), (1, 8, 1920, 2)]:
        ring, sf = full_pool_ring_tokens(p, e, cap, k)
        local = e // p
        for bm in (16, 32, 64, 96, 128, 192, 240):
            assert ring >= p * cap * min(k, local) + local * (bm - 1)
            assert sf >= ring // bm * ((bm + 127) // 128 * 128)
        assert ring % 1920 == 0 and sf % 4 == 0


def test_sf_row_in_block_is_a_permutation_of_each_128():
    for base in (0, 128):
        rows = sorted(sf_row_in_block(base + u) for u in range(128))
        assert rows == list(range(base, base + 128))
    assert sf_row_in_block(33) == 1 * 4 + 1 and sf_row_in_block(5) == 20
