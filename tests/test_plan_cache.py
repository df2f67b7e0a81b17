"""Lifetime of cached launch plans: a plan that a CUDA graph may refer to is
never evicted (the graph's kernel parameters hold the plan's scratch addresses
by value), only plans used in eager mode are.  Host logic only: the native
plan is replaced by a stand-in, so no GPU is needed."""
import types

import pytest

from gc_moe_b200 import operator


class FakeScratch:
    freed = 0

    def __del__(self):
        FakeScratch.freed += 1


@pytest.fixture
def cache(monkeypatch):
    state = types.SimpleNamespace(capturing=False, built=0, released=[])

    def build(config, *args):
        state.built += 1
        return operator._Plan(handle=object(), scratch=FakeScratch(), keepalive=())

    def release(plan):
        state.released.append(plan)
        plan.handle = None

    monkeypatch.setattr(operator, '_build_plan', build)
    monkeypatch.setattr(operator, 'release_plan', release)
    monkeypatch.setattr(operator, '_capturing', lambda: state.capturing)
    monkeypatch.setattr(operator, '_plan_key', lambda config, *a: config)
    state.owner = types.SimpleNamespace(_plans={}, _retired_scratch=[])
    state.get = lambda key: operator.get_plan(key, None, None, None, state.owner, None, None, None)
    return state


def test_captured_plans_survive_any_number_of_new_signatures(cache):
    cache.capturing = True
    captured = [cache.get(('graph', i)) for i in range(3)]
    cache.capturing = False
    assert all(p.pinned for p in captured)
    for i in range(operator._PLAN_CACHE_LIMIT + 5):      # 65+ distinct eager signatures
        cache.get(('eager', i))
    assert all(p.handle is not None for p in captured)
    assert not any(p in cache.released for p in captured)
    assert all(cache.owner._plans[('graph', i)] is captured[i] for i in range(3))
    # the eager ones did get evicted, oldest first, and their scratch is parked, not freed
    assert len(cache.released) >= 5
    assert cache.released[0] is not captured[0]
    assert len(cache.owner._retired_scratch) == len(cache.released)
    assert len(cache.owner._plans) <= operator._PLAN_CACHE_LIMIT


def test_plan_first_used_eagerly_then_captured_becomes_pinned(cache):
    plan = cache.get('a')
    assert not plan.pinned
    cache.capturing = True
    assert cache.get('a') is plan and plan.pinned
    cache.capturing = False
    for i in range(2 * operator._PLAN_CACHE_LIMIT):
        cache.get(('eager', i))
    assert plan.handle is not None and cache.owner._plans['a'] is plan


def test_nothing_is_evicted_while_capturing_and_cache_may_grow(cache):
    cache.capturing = True
    for i in range(operator._PLAN_CACHE_LIMIT + 10):
        cache.get(i)
    assert cache.released == [] and len(cache.owner._plans) == operator._PLAN_CACHE_LIMIT + 10
    cache.capturing = False
    cache.get('eager')            # every cached plan is pinned: nothing can go
    assert cache.released == []
