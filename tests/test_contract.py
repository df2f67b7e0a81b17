"""Argument checks of fp8_fp4_gc_moe that do not need a GPU: same conditions
and exception types as the reference's validate_call
(gc_moe/apis/gc_moe.py:69-137)."""
import types

import pytest
import torch

from gc_moe_b200.contract import _activation_scalars, validate_call
from gc_moe_b200.operator import _timeout_ms


def _fake_buffer(destroyed=False):
    return types.SimpleNamespace(buffer=None if destroyed else object(), handle=object(),
                                 hidden=1024, intermediate_hidden=512, num_experts=8,
                                 num_max_tokens_per_rank=1920, num_topk=2,
                                 group=types.SimpleNamespace(size=lambda: 1))


def _call(**over):
    t = torch.zeros(1)
    args = dict(y=torch.zeros((4, 1024), dtype=torch.bfloat16), l1_weights=(t, t), l2_weights=(t, t),
                sym_buffer=_fake_buffer(), shared_l1_weights=None, shared_l2_weights=None,
                cumulative_local_expert_recv_stats=None, recipe=(1, 1, 32), activation='swiglu',
                activation_clamp=None, fast_math=True, shared_recipe=None, activation_alpha=None)
    args.update(over)
    return validate_call(**args)


def test_rejections_in_reference_order():
    t = torch.zeros(1)
    with pytest.raises(ValueError, match='pairs'):
        _call(l1_weights=(t,))
    with pytest.raises(ValueError, match='destroyed'):
        _call(sym_buffer=_fake_buffer(destroyed=True))
    with pytest.raises(ValueError, match='recipe'):
        _call(recipe=(1, 1, 128))
    with pytest.raises(ValueError, match='recipe'):
        _call(activation='gelu')
    with pytest.raises(ValueError, match='shared recipe'):
        _call(shared_recipe=(1, 1, 64))
    with pytest.raises(ValueError, match='clamp'):
        _call(activation_clamp=-1.0)
    with pytest.raises(ValueError, match='alpha'):
        _call(activation_alpha=0.0)
    with pytest.raises(ValueError, match='together'):
        _call(shared_l1_weights=(t, t))
    with pytest.raises(ValueError, match='y must be'):
        _call()                      # a CPU tensor is not a valid output


def test_activation_scalars_round_to_float32():
    clamp, alpha = _activation_scalars(0.1, None)
    assert clamp == torch.tensor(0.1, dtype=torch.float32).item() and alpha == 1.0
    assert _activation_scalars(None, 2)[0] == float('inf')


def test_timeout_env_parsing(monkeypatch):
    monkeypatch.delenv('GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS', raising=False)
    assert _timeout_ms() == 2000
    monkeypatch.setenv('GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS', ' +3')
    assert _timeout_ms() == 3000
    for bad in ('0', '-1', '1.5', 'abc', '3s'):
        monkeypatch.setenv('GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS', bad)
        with pytest.raises(ValueError):
            _timeout_ms()


def test_foreign_base_and_other_recipes_are_rejected_before_anything_is_allocated():
    """gc_moe/gc/__init__.py:41-44: the recipe check, then the type of ``base``."""
    from gc_moe_b200 import GCSymmBuffer
    with pytest.raises(ValueError, match='fp8xfp4/swiglu'):
        GCSymmBuffer(None, 8, 16, 2, 1024, 512, mma_type='fp8xfp8')
    with pytest.raises(ValueError, match='foreign workspaces are unsupported'):
        GCSymmBuffer(None, 8, 16, 2, 1024, 512, base=types.SimpleNamespace(buffer=None))
