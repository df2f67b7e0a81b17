"""``fp8_fp4_gc_moe``: the layer call, and the launch shim below it.

Above the seam the flow is the reference's (gc_moe/apis/gc_moe.py:140-161):
validate, re-slice the workspace for the call, launch.  Below it the
reference JIT-compiles three role kernels and replays a three-node graph on
green contexts; here ``_launch`` looks up (or creates) a native plan and
enqueues the layer's kernels on the current stream through the C ABI.
"""

from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Tuple

import torch

from . import _native
from .contract import ValidatedCall, validate_call
from .layout import SIGNAL_OFFSETS

_PLAN_CACHE_LIMIT = 64


class _Plan:
    """A native plan plus everything whose lifetime it depends on.

    ``pinned`` is set once the plan has been created or launched while its
    stream was being captured: a CUDA graph then holds the addresses of the
    plan's scratch block in its kernel parameters, so the plan (and with it the
    scratch) must stay alive for as long as the workspace does.
    """

    def __init__(self, handle, scratch, keepalive):
        self.handle = handle
        self.scratch = scratch
        self.keepalive = keepalive
        self.pinned = False


def _timeout_ms() -> int:
    """Limit of every device-side wait.  GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS is
    honoured with the reference's strict integer parsing
    (gc_moe/jit_kernels/impls/sm100_fp8_fp4_gc_moe.py:166-180); the default is
    2 s instead of the reference's hour because a shared GPU must not spin."""
    import re
    name = 'GC_MOE_NVLINK_BARRIER_TIMEOUT_SECS'
    value = os.getenv(name)
    if value is None or value == '':
        return 2000
    if re.fullmatch(r'[ \t\n\v\f\r]*[+-]?[0-9]+', value, re.ASCII) is None:
        raise ValueError(f'Invalid {name}: {value}')
    seconds = int(value, 10)
    if not 0 < seconds <= 2_147_483_647:
        raise ValueError(f'Invalid {name}: {value}')
    return min(seconds * 1000, 2_000_000_000)


def _dispatch_sms() -> int:
    """Upper bound of the SMs the dispatch kernel occupies (0 = the library's default
    of 32).  GC_MOE_DISPATCH_SMS is parsed as the reference parses it: a signed decimal
    int32 without whitespace (gc_moe/runtime/gc_moe.py:29-49); a request outside
    [2, SM count) is refused like the reference's SM split refuses it
    (gc_moe/runtime/gc_moe.py:92-93)."""
    import re
    name = 'GC_MOE_DISPATCH_SMS'
    raw = os.environ.get(name)
    if raw is None:
        return 0
    if re.fullmatch(r'-?[0-9]+', raw) is None:
        raise ValueError(f'invalid value for {name}: {raw}')
    value = int(raw)
    if not -(1 << 31) <= value < (1 << 31):
        raise ValueError(f'invalid value for {name}: {raw}')
    total = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    if not 2 <= value < total:
        raise ValueError('invalid dispatch SM request')
    return value


def _build_plan(config: ValidatedCall, y, l1_weights, l2_weights, call_buffer,
                shared_l1, shared_l2, stats) -> _Plan:
    lib = _native.library()
    layout = call_buffer.layout
    views, work = layout.views, layout.workspace_offsets
    prob = _native.Problem(
        num_ranks=layout.num_ranks, rank=call_buffer.rank_idx, num_experts=layout.num_experts,
        capacity=layout.capacity, topk=layout.topk, hidden=layout.hidden,
        intermediate=layout.intermediate, num_tokens=config.tokens, block_m=config.block_m,
        ring_tokens=layout.ring_tokens, sf_ring_tokens=layout.sf_ring_tokens,
        num_shared_experts=config.shared_experts, shared_gran_k=config.shared_weight_gran_k,
        has_clamp=int(math.isfinite(config.clamp)),
        clamp=config.clamp if math.isfinite(config.clamp) else 0.0,
        fast_math=int(config.fast_math), timeout_ms=_timeout_ms(), num_sms=0,
        dispatch_sms=_dispatch_sms())
    scratch = torch.zeros(lib.gcmoe_scratch_bytes(ctypes.byref(prob)), dtype=torch.uint8,
                          device=y.device)
    buf = _native.Buffers()
    for rank, address in enumerate(call_buffer.peer_addresses):
        buf.arena_base[rank] = address
    buf.off_recv_parity = SIGNAL_OFFSETS['recv_parity']
    buf.off_routed_pool_blocks = SIGNAL_OFFSETS['routed_pool_blocks']
    buf.off_recv_count = SIGNAL_OFFSETS['expert_recv_count']
    buf.off_recv_count_sum = SIGNAL_OFFSETS['expert_recv_count_sum']
    buf.off_index_table = work['src_token_topk_idx']
    buf.off_metadata = work['token_src_metadata']
    for field, view in (('off_x', 'x'), ('off_x_sf', 'x_sf'), ('off_topk_idx', 'topk_idx'),
                        ('off_topk_weights', 'topk_weights'), ('off_l1_acts', 'l1_acts'),
                        ('off_l1_acts_sf', 'l1_acts_sf'),
                        ('off_l1_topk_weights', 'l1_topk_weights'), ('off_l2_acts', 'l2_acts'),
                        ('off_l2_acts_sf', 'l2_acts_sf'), ('off_combine_tokens', 'combine_tokens'),
                        ('off_shared_l1_acts_sf', 'shared_l1_acts_sf'),
                        ('off_shared_l2_acts', 'shared_l2_acts'),
                        ('off_shared_l2_acts_sf', 'shared_l2_acts_sf')):
        setattr(buf, field, views[view].offset)
    buf.shared_sf_rows = views['shared_l1_acts_sf'].shape[0]
    buf.y = y.data_ptr()
    buf.stats = stats.data_ptr() if stats is not None else 0
    buf.w1, buf.w1_sf = l1_weights[0].data_ptr(), l1_weights[1].data_ptr()
    buf.w2, buf.w2_sf = l2_weights[0].data_ptr(), l2_weights[1].data_ptr()
    buf.w1_sf_stride, buf.w2_sf_stride = l1_weights[1].stride(-1), l2_weights[1].stride(-1)
    if shared_l1 is not None:
        buf.sw1, buf.sw1_sf = shared_l1[0].data_ptr(), shared_l1[1].data_ptr()
        buf.sw2, buf.sw2_sf = shared_l2[0].data_ptr(), shared_l2[1].data_ptr()
        buf.sw1_sf_stride, buf.sw2_sf_stride = shared_l1[1].stride(-1), shared_l2[1].stride(-1)
    buf.scratch, buf.scratch_bytes = scratch.data_ptr(), scratch.numel()
    buf.off_exchange = SIGNAL_OFFSETS['l2_full_mask']
    handle = ctypes.c_void_p()
    _native.raise_for(lib.gcmoe_plan_create(ctypes.byref(prob), ctypes.byref(buf),
                                            ctypes.byref(handle)))
    keepalive = (y, l1_weights, l2_weights, shared_l1, shared_l2, stats, call_buffer.buffer)
    return _Plan(handle, scratch, keepalive)


def _plan_key(config: ValidatedCall, y, l1_weights, l2_weights, shared_l1, shared_l2, stats):
    tensors = [y, *l1_weights, *l2_weights, *(shared_l1 or ()), *(shared_l2 or ())]
    return (config, tuple(t.data_ptr() for t in tensors),
            stats.data_ptr() if stats is not None else 0, _timeout_ms(),
            os.environ.get('GC_MOE_DISPATCH_SMS'))


def _capturing() -> bool:
    return torch.cuda.is_current_stream_capturing()


def get_plan(config, y, l1_weights, l2_weights, call_buffer, shared_l1, shared_l2, stats) -> _Plan:
    """Plan for this exact call signature, cached on the workspace.  Cached
    plans keep their tensors alive, as the reference's launch cache does for
    graphs that captured them (jit_kernels/impls/sm100_fp8_fp4_gc_moe.py:206-209:
    "Entries remain alive; no cache clear may release in-flight graph
    resources").  Only plans no graph can refer to are ever evicted: the oldest
    one that was never used under stream capture, and only outside capture."""
    owner = getattr(call_buffer, '_base', call_buffer)
    key = _plan_key(config, y, l1_weights, l2_weights, shared_l1, shared_l2, stats)
    capturing = _capturing()
    plan = owner._plans.get(key)
    if plan is None:
        if len(owner._plans) >= _PLAN_CACHE_LIMIT and not capturing:
            victim = next((k for k, cached in owner._plans.items() if not cached.pinned), None)
            if victim is not None:
                retire_plan(owner, owner._plans.pop(victim))
        plan = _build_plan(config, y, l1_weights, l2_weights, call_buffer, shared_l1,
                           shared_l2, stats)
        owner._plans[key] = plan
    if capturing:
        plan.pinned = True
    return plan


def retire_plan(owner, plan: _Plan) -> None:
    """Drop an evicted plan.  Its kernels may still be running and its status
    block may hold a failure nobody has read yet: the scratch block is parked on
    the workspace until the next ``raise_on_device_error`` has looked at it."""
    owner._retired_scratch.append(plan.scratch)
    del owner._retired_scratch[:-256]       # bounded: beyond that the oldest blocks go back to the allocator
    release_plan(plan)


def release_plan(plan: _Plan) -> None:
    if plan.handle:
        _native.library().gcmoe_plan_destroy(plan.handle)
        plan.handle = None


def check_plan_status(plan: _Plan) -> None:
    words = (ctypes.c_uint32 * _native.STATUS_WORDS)()
    stream = torch.cuda.current_stream().cuda_stream
    _native.raise_for(_native.library().gcmoe_status_read(plan.handle, ctypes.c_void_p(stream), words))


def check_retired_status(scratch: torch.Tensor) -> None:
    """Status words of a plan that has been evicted (the block starts with them)."""
    words = scratch[:_native.STATUS_WORDS * 4].view(torch.int32).tolist()
    if words[0] != 0:
        raise RuntimeError(f'device wait gave up: code {words[0]} kernel {words[1]} site {words[2]} '
                           f'block {words[3]} observed {words[4]} expected {words[5]}')


def _launch(config, y, l1_weights, l2_weights, call_buffer, shared_l1, shared_l2, stats) -> None:
    """Replacement of launch_gc_moe
    (gc_moe/jit_kernels/impls/sm100_fp8_fp4_gc_moe.py:721-727)."""
    plan = get_plan(config, y, l1_weights, l2_weights, call_buffer, shared_l1, shared_l2, stats)
    stream = torch.cuda.current_stream().cuda_stream
    _native.raise_for(_native.library().gcmoe_launch(plan.handle, ctypes.c_void_p(stream)))


def fp8_fp4_gc_moe(y: torch.Tensor,
                   l1_weights: Tuple[torch.Tensor, torch.Tensor],
                   l2_weights: Tuple[torch.Tensor, torch.Tensor],
                   sym_buffer,
                   shared_l1_weights: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                   shared_l2_weights: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                   cumulative_local_expert_recv_stats: Optional[torch.Tensor] = None,
                   recipe: Tuple[int, int, int] = (1, 1, 32),
                   activation: str = 'swiglu', activation_clamp: Optional[float] = None,
                   fast_math: bool = True,
                   shared_recipe: Optional[Tuple[int, int, int]] = None,
                   activation_alpha: Optional[float] = None) -> None:
    """One MoE layer call: y[:T] = combine(experts(dispatch(x, topk))) in BF16.

    Signature and semantics of gc_moe.fp8_fp4_gc_moe
    (gc_moe/gc/__init__.py:226-243): T = y.shape[0]; inputs are read from
    ``sym_buffer``; all ranks of the group call collectively; the work is
    enqueued on the current CUDA stream and may be captured into a CUDA graph.
    """
    if hasattr(sym_buffer, 'num_shared_experts'):
        assert (sym_buffer.num_shared_experts > 0) == (shared_l1_weights is not None)
    config = validate_call(y, l1_weights, l2_weights, sym_buffer, shared_l1_weights,
                           shared_l2_weights, cumulative_local_expert_recv_stats, recipe,
                           activation, activation_clamp, fast_math, shared_recipe,
                           activation_alpha)
    call_buffer = sym_buffer._for_call(config.shared_experts)
    _launch(config, y, l1_weights, l2_weights, call_buffer, shared_l1_weights,
            shared_l2_weights, cumulative_local_expert_recv_stats)
