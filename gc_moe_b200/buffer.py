"""The symmetric workspace object of the operator API.

Same constructor arguments (``base=`` included), attributes and views as the
reference's ``GCSymmBuffer`` (gc_moe/gc/__init__.py:16-163).  Two deliberate differences:
the activation rings hold the whole receive pool (no slot reuse inside a
call, see ``heuristics.full_pool_ring_tokens``), and device-side failures are
reported through ``raise_on_device_error`` instead of trapping the GPU.
"""

from __future__ import annotations

import types

import torch
import torch.distributed as dist

from .heuristics import full_pool_ring_tokens
from .layout import GCBufferLayout, TOKEN_ALIGNMENT, round_up

_VIEW_NAMES = ('x', 'x_sf', 'topk_idx', 'topk_weights', 'shared_l1_acts',
               'shared_l1_acts_sf', 'shared_l2_acts', 'shared_l2_acts_sf',
               'l1_acts', 'l1_acts_sf', 'l2_acts', 'l2_acts_sf')


def _typed_views(buffer: torch.Tensor, layout: GCBufferLayout, target) -> None:
    for name in _VIEW_NAMES:
        spec = layout.views[name]
        if spec.nbytes == 0:
            view = None
        elif name == 'shared_l1_acts':
            view = target.x
        else:
            dtype = getattr(torch, spec.dtype)
            raw = buffer.narrow(0, spec.offset, spec.nbytes).view(dtype)
            view = raw.as_strided(spec.shape, spec.stride) if spec.stride else raw.view(spec.shape)
        setattr(target, name, view)


class GCSymmBuffer:
    """Workspace shared by the ranks of one expert-parallel group.

    The caller stages ``x[:T]``, ``x_sf[:T]``, ``topk_idx[:T]`` and
    ``topk_weights[:T]`` before each call.  Callers of the fused shared expert
    also stage ``shared_l1_acts_sf`` at row
    ``(t // BM) * align(BM, 128) + (u // 128) * 128 + (u % 32) * 4 + (u % 128) // 32``
    with ``u = t % BM`` and BM from ``get_block_m_for_gc_moe``.  Calls that
    share one workspace must be serialised by the caller, and graphs captured
    on it retired before ``destroy()``.

    ``base`` makes this object a second wrapper over the allocation of a live
    ``GCSymmBuffer`` of the same group and exactly the same geometry instead of
    allocating (gc_moe/gc/__init__.py:38,73-93): no rendezvous, no zeroing, the
    protocol state in the arena (call parity, counters) is shared, launch plans
    are per wrapper.  Calls through all wrappers of one allocation must be
    serialised; destroying a wrapper leaves the allocation to its owner.
    """

    _views = _VIEW_NAMES

    def __init__(self, group, num_experts: int, num_max_tokens_per_rank: int,
                 num_topk: int, hidden: int, intermediate_hidden: int,
                 num_shared_experts: int = 0, mma_type: str = 'fp8xfp4',
                 activation: str = 'swiglu', base=None):
        if mma_type != 'fp8xfp4' or activation != 'swiglu':
            raise ValueError('GC MoE requires fp8xfp4/swiglu')
        if base is not None and not isinstance(base, GCSymmBuffer):
            raise ValueError('base must be a GCSymmBuffer of this package; foreign workspaces are unsupported')
        self.group = group
        self.rank_idx = dist.get_rank(group=group)
        world = group.size()
        self.num_experts = num_experts
        self.num_max_tokens_per_rank = round_up(num_max_tokens_per_rank, TOKEN_ALIGNMENT)
        self.num_topk = num_topk
        self.hidden, self.intermediate_hidden = hidden, intermediate_hidden
        self.num_shared_experts = num_shared_experts
        self.mma_type, self.activation = mma_type, activation
        ring, sf_ring = full_pool_ring_tokens(world, num_experts,
                                              self.num_max_tokens_per_rank, num_topk)
        self.layout = GCBufferLayout(world, num_experts, self.num_max_tokens_per_rank,
                                     num_topk, hidden, intermediate_hidden, ring, sf_ring,
                                     num_shared_experts)
        if base is None:
            if world == 1:
                self.buffer = torch.empty(self.layout.nbytes, dtype=torch.int8, device='cuda')
                self.handle = types.SimpleNamespace(buffer_ptrs=[self.buffer.data_ptr()])
            else:
                import torch.distributed._symmetric_memory as symm_mem
                self.buffer = symm_mem.empty(self.layout.nbytes, dtype=torch.int8, device='cuda')
                self.handle = symm_mem.rendezvous(self.buffer, group=group)
        else:
            if base.buffer is None or base.handle is None or base.group is not group:
                raise ValueError('base must be a live allocation in the same group')
            for name in ('num_experts', 'num_max_tokens_per_rank', 'num_topk', 'hidden',
                         'intermediate_hidden', 'num_shared_experts', 'mma_type', 'activation'):
                if getattr(base, name) != getattr(self, name):
                    raise ValueError(f'incompatible base: {name}')
            if self.layout != base.layout:
                raise ValueError('incompatible base: GC workspace layout')
            if self.layout.nbytes > base.buffer.nbytes:
                raise ValueError('base allocation too small')
            self.buffer, self.handle = base.buffer, base.handle
        peers = tuple(int(ptr) for ptr in self.handle.buffer_ptrs)
        if (len(peers) != world or any(ptr <= 0 or ptr % 16 for ptr in peers)
                or peers[self.rank_idx] != self.buffer.data_ptr()):
            raise RuntimeError('symmetric rendezvous returned invalid peer addresses')
        self.peer_addresses = peers
        if base is None:
            self.buffer.zero_()
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier(group=group)
        _typed_views(self.buffer, self.layout, self)
        self._plans = {}          # launch plans cached per call signature
        self._retired_scratch = []   # scratch blocks of evicted plans, until their status has been read

    def _for_call(self, num_shared_experts: int):
        """View of the same bytes laid out for the shared-expert count of one
        call (gc_moe/gc/__init__.py:109-123)."""
        if self.buffer is None or self.handle is None:
            raise ValueError('symmetric buffer has been destroyed')
        if num_shared_experts == self.num_shared_experts:
            return self
        layout = GCBufferLayout(self.group.size(), self.num_experts,
                                self.num_max_tokens_per_rank, self.num_topk, self.hidden,
                                self.intermediate_hidden, self.layout.ring_tokens,
                                self.layout.sf_ring_tokens, num_shared_experts)
        if layout.nbytes > self.buffer.nbytes:
            raise ValueError("symmetric buffer is too small for call's shared experts")
        return _CallView(self, layout)

    def region(self, name: str) -> torch.Tensor:
        """Raw bytes of a named arena region (signals, workspace or view), for
        inspection by tests and tools."""
        from .layout import SIGNAL_OFFSETS
        if name in self.layout.views:
            spec = self.layout.views[name]
            return self.buffer.narrow(0, spec.offset, spec.nbytes)
        offsets = self.layout.workspace_offsets
        if name == 'src_token_topk_idx':
            return self.buffer.narrow(0, offsets[name], offsets['token_src_metadata'] - offsets[name])
        if name == 'token_src_metadata':
            return self.buffer.narrow(0, offsets[name], self.layout.num_max_pool_tokens * 12)
        order = sorted((off, key) for key, off in SIGNAL_OFFSETS.items())
        for (off, key), (end, _) in zip(order, order[1:] + [(SIGNAL_OFFSETS['size'], '')]):
            if key == name:
                return self.buffer.narrow(0, off, end - off)
        raise KeyError(name)

    def raise_on_device_error(self) -> None:
        """Synchronise and raise RuntimeError if a kernel of any call on this
        workspace gave up on a bounded wait."""
        from . import operator
        for plan in list(self._plans.values()):
            operator.check_plan_status(plan)
        retired, self._retired_scratch = self._retired_scratch, []
        for scratch in retired:       # the status reads above have synchronised the stream
            operator.check_retired_status(scratch)

    def destroy(self):
        from . import operator
        for plan in self._plans.values():
            operator.release_plan(plan)
        self._plans = {}
        self._retired_scratch = []
        for name in self._views:
            setattr(self, name, None)
        self.peer_addresses = self.handle = self.buffer = self.group = None


class _CallView:
    """Per-call re-slicing of a workspace for a different shared-expert count."""

    def __init__(self, base: GCSymmBuffer, layout: GCBufferLayout):
        self._base = base
        self.layout = layout
        self.num_shared_experts = layout.num_shared_experts
        _typed_views(base.buffer, layout, self)

    def __getattr__(self, name):
        return getattr(self._base, name)


def get_symm_buffer_for_gc_moe(group, num_experts: int, num_max_tokens_per_rank: int,
                               num_topk: int, hidden: int, intermediate_hidden: int,
                               num_shared_experts: int = 0, mma_type: str = 'fp8xfp4',
                               activation: str = 'swiglu') -> GCSymmBuffer:
    """Allocate a workspace (gc_moe/gc/__init__.py:155-163; like the reference's factory it
    does not take ``base`` -- construct ``GCSymmBuffer(..., base=owner)`` for a second wrapper)."""
    return GCSymmBuffer(group, num_experts, num_max_tokens_per_rank, num_topk, hidden,
                        intermediate_hidden, num_shared_experts, mma_type, activation)
