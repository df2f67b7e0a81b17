"""Upstream producer for ``fp8_fp4_gc_moe``: fills the workspace's input views
from BF16 activations and router logits in one kernel.

The reference leaves input staging to the caller -- four ``copy_`` calls, a
quantiser from a package it does not vendor, and for the fused shared expert
an ``index_put`` of the scale rows (README.md:234-252, 363-377;
tests/test_gc_moe.py:368-372) -- and notes that the staging "can be fused into
an upstream producer" (README.md:387).  ``stage_inputs_for_gc_moe`` is that
producer; it has no counterpart function in the reference.
"""

from __future__ import annotations

import ctypes

import torch

from . import _native
from .heuristics import get_block_m_for_gc_moe


def stage_inputs_for_gc_moe(sym_buffer, x: torch.Tensor, router_logits: torch.Tensor | None = None,
                            topk_idx: torch.Tensor | None = None,
                            topk_weights: torch.Tensor | None = None) -> int:
    """Write ``x[:T]``, ``x_sf[:T]``, ``topk_idx[:T]``, ``topk_weights[:T]`` (and
    the rows of ``shared_l1_acts_sf`` when the workspace has a shared expert)
    of ``sym_buffer`` from BF16 ``x`` [T, H] and either ``router_logits``
    [T, E] (top-k by value, ties to the lower expert id, softmax over the
    selected k) or ready ``topk_idx`` int64 / ``topk_weights`` f32 [T, k].

    Runs on the current stream, allocates nothing and can be captured together
    with the layer call.  Returns the call's block-M.
    """
    if x.dim() != 2 or x.dtype != torch.bfloat16 or not x.is_cuda or not x.is_contiguous():
        raise ValueError('x must be a contiguous 2-D CUDA bfloat16 tensor')
    tokens, hidden = x.shape
    topk = sym_buffer.topk_idx.shape[1]
    if hidden != sym_buffer.x.shape[1]:
        raise ValueError(f'x has hidden {hidden}, the workspace {sym_buffer.x.shape[1]}')
    if tokens > sym_buffer.num_max_tokens_per_rank:
        raise ValueError(f'{tokens} tokens exceed the workspace capacity {sym_buffer.num_max_tokens_per_rank}')
    args = _native.StageArgs()
    num_experts = sym_buffer.num_experts
    if router_logits is not None:
        if topk_idx is not None or topk_weights is not None:
            raise ValueError('give router_logits or topk_idx/topk_weights, not both')
        if (router_logits.shape != (tokens, num_experts) or router_logits.dtype != torch.float32
                or not router_logits.is_cuda or not router_logits.is_contiguous()):
            raise ValueError(f'router_logits must be contiguous CUDA float32 [{tokens}, {num_experts}]')
        args.router_logits = router_logits.data_ptr()
    else:
        if topk_idx is None or topk_weights is None:
            raise ValueError('give router_logits or both topk_idx and topk_weights')
        if (topk_idx.shape != (tokens, topk) or topk_idx.dtype != torch.int64 or not topk_idx.is_cuda
                or not topk_idx.is_contiguous()):
            raise ValueError(f'topk_idx must be contiguous CUDA int64 [{tokens}, {topk}]')
        if (topk_weights.shape != (tokens, topk) or topk_weights.dtype != torch.float32
                or not topk_weights.is_cuda or not topk_weights.is_contiguous()):
            raise ValueError(f'topk_weights must be contiguous CUDA float32 [{tokens}, {topk}]')
        args.topk_idx_in, args.topk_weights_in = topk_idx.data_ptr(), topk_weights.data_ptr()
    block_m = get_block_m_for_gc_moe(sym_buffer.group.size(), num_experts,
                                     sym_buffer.num_max_tokens_per_rank, tokens, topk)
    args.x = x.data_ptr()
    args.x_q, args.x_sf = sym_buffer.x.data_ptr(), sym_buffer.x_sf.data_ptr()
    args.topk_idx, args.topk_weights = sym_buffer.topk_idx.data_ptr(), sym_buffer.topk_weights.data_ptr()
    shared_sf = getattr(sym_buffer, 'shared_l1_acts_sf', None)
    if shared_sf is not None:
        args.shared_sf, args.shared_sf_rows = shared_sf.data_ptr(), shared_sf.shape[0]
    args.block_m, args.num_tokens, args.hidden = block_m, tokens, hidden
    args.num_experts, args.topk = num_experts, topk
    stream = torch.cuda.current_stream().cuda_stream
    _native.raise_for(_native.library().gcmoe_stage_inputs(ctypes.byref(args), ctypes.c_void_p(stream)))
    return block_m
