"""Weight re-layout for the kernels: ``transform_weights_for_gc_moe``.

Produces byte-for-byte the tensors the reference transform produces
(gc_moe/gc/__init__.py:166-223, gc_moe/jit_kernels/impls/runtime_utils.py:
86-118), because the kernels of this package consume exactly that layout:

* gate/up rows interleaved in groups of 16 (8 gate rows, then the 8 up rows
  of the same channels), so the two halves of a SwiGLU pair sit 8 TMEM lanes
  apart in one accumulator tile;
* payload tiled so that each (K128 block, 128 rows) weight tile is one
  contiguous 8 KiB (FP4) or 16 KiB (FP8) range -- a single TMA box;
* scale rows permuted, inside every 128 rows, to position
  ``(u % 32) * 4 + u // 32``: the order in which ``tcgen05.cp`` lays 128 scale
  words across 32 TMEM lanes x 4 columns.


On the GPU the re-layout is two kernels of the native library
(``gcmoe_transform_weights``); tensors on the CPU (host-side tests against the
reference's golden bytes) take the torch formulation of the same permutation.
As an extension, the scale tensor of a 2-D FP8 weight may be the raw
128 x 128 block codes (uint8 ``[rows / 128, K / 128]``): the kernel expands them
to one packed row per output row on the fly, which the reference asks the
caller to do beforehand (README.md:347-351).
"""

from __future__ import annotations

import ctypes

import torch


def _interleave_gate_up(t: torch.Tensor) -> torch.Tensor:
    if t.ndim not in (2, 3) or t.shape[-2] % 16:
        raise ValueError('W1 rows must be a multiple of 16')
    batched = t if t.ndim == 3 else t.unsqueeze(0)
    groups, rows = batched.shape[:2]
    tail = batched.shape[2:]
    halves = batched.reshape(groups, 2, rows // 16, 8, *tail)     # [gate|up][channel group][8]
    out = torch.empty_like(batched)
    out.copy_(halves.transpose(1, 2).reshape(batched.shape))
    return out if t.ndim == 3 else out.squeeze(0)


def _sf_rows_to_4x32(sf: torch.Tensor) -> torch.Tensor:
    if sf.dtype != torch.int32 or sf.ndim not in (2, 3) or sf.shape[-2] % 128:
        raise ValueError('SF must be packed int32 with 128-aligned rows')
    batched = sf if sf.ndim == 3 else sf.unsqueeze(0)
    groups, rows, packs = batched.shape
    out = torch.empty_like(batched)              # keeps the MN-major strides of the input
    out.copy_(batched.reshape(groups, rows // 128, 4, 32, packs).transpose(2, 3)
              .reshape(batched.shape))
    return out if sf.ndim == 3 else out.squeeze(0)


def _tile_k128(payload: torch.Tensor) -> torch.Tensor:
    """[E, rows, K/2] int8 -> [E, K/128, rows, 64]; [rows, K] e4m3 -> [K/128, rows, 128]."""
    if payload.dtype == torch.int8:
        if payload.ndim != 3:
            raise ValueError('routed FP4 weights must be packed int8 3D')
        segment = 64
    elif payload.dtype == torch.float8_e4m3fn:
        if payload.ndim != 2:
            raise ValueError('shared FP8 weights must be 2D FP8')
        segment = 128
    else:
        raise ValueError('weights must be packed FP4 (int8) or FP8 e4m3')
    if not payload.is_contiguous():
        raise ValueError('weight dense storage must be contiguous')
    if payload.shape[-1] % segment:
        raise ValueError('weight K axis must contain whole tile segments')
    *lead, rows, cols = payload.shape
    return (payload.view(*lead, rows, cols // segment, segment)
            .transpose(-2, -3).contiguous())


def _transform_on_gpu(payload: torch.Tensor, sf: torch.Tensor, interleave: bool):
    """One (payload, SF) pair through the native kernels."""
    from . import _native
    if payload.dtype == torch.int8:
        if payload.ndim != 3:
            raise ValueError('routed FP4 weights must be packed int8 3D')
        segment = 64
    elif payload.dtype == torch.float8_e4m3fn:
        if payload.ndim != 2:
            raise ValueError('shared FP8 weights must be 2D FP8')
        segment = 128
    else:
        raise ValueError('weights must be packed FP4 (int8) or FP8 e4m3')
    if not payload.is_contiguous():
        raise ValueError('weight dense storage must be contiguous')
    *lead, rows, cols = payload.shape
    if cols % segment:
        raise ValueError('weight K axis must contain whole tile segments')
    if interleave and rows % 16:
        raise ValueError('W1 rows must be a multiple of 16')
    groups = lead[0] if lead else 1
    out = torch.empty((*lead, cols // segment, rows, segment), dtype=payload.dtype, device=payload.device)
    args = _native.TransformArgs(payload_in=payload.data_ptr(), payload_out=out.data_ptr(), groups=groups, rows=rows,
                                 row_bytes=cols, segment_bytes=segment, interleave_gate_up=int(interleave))
    if sf.dtype == torch.uint8:
        # raw 128 x 128 block codes of a 2-D FP8 weight: expanded by the kernel
        k_blocks = cols // 128
        if payload.ndim != 2 or rows % 128 or sf.shape != (rows // 128, k_blocks) or not sf.is_contiguous():
            raise ValueError('block codes must be contiguous uint8 [rows / 128, K / 128] of a 2D FP8 weight')
        packs = (k_blocks + 3) // 4
        sf_out = torch.empty_strided((rows, packs), (1, rows), dtype=torch.int32, device=payload.device)
        args.block_codes, args.k_blocks = sf.data_ptr(), k_blocks
    else:
        if sf.dtype != torch.int32 or sf.ndim != payload.ndim or sf.shape[-2] != rows or rows % 128:
            raise ValueError('SF must be packed int32 with 128-aligned rows')
        if sf.ndim == 3 and sf.shape[0] != groups:
            raise ValueError('SF and payload must have the same leading dimension')
        packs = sf.shape[-1]
        sf_out = torch.empty_like(sf)              # keeps the MN-major strides of the input
        args.sf_in = sf.data_ptr()
        strides = sf.stride() if sf.ndim == 3 else (0, *sf.stride())
        args.sf_in_stride_g, args.sf_in_stride_r, args.sf_in_stride_p = strides
    out_strides = sf_out.stride() if sf_out.ndim == 3 else (0, *sf_out.stride())
    args.sf_out = sf_out.data_ptr()
    args.sf_out_stride_g, args.sf_out_stride_r, args.sf_out_stride_p = out_strides
    args.sf_packs = packs
    stream = torch.cuda.current_stream().cuda_stream
    _native.raise_for(_native.library().gcmoe_transform_weights(ctypes.byref(args), ctypes.c_void_p(stream)))
    return out, sf_out


def transform_weights_for_gc_moe(l1_weights, l2_weights, activation: str = 'swiglu'):
    """Convert original quantised (payload, SF) pairs into the K128-tiled form
    the operator consumes.  Runs on the current stream; call outside graph
    capture.  The returned tensors own their storage."""
    if activation != 'swiglu':
        raise ValueError('GC MoE supports swiglu')
    pairs = (l1_weights, l2_weights)
    if any(not isinstance(pair, (tuple, list)) or len(pair) != 2
           or any(not isinstance(t, torch.Tensor) for t in pair) for pair in pairs):
        raise ValueError('transform needs two original quantized (payload, SF) pairs')
    on_gpu = all(t.is_cuda for pair in pairs for t in pair)
    if on_gpu:
        if any(t.device.index != torch.cuda.current_device() for pair in pairs for t in pair):
            raise ValueError('transform inputs must use the current CUDA device')
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError('transform weights outside CUDA Graph capture')
    elif any(t.is_cuda for pair in pairs for t in pair):
        raise ValueError('transform inputs must live on one device')
    if on_gpu:
        return _transform_on_gpu(*l1_weights, interleave=True), _transform_on_gpu(*l2_weights, interleave=False)
    sources = {pair[0].untyped_storage().data_ptr() for pair in pairs}
    tiled = [_tile_k128(_interleave_gate_up(l1_weights[0])), _tile_k128(l2_weights[0])]
    tiled = [t.clone() if t.untyped_storage().data_ptr() in sources else t for t in tiled]
    sf1 = _sf_rows_to_4x32(_interleave_gate_up(l1_weights[1]))
    sf2 = _sf_rows_to_4x32(l2_weights[1])
    return (tiled[0], sf1), (tiled[1], sf2)
