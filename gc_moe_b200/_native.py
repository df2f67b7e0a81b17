"""ctypes binding of libgcmoe_sm100.so (the C ABI declared in include/gcmoe.h).

There is no fallback: if the library is missing or a call fails, the caller
gets an exception.  The library is built by ``python -m gc_moe_b200.build``.
"""

from __future__ import annotations

import ctypes
import os

MAX_RANKS = 72
STATUS_WORDS = 8

ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_DEVICE = -1, -2, -3, -4


class Problem(ctypes.Structure):
    _fields_ = [(name, ctypes.c_int32) for name in (
        'num_ranks', 'rank', 'num_experts', 'capacity', 'topk', 'hidden',
        'intermediate', 'num_tokens', 'block_m', 'ring_tokens', 'sf_ring_tokens',
        'num_shared_experts', 'shared_gran_k', 'has_clamp')] + [
        ('clamp', ctypes.c_float)] + [(name, ctypes.c_int32) for name in (
            'fast_math', 'timeout_ms', 'num_sms', 'dispatch_sms')]


class Buffers(ctypes.Structure):
    _fields_ = [('arena_base', ctypes.c_uint64 * MAX_RANKS)] + [
        (name, ctypes.c_uint64) for name in (
            'off_recv_parity', 'off_routed_pool_blocks',
            'off_recv_count', 'off_recv_count_sum',
            'off_index_table', 'off_metadata',
            'off_x', 'off_x_sf', 'off_topk_idx', 'off_topk_weights',
            'off_l1_acts', 'off_l1_acts_sf', 'off_l1_topk_weights',
            'off_l2_acts', 'off_l2_acts_sf', 'off_combine_tokens',
            'off_shared_l1_acts_sf', 'off_shared_l2_acts', 'off_shared_l2_acts_sf',
            'shared_sf_rows', 'y', 'stats',
            'w1', 'w1_sf', 'w2', 'w2_sf', 'w1_sf_stride', 'w2_sf_stride',
            'sw1', 'sw1_sf', 'sw2', 'sw2_sf', 'sw1_sf_stride', 'sw2_sf_stride',
            'scratch', 'scratch_bytes', 'off_exchange')]


class StageArgs(ctypes.Structure):
    _fields_ = [(name, ctypes.c_uint64) for name in (
        'x', 'router_logits', 'topk_idx_in', 'topk_weights_in', 'x_q', 'x_sf', 'topk_idx',
        'topk_weights', 'shared_sf')] + [(name, ctypes.c_uint32) for name in (
            'shared_sf_rows', 'block_m', 'num_tokens', 'hidden', 'num_experts', 'topk')]


class TransformArgs(ctypes.Structure):
    _fields_ = [(name, ctypes.c_uint64) for name in (
        'payload_in', 'payload_out', 'sf_in', 'sf_out', 'block_codes',
        'sf_in_stride_g', 'sf_in_stride_r', 'sf_in_stride_p',
        'sf_out_stride_g', 'sf_out_stride_r', 'sf_out_stride_p')] + [(name, ctypes.c_uint32) for name in (
            'groups', 'rows', 'row_bytes', 'segment_bytes', 'sf_packs', 'k_blocks', 'interleave_gate_up',
            'reserved')]


# GC_MOE_B200_LIBRARY points at another build of the same library (a tuning variant).
LIBRARY_PATH = os.environ.get('GC_MOE_B200_LIBRARY') or os.path.join(
    os.path.dirname(os.path.abspath(__file__)), 'libgcmoe_sm100.so')

# name -> (restype, argtypes); every symbol include/gcmoe.h declares.
_SIGNATURES = {
    'gcmoe_version': (ctypes.c_int, []),
    'gcmoe_last_error': (ctypes.c_char_p, []),
    'gcmoe_scratch_bytes': (ctypes.c_size_t, [ctypes.POINTER(Problem)]),
    'gcmoe_plan_create': (ctypes.c_int, [ctypes.POINTER(Problem), ctypes.POINTER(Buffers),
                                         ctypes.POINTER(ctypes.c_void_p)]),
    'gcmoe_plan_destroy': (ctypes.c_int, [ctypes.c_void_p]),
    'gcmoe_launch': (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p]),
    'gcmoe_launch_kernels': (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p]),
    'gcmoe_kernels_per_launch': (ctypes.c_int, [ctypes.c_void_p]),
    'gcmoe_status_read': (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p,
                                         ctypes.POINTER(ctypes.c_uint32)]),
    'gcmoe_stage_inputs': (ctypes.c_int, [ctypes.POINTER(StageArgs), ctypes.c_void_p]),
    'gcmoe_transform_weights': (ctypes.c_int, [ctypes.POINTER(TransformArgs), ctypes.c_void_p]),
    'gcmoe_launch_static_scratch': (ctypes.c_int, [ctypes.POINTER(Problem), ctypes.POINTER(Buffers), ctypes.c_void_p]),
    'gcmoe_static_scratch_status': (ctypes.c_int, [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint32)]),
    'gcmoe_debug_expire_wait': (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint, ctypes.c_void_p]),
    'gcmoe_debug_gemm_l1_raw': (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]),
}
EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def library() -> ctypes.CDLL:
    """Load the native library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY_PATH):
            raise RuntimeError(
                f'{LIBRARY_PATH} is missing: build it with `python -m gc_moe_b200.build`; '
                'there is no fallback path')
        lib = ctypes.CDLL(LIBRARY_PATH)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = lib
    return _lib


def last_error() -> str:
    return library().gcmoe_last_error().decode('utf-8', 'replace')


def raise_for(code: int) -> None:
    """Map a gcmoe_error to the exception type the reference raises for the
    same class of failure (gc_moe/apis/gc_moe.py:43-137 ValueError,
    gc_moe/jit_kernels/impls/sm100_fp8_fp4_gc_moe.py:524,530
    NotImplementedError, gc_moe/runtime/gc_moe.py:23-26 RuntimeError)."""
    if code == 0:
        return
    message = last_error()
    if code == ERR_INVALID:
        raise ValueError(message)
    if code == ERR_UNSUPPORTED:
        raise NotImplementedError(message)
    raise RuntimeError(message)
