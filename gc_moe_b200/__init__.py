"""B200-native (sm_100a) implementation of the gc-moe fp8 x fp4 MoE layer.

The public names and signatures are the reference's (gc_moe/__init__.py:3-39)
so that ``import gc_moe_b200 as gc_moe`` is a drop-in for this operator.
``stage_inputs_for_gc_moe`` is an addition: the fused upstream producer the
reference's README suggests (README.md:387).
"""

from .buffer import GCSymmBuffer, get_symm_buffer_for_gc_moe
from .heuristics import get_block_m_for_gc_moe
from .operator import fp8_fp4_gc_moe
from .producer import stage_inputs_for_gc_moe
from .weights import transform_weights_for_gc_moe

__all__ = ['GCSymmBuffer', 'get_symm_buffer_for_gc_moe', 'get_block_m_for_gc_moe',
           'fp8_fp4_gc_moe', 'transform_weights_for_gc_moe', 'stage_inputs_for_gc_moe']
__version__ = '0.1.0'
