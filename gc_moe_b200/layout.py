"""Byte layout of the symmetric MoE workspace (one arena per rank).

The arena is laid out exactly as the reference operator lays out its own
(gc_moe/layout/gc_moe.py:110-251): a fixed signal header, the routing
workspace, then the tensor regions.  Keeping the offsets identical is what
lets the dispatch data products be compared byte for byte with the oracle,
and lets peers address each other's regions as ``peer_base + offset``.

Only the arithmetic is shared with the reference; how the regions are used by
the kernels of this package is described next to each kernel.
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import cached_property

# Geometry limits of the operator (gc_moe/layout/gc_moe.py:12-24).
CANDIDATE_BLOCK_M = (8, 16, 32, 64, 96, 128, 192, 240)
TOKEN_ALIGNMENT = 1920          # lcm of the usable block-M candidates
MAX_RANKS = 72
MAX_EXPERTS = 2048
MAX_EXPERTS_PER_RANK = 512
MAX_RING_BLOCKS = 1 << 20
MAX_SHARED_L2_BLOCKS = 1 << 15


def round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


def ceil_div(value: int, divisor: int) -> int:
    return -(-value // divisor)


# (name, element count, element bytes, alignment) in arena order.
_SIGNAL_FIELDS = (
    ('grid_sync_count', 4, 4, 4),
    ('l1_task_count', 2, 4, 4),
    ('l2_task_count', 2, 4, 4),
    ('shared_l1_task_count', 2, 4, 4),
    ('shared_l2_task_count', 2, 4, 4),
    ('recv_parity', 1, 4, 4),
    ('role3_epoch', 1, 4, 4),
    ('routed_pool_blocks', 1, 4, 4),
    ('combine_ready_grid_idx', MAX_RANKS, 8, 128),
    ('expert_send_count', MAX_EXPERTS, 8, 128),
    ('expert_recv_count', 2 * MAX_EXPERTS, 8, 8),
    ('expert_recv_count_sum', 2 * MAX_EXPERTS_PER_RANK, 8, 8),
    ('l1_full_count', MAX_RING_BLOCKS, 4, 4),
    ('l1_empty_count', MAX_RING_BLOCKS, 4, 4),
    ('l2_full_mask', MAX_RING_BLOCKS, 8, 8),
    ('l2_empty_count', MAX_RING_BLOCKS, 4, 4),
    ('shared_l2_full_count', MAX_SHARED_L2_BLOCKS, 4, 4),
)


def _build_signal_offsets() -> dict[str, int]:
    cursor, table = 0, {}
    for name, count, width, alignment in _SIGNAL_FIELDS:
        cursor = round_up(cursor, alignment)
        table[name] = cursor
        cursor += count * width
    table['size'] = round_up(cursor, 128)
    return table


SIGNAL_OFFSETS = _build_signal_offsets()


@dataclass(frozen=True)
class BufferView:
    """One typed region of the arena: byte offset, size, logical shape."""
    offset: int
    nbytes: int
    shape: tuple
    dtype: str
    stride: tuple | None = None


@dataclass(frozen=True)
class GCBufferLayout:
    """Offsets of every region for one (ranks, experts, capacity, ...) tuple.

    Field names and validation follow gc_moe/layout/gc_moe.py:161-196 so that
    a layout built here compares equal, field by field, to the reference's.
    """
    num_ranks: int
    num_experts: int
    capacity: int
    topk: int
    hidden: int
    intermediate: int
    ring_tokens: int
    sf_ring_tokens: int
    num_shared_experts: int = 0

    def __post_init__(self) -> None:
        p, e = self.num_ranks, self.num_experts
        if not (0 < p <= MAX_RANKS and 0 < e <= MAX_EXPERTS and e % p == 0
                and e // p <= MAX_EXPERTS_PER_RANK):
            raise ValueError('invalid rank/expert configuration')
        if not (self.capacity > 0 and self.topk > 0
                and self.topk + bool(self.num_shared_experts) <= 32):
            raise ValueError('invalid capacity/topk/shared configuration')
        if (self.hidden <= 0 or self.intermediate <= 0 or self.hidden % 128
                or self.intermediate % 128):
            raise ValueError('hidden dimensions must be positive multiples of 128')
        if self.ring_tokens <= 0 or self.ring_tokens % TOKEN_ALIGNMENT:
            raise ValueError('ring token capacity must be positive and 1920-aligned')
        if (self.sf_ring_tokens < min_sf_ring_tokens(self.ring_tokens)
                or self.sf_ring_tokens % 4):
            raise ValueError('invalid scale-factor ring capacity')
        if (self.num_shared_experts < 0
                or self.intermediate * self.num_shared_experts % 128):
            raise ValueError('invalid shared expert configuration')
        if self.ring_tokens > MAX_RING_BLOCKS * min(CANDIDATE_BLOCK_M):
            raise ValueError('ring signal capacity exceeded')
        if ceil_div(self.capacity, 8) > MAX_SHARED_L2_BLOCKS:
            raise ValueError('shared L2 signal capacity exceeded')

    @property
    def local_experts(self) -> int:
        return self.num_experts // self.num_ranks

    @property
    def num_max_pool_tokens(self) -> int:
        """Upper bound of pool rows a rank can receive, padding included
        (gc_moe/layout/gc_moe.py:198-203)."""
        routes = self.num_ranks * self.capacity * min(self.topk, self.local_experts)
        padding = self.local_experts * (max(CANDIDATE_BLOCK_M) - 1)
        return round_up(routes + padding, TOKEN_ALIGNMENT)

    @cached_property
    def workspace_offsets(self) -> dict[str, int]:
        index_table = SIGNAL_OFFSETS['size']
        metadata = index_table + self.num_experts * self.capacity * 4
        end = round_up(metadata + self.num_max_pool_tokens * 12, 16)
        return {'signals': 0, 'src_token_topk_idx': index_table,
                'token_src_metadata': metadata, 'end': end}

    @cached_property
    def views(self) -> dict[str, BufferView]:
        c, h, i = self.capacity, self.hidden, self.intermediate
        s, k = self.num_shared_experts, self.topk
        ring, sf_ring = self.ring_tokens, self.sf_ring_tokens
        shared_sf_rows = ceil_div(c, 8) * 128 if s else 0
        mn_major = lambda rows: (1, rows)
        # (name, nbytes, shape, dtype, stride) in arena order.
        regions = [
            ('x', c * h, (c, h), 'float8_e4m3fn', None),
            ('x_sf', c * h // 32, (c, h // 128), 'int32', None),
            ('topk_idx', c * k * 8, (c, k), 'int64', None),
            ('topk_weights', c * k * 4, (c, k), 'float32', None),
            ('shared_l1_acts_sf', shared_sf_rows * h // 32,
             (shared_sf_rows, h // 128), 'int32',
             mn_major(shared_sf_rows) if s else None),
            ('shared_l2_acts', c * s * i, (c, s * i) if s else (0, 0),
             'float8_e4m3fn', None),
            ('shared_l2_acts_sf', shared_sf_rows * s * i // 32,
             (shared_sf_rows, s * i // 128) if s else (0, 0), 'int32',
             mn_major(shared_sf_rows) if s else None),
            ('l1_acts', ring * h, (ring, h), 'float8_e4m3fn', None),
            ('l1_acts_sf', sf_ring * h // 32, (sf_ring, h // 128), 'int32',
             mn_major(sf_ring)),
            ('l1_topk_weights', ring * 4, (ring,), 'float32', None),
            ('l2_acts', ring * i, (ring, i), 'float8_e4m3fn', None),
            ('l2_acts_sf', sf_ring * i // 32, (sf_ring, i // 128), 'int32',
             mn_major(sf_ring)),
            ('combine_tokens', (k + bool(s)) * c * h * 2, (k + bool(s), c, h),
             'bfloat16', None),
        ]
        cursor, table = self.workspace_offsets['end'], {}
        for name, nbytes, shape, dtype, stride in regions:
            table[name] = BufferView(cursor, nbytes, shape, dtype, stride)
            cursor += nbytes
            if name == 'topk_weights':
                table['shared_l1_acts'] = table['x']   # the shared expert reads x in place
        return table

    @property
    def nbytes(self) -> int:
        last = self.views['combine_tokens']
        return last.offset + last.nbytes


def min_sf_ring_tokens(ring_tokens: int) -> int:
    """Scale rows needed so that every candidate block-M can pad each of its
    blocks to a multiple of 128 scale rows."""
    return max((ring_tokens // bm) * round_up(bm, 128) for bm in CANDIDATE_BLOCK_M)


def sf_row_in_block(u: int) -> int:
    """Row, inside a 128-row-aligned scale block, that holds the packed scale
    words of the block's u-th token (gc_moe/gc/__init__.py:19-23): the 4x32
    order in which the tensor core's scale copy expects 128 rows."""
    return (u & ~127) + (u & 31) * 4 + ((u >> 5) & 3)
