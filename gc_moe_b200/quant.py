"""Input producers for the operator: FP8/FP4 quantisers in the formats
``fp8_fp4_gc_moe`` consumes.  Plain torch ops, so they run on the GPU.

The reference takes these from a third-party package it does not vendor
(deep-gemm, tests/test_gc_moe.py:117-122,149-150); the formats below are the
ones its own code decodes (tests/test_sm120_gc_moe.py:43,80-98;
tests/test_gc_moe_se.py:167-179): e4m3 activations and e2m1 weights (two codes
per byte, even k in the low nibble, sign in bit 3) with one UE8M0 scale
``2^ceil(log2(amax / max_code))`` per 32 elements along K, four scale bytes
per little-endian int32 word, weight scale words MN-major.
"""

from __future__ import annotations

import torch

E4M3_MAX = 448.0
_FP4_MIDPOINTS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)


def _scale_exponent_byte(ratio: torch.Tensor) -> torch.Tensor:
    """Biased exponent of the smallest power of two >= ratio (ratio >= 0)."""
    ratio = ratio.double().clamp_min(2.0 ** -127)
    exp = torch.ceil(torch.log2(ratio))
    exp = torch.where(torch.exp2(exp - 1) >= ratio, exp - 1, exp)
    exp = torch.where(torch.exp2(exp) < ratio, exp + 1, exp)
    return (exp + 127).clamp(0, 254).to(torch.uint8)


def pack_scale_bytes(codes: torch.Tensor) -> torch.Tensor:
    """[..., n] uint8 -> [..., ceil(n/4)] int32; missing bytes are 127 (scale 1)."""
    pad = -codes.shape[-1] % 4
    if pad:
        codes = torch.nn.functional.pad(codes, (0, pad), value=127)
    return codes.contiguous().view(torch.int32)


def quantize_activations(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[T, K] -> (e4m3 [T, K], int32 [T, K/128]) with K32 UE8M0 scales."""
    t, k = x.shape
    groups = x.float().reshape(t, k // 32, 32)
    codes = _scale_exponent_byte(groups.abs().amax(-1) / E4M3_MAX)
    scale = torch.exp2(codes.float() - 127.0)
    q = (groups / scale[..., None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(t, k), pack_scale_bytes(codes)


def quantize_weights_fp4(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """[..., rows, K] -> (int8 [..., rows, K/2], uint8 scale bytes [..., rows, K/32])."""
    *lead, rows, k = w.shape
    groups = w.float().reshape(*lead, rows, k // 32, 32)
    codes = _scale_exponent_byte(groups.abs().amax(-1) / 6.0)
    v = groups / torch.exp2(codes.float() - 127.0)[..., None]
    mids = torch.tensor(_FP4_MIDPOINTS, dtype=torch.float32, device=w.device)
    a = v.abs().clamp_max(6.0)
    code = torch.bucketize(a, mids, right=False)             # a == midpoint -> lower code
    tie = (a == mids[code.clamp_max(6)]) & (code < 7) & (code % 2 == 1)
    code = torch.where(tie, code + 1, code)                   # ties to the even code
    nib = (code | ((v < 0).long() << 3)).to(torch.uint8).reshape(*lead, rows, k // 2, 2)
    return (nib[..., 0] | (nib[..., 1] << 4)).view(torch.int8), codes


def _mn_major(words: torch.Tensor) -> torch.Tensor:
    """Same values, memory MN-major: stride 1 along rows and `rows` along the
    packed K axis (also when that axis has a single column)."""
    *lead, rows, packs = words.shape
    strides = [rows * packs * int(torch.tensor(lead[i + 1:]).prod()) if lead[i + 1:] else rows * packs
               for i in range(len(lead))] + [1, rows]
    out = torch.empty_strided(tuple(words.shape), tuple(strides), dtype=words.dtype, device=words.device)
    out.copy_(words)
    return out


def weight_scales_mn_major(codes: torch.Tensor) -> torch.Tensor:
    """uint8 [E, rows, K/32] -> int32 [E, rows, K/128] stored MN-major, the
    form transform_weights_for_gc_moe expects."""
    return _mn_major(pack_scale_bytes(codes))


def route(logits: torch.Tensor, topk: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Top-k expert ids (int64) and softmax-over-the-selected-k weights (f32)."""
    top, idx = torch.topk(logits.float(), topk, dim=-1, sorted=False)
    return idx.to(torch.int64), torch.softmax(top, dim=-1)


def quantize_weights_fp8_blocks(w: torch.Tensor, block: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """[rows, K] -> (e4m3 [rows, K], uint8 scale bytes [rows/block, K/block]):
    one UE8M0 scale per block x block tile, the shared expert's K128 recipe
    (tests/test_gc_moe_se.py:69-71)."""
    rows, k = w.shape
    tiles = w.float().reshape(rows // block, block, k // block, block)
    codes = _scale_exponent_byte(tiles.abs().amax(dim=(1, 3)) / E4M3_MAX)
    scale = torch.exp2(codes.float() - 127.0)[:, None, :, None]
    q = (tiles / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.reshape(rows, k), codes


def expand_block_scales(codes: torch.Tensor, rows: int, block: int = 128) -> torch.Tensor:
    """Block-row scale bytes [rows/block, K/block] -> one packed int32 scale row
    per output row, MN-major [rows, ceil(K/block/4)]: the form
    transform_weights_for_gc_moe expects for K128 shared weights
    (README.md:347-351)."""
    per_row = codes.repeat_interleave(block, 0)[:rows]
    return _mn_major(pack_scale_bytes(per_row))
