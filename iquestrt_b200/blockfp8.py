"""Block-FP8 weights: dequantisation and rank-local scale tables.

Same names, arguments and errors as the reference's `iquestrt/blockfp8.py` (L10-36).
These run at weight-preparation time on whatever device the tensors live on; the decode
path itself never dequantises (the kernels apply the scales to fp32 partial sums)."""

from __future__ import annotations

import torch

BLOCK = 128


def dequant(q: torch.Tensor, scale: torch.Tensor, block: tuple[int, int] = (BLOCK, BLOCK),
            dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """`q [..., R, C]` e4m3 with `scale [..., R/br, C/bc]` -> `q * scale[block]`."""
    br, bc = block
    if q.shape[-2] != scale.shape[-2] * br or q.shape[-1] != scale.shape[-1] * bc:
        raise ValueError(f"scale {tuple(scale.shape)} at block {block} does not tile "
                         f"weight {tuple(q.shape)}")
    s = scale.to(dtype).repeat_interleave(br, -2).repeat_interleave(bc, -1)
    return q.to(dtype) * s


def shard_scale(scale: torch.Tensor, dim: int, start: int, length: int,
                grain: int) -> torch.Tensor:
    """The scale table of the weight slice `[start, start + length)` along `dim`, one
    entry per `grain` (which must divide 128 and tile the slice)."""
    if BLOCK % grain or start % grain or length % grain:
        raise ValueError(f"grain {grain} does not tile slice [{start}, {start + length}) "
                         f"inside {BLOCK}-blocks")
    blocks = (start + torch.arange(0, length, grain, device=scale.device)) // BLOCK
    return scale.index_select(dim, blocks)
