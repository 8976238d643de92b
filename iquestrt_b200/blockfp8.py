"""Block-FP8 weights: dequantisation and rank-local scale tables.

Same names, argument meaning and error type as the reference's `iquestrt/blockfp8.py`
(`dequant` L10-21, `shard_scale` L24-36).  These run at weight-preparation time on whatever
device the tensors live on; the decode path itself never dequantises (the kernels apply
the scales to fp32 partial sums)."""

from __future__ import annotations

import torch

BLOCK = 128


def dequant(q: torch.Tensor, scale: torch.Tensor, block: tuple[int, int] = (BLOCK, BLOCK),
            dtype: torch.dtype = torch.float64) -> torch.Tensor:
    """`q [..., R, C]` e4m3 times its scale table `[..., R/br, C/bc]`, in `dtype`.

    The weight is viewed as a grid of `br x bc` tiles and every tile is multiplied by its
    own table entry (a broadcast over two inserted axes; the table is never expanded to
    the weight's size)."""
    br, bc = block
    *lead, rows, cols = q.shape
    grid = (*lead, rows // br, cols // bc)
    if rows % br or cols % bc or tuple(scale.shape) != grid:
        raise ValueError(f"a {tuple(q.shape)} weight in {br}x{bc} blocks needs a scale table of "
                         f"shape {grid}, got {tuple(scale.shape)}")
    tiles = q.to(dtype).reshape(*lead, rows // br, br, cols // bc, bc)
    return (tiles * scale.to(dtype)[..., :, None, :, None]).reshape(q.shape)


def shard_scale(scale: torch.Tensor, dim: int, start: int, length: int,
                grain: int) -> torch.Tensor:
    """Scale table of the weight slice `[start, start + length)` along `dim`, with one
    entry per `grain` elements.  `grain` must divide the 128-element block and tile the
    slice; entry j of the result is the checkpoint entry of the block that holds element
    `start + j * grain`."""
    if grain <= 0 or BLOCK % grain or start % grain or length % grain:
        raise ValueError(f"a grain of {grain} cannot tile [{start}, {start + length}) inside "
                         f"{BLOCK}-element blocks")
    per_block = BLOCK // grain
    first, count = start // grain, length // grain
    source = torch.arange(first, first + count, device=scale.device).div(per_block,
                                                                         rounding_mode="floor")
    return scale.index_select(dim, source)
