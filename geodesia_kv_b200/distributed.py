"""Decode over several GPUs.

Two ways the path shards (one process per GPU, ``torch.distributed``):

* independent sequences (batched serving): each rank owns whole sequences and calls
  ``mixed_attn_decode`` on them — no communication at all;
* one long sequence: the block range of every cache row is cut into ``world`` contiguous,
  byte-balanced slices (:func:`split_blocks`); each rank runs ``mixed_attn_decode_partial`` on its
  slice, the per-head records ``[m, l, o[D]]`` are all-gathered (``Hq * (D + 2)`` floats per rank)
  and merged locally (:func:`sequence_split_decode`).  The gathered records land in local memory
  before any kernel reads them.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist

from .pack_layout import block_nbytes


def block_cost_bytes(level: Sequence[int], D: int, group: int) -> list[int]:
    """Bytes the decode kernel reads for each block: packed bytes + scale planes of quantised rungs."""
    G, gv = (64 + group - 1) // group, (D + group - 1) // group
    scale = 4 * (G * D + 64 * gv)
    return [block_nbytes(int(lv), D) + (scale if int(lv) in (8, 4, 2) else 0) for lv in level]


def split_blocks(level: Sequence[int], D: int, group: int, world: int) -> list[tuple[int, int]]:
    """Contiguous block ranges [(lo, hi)] per rank with (nearly) equal bytes to read.

    Rung sizes span 64x, so equal block counts would leave ranks unevenly loaded.  Every block
    belongs to exactly one rank; trailing ranks may be empty when there are fewer blocks than ranks.
    """
    cost = block_cost_bytes(level, D, group)
    nb, total = len(cost), sum(cost)
    bounds, acc, b = [0], 0, 0
    for r in range(1, world):
        target = total * r / world
        while b < nb and acc + cost[b] / 2 <= target:
            acc += cost[b]
            b += 1
        bounds.append(b)
    bounds.append(nb)
    return [(bounds[r], bounds[r + 1]) for r in range(world)]


def gather_and_combine(partial: torch.Tensor, combine: Callable[[torch.Tensor], torch.Tensor],
                       group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """All-gather the (B, Hq, D+2) records of every rank and merge them with ``combine``."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return combine(partial[None])
    partial = partial.contiguous()
    gathered = torch.empty((world * partial.shape[0],) + tuple(partial.shape[1:]), dtype=partial.dtype,
                           device=partial.device)            # rank-major concatenation along dim 0
    dist.all_gather_into_tensor(gathered, partial, group=group)
    return combine(gathered.view((world,) + tuple(partial.shape)))


def sequence_split_decode(q: torch.Tensor, cache, lo: int, hi: int, group: dist.ProcessGroup | None = None):
    """This rank's share of a sequence-split decode step.

    ``cache`` is a :class:`PackedCache` holding (at least) blocks [lo, hi) of every row at their
    usual offsets; q (B, Hq, D) is the full, pre-scaled query on every rank.  Returns (B, Hq, D).
    """
    from .cuda_ext import get_ext
    ext = get_ext()
    if ext is None:
        raise RuntimeError("sequence_split_decode needs the CUDA extension; there is no CPU path")
    if lo == 0 and hi == cache.offs.shape[-1] and cache.offs.is_contiguous():
        # the rank holds exactly its own blocks: pass the tensors through (no slicing, no copies)
        views = (cache.data, cache.offs, cache.klo, cache.kstep, cache.vlo, cache.vstep, cache.level, cache.valid)
    else:
        sl = slice(lo, hi)
        views = (cache.data, cache.offs[..., sl].contiguous(), cache.klo[:, :, sl].contiguous(),
                 cache.kstep[:, :, sl].contiguous(), cache.vlo[:, :, sl].contiguous(),
                 cache.vstep[:, :, sl].contiguous(), cache.level[..., sl].contiguous(),
                 cache.valid[..., sl].contiguous())
    partial = ext.mixed_attn_decode_partial(q, *views, 64, cache.group)
    return gather_and_combine(partial, ext.combine_partials, group)
