"""Decode over several GPUs.

Two ways the path shards (one process per GPU, ``torch.distributed``):

* independent sequences (batched serving): each rank owns whole sequences and calls
  ``mixed_attn_decode`` on them — no communication at all;
* one long sequence: the block range of every cache row is cut into ``world`` contiguous,
  byte-balanced slices (:func:`split_blocks`); each rank attends over its slice and the per-head
  records ``[m, l, o[D]]`` (``Hq * (D + 2)`` floats per rank) are exchanged and merged.

The exchange has two forms.  :class:`SequenceSplitDecoder` does it inside this library's own merge
kernel: every rank stores its records into every rank's inbox (one symmetric allocation, plain
peer stores over NVLink), raises a sequence number and waits, bounded, for the others' — a step
is then made of this library's kernels only and can be replayed from a CUDA graph.  Where peer
memory cannot be set up it falls back to :func:`gather_and_combine`: one NCCL all-gather into
local memory, then the local merge kernel.
"""
from __future__ import annotations

import ctypes
from typing import Callable

import torch
import torch.distributed as dist

from .pack_layout import block_nbytes


def block_cost_bytes(level, D: int, group: int) -> list[int]:
    """Bytes the decode kernel reads for each block: packed bytes + scale planes of quantised rungs."""
    G, gv = (64 + group - 1) // group, (D + group - 1) // group
    scale = 4 * (G * D + 64 * gv)
    return [block_nbytes(int(lv), D) + (scale if int(lv) in (8, 4, 2) else 0) for lv in level]


def block_cost_tensor(level: torch.Tensor, D: int, group: int) -> torch.Tensor:
    """:func:`block_cost_bytes` for a tensor of rungs of any shape (int64, same shape, same device)."""
    G, gv = (64 + group - 1) // group, (D + group - 1) // group
    scale = 4 * (G * D + 64 * gv)
    cost = torch.zeros_like(level, dtype=torch.int64)
    for rung in (16, 8, 4, 2, 1):
        cost += (level == rung).to(torch.int64) * (block_nbytes(rung, D) + (scale if rung in (8, 4, 2) else 0))
    return cost


def split_blocks(level, D: int, group: int, world: int) -> list[tuple[int, int]]:
    """Contiguous block ranges [(lo, hi)] per rank with (nearly) equal bytes to read.

    ``level`` holds the rungs of the blocks, (nb,) or (rows, nb); with several rows the cut balances
    the summed cost of the rows (one cut for all of them).  Rung sizes span 64x, so equal block
    counts would leave ranks unevenly loaded.  Every block belongs to exactly one rank; trailing
    ranks may be empty when there are fewer blocks than ranks.
    """
    lv = torch.as_tensor(level).to(torch.int64)
    cost = block_cost_tensor(lv.reshape(-1, lv.shape[-1]), D, group).sum(0).cpu()
    nb = cost.numel()
    if nb == 0:
        return [(0, 0)] * world
    ends = torch.cumsum(cost, 0)
    mids = ends - cost // 2                                  # a block goes to the rank its middle byte falls in
    total = int(ends[-1])
    targets = torch.tensor([total * r // world for r in range(1, world)], dtype=torch.int64)
    cuts = torch.searchsorted(mids, targets, right=False).tolist() if world > 1 else []
    bounds = [0] + [min(max(int(c), 0), nb) for c in cuts] + [nb]
    for i in range(1, len(bounds)):                          # keep the cuts ordered
        bounds[i] = max(bounds[i], bounds[i - 1])
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


def slice_cache(cache, lo: int, hi: int):
    """The blocks [lo, hi) of every row of a :class:`PackedCache` as a cache of its own (one copy of
    the metadata and scale planes, made once; the packed bytes are shared, not copied)."""
    from .pack_layout import PackedCache
    if lo == 0 and hi == cache.nb:
        return cache
    sl = slice(lo, hi)
    return PackedCache(cache.data, cache.offs[..., sl].contiguous(), cache.klo[:, :, sl].contiguous(),
                       cache.kstep[:, :, sl].contiguous(), cache.vlo[:, :, sl].contiguous(),
                       cache.vstep[:, :, sl].contiguous(), cache.level[..., sl].contiguous(),
                       cache.valid[..., sl].contiguous(), cache.group, cache.D)


def sequence_split_decode(q: torch.Tensor, cache, lo: int, hi: int, group: dist.ProcessGroup | None = None):
    """This rank's share of a sequence-split decode step, exchanged with an NCCL all-gather.

    ``cache`` is a :class:`PackedCache` holding (at least) blocks [lo, hi) of every row at their
    usual offsets; q (B, Hq, D) is the full, pre-scaled query on every rank.  Returns (B, Hq, D).
    A caller that attends over the same slice step after step slices once with :func:`slice_cache`
    and passes ``lo = 0, hi = nb`` of the slice: nothing is copied per call then.
    """
    from .cuda_ext import get_ext
    ext = get_ext()
    if ext is None:
        raise RuntimeError("sequence_split_decode needs the CUDA extension; there is no CPU path")
    mine = slice_cache(cache, lo, hi)
    partial = ext.mixed_attn_decode_partial(q, *mine.kernel_args())
    return gather_and_combine(partial, ext.combine_partials, group)


class SequenceSplitDecoder:
    """Sequence-split decode whose exchange happens inside the merge kernel (peer stores, no collective).

    One instance serves every layer of a model for a fixed (B, Hq, D): it owns this rank's inbox (a
    symmetric allocation every rank can store into), the per-row sequence numbers and the status
    word.  All ranks must call it the same number of times in the same order.  ``available`` is
    False when peer memory could not be set up; callers then use :func:`sequence_split_decode`.
    """

    def __init__(self, B: int, Hq: int, D: int, device, group: dist.ProcessGroup | None = None):
        from .cuda_ext import get_ext
        self.ext = get_ext()
        if self.ext is None:
            raise RuntimeError("SequenceSplitDecoder needs the CUDA extension; there is no CPU path")
        self.B, self.Hq, self.D = B, Hq, D
        self.device = torch.device(device)
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.available, self.why = False, ""
        lib = self.ext.lib
        nbytes = lib.gkv_exchange_inbox_bytes(self.world, B * Hq, D)
        if nbytes == 0:
            self.why = "world size beyond what the exchange kernel takes"
            return
        try:
            if self.world == 1:
                self.inbox = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
                ptrs = [self.inbox.data_ptr()]
            else:
                import torch.distributed._symmetric_memory as symm
                pg = group if group is not None else dist.group.WORLD
                self.inbox = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
                self.inbox.zero_()
                self._handle = symm.rendezvous(self.inbox, pg.group_name)
                ptrs = [int(p) for p in self._handle.buffer_ptrs]
                torch.cuda.synchronize(self.device)
                dist.barrier(group)                      # every inbox is zero before anyone stores into it
        except Exception as e:                           # no peer access, no symmetric memory in this build, ...
            self.why = f"{type(e).__name__}: {e}"
            return
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        self.seq = torch.zeros(B * Hq, dtype=torch.int32, device=self.device)
        self.xstatus = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.available = True

    def __call__(self, q: torch.Tensor, cache) -> torch.Tensor:
        """Attend over this rank's ``cache`` (its slice of every row) and return the full (B, Hq, D) output."""
        from . import _lib
        from .cuda_ext import _ptr, _stream
        ext, lib = self.ext, self.ext.lib
        B, Hq, D = q.shape
        if (B, Hq, D) != (self.B, self.Hq, self.D) or q.dtype != torch.float32 or not q.is_contiguous():
            raise RuntimeError("q must be contiguous float32 of the shape the decoder was made for")
        Hkv, nb = cache.data.size(1), cache.nb
        dev = q.device
        with torch.cuda.device(dev):
            need = lib.gkv_decode_workspace_bytes(B, Hq, Hkv, D, nb)
            ws = ext._workspace(dev, need)
            plan = ext._plan(cache.offs, cache.level, cache.valid, B * Hkv, nb)
            out = torch.empty(B, Hq, D, dtype=torch.float32, device=dev)
            rc = lib.gkv_mixed_attn_decode_exchange(
                q.data_ptr(), _ptr(cache.data), _ptr(cache.offs), _ptr(cache.klo), _ptr(cache.kstep), _ptr(cache.vlo),
                _ptr(cache.vstep), _ptr(cache.level), _ptr(cache.valid), out.data_ptr(), _ptr(plan), ws.data_ptr(),
                ws.numel(), B, Hq, Hkv, D, nb, 64, cache.group, cache.data.size(-1), B * Hkv, self._ptrs, self.rank,
                self.world, self.seq.data_ptr(), self.xstatus.data_ptr(), _stream(dev))
        _lib.check(rc, "gkv_mixed_attn_decode_exchange")
        return out

    def status(self) -> int:
        """0, or non-zero once a wait for another rank's records has run out (synchronises)."""
        return int(self.xstatus.item())
