"""Paged packed KV cache: one byte pool per GPU, size-class free lists, per-row block tables.

The reference's serving plugin keeps one ``GeodesiaBlockCache`` per sequence in a dict
(``geodesia_kv/vllm_plugin/kv_cache.py:85-104``) and its capacity claim — more sequences per
GPU at a bit budget (``README.md:243-248``) — needs demotion to hand memory back.  Here it does:

* :class:`PagedPool` owns ONE ``uint8`` pool.  The pool is cut into slabs whose size is the least
  common multiple of the five slot sizes (1 474 560 bytes at D=128, g=32: 45 / 80 / 144 / 240 /
  2880 slots of the 16 / 8 / 4 / 2-bit / centroid rungs), so a slab serves exactly one rung with
  no waste and returns to the common free list when its last slot is freed.  A slot holds a block's
  bytes AND, for the quantised rungs, its four fp16 scale planes right behind them — a block is
  allocated, demoted ("allocate smaller, re-quantise, free larger") and freed as one piece.
* :class:`PagedLayerCache` is the block table of one layer: ``offs / level / valid`` of shape
  (sequences x KV heads, blocks), rows of different lengths padded with ``valid = 0``.  Prefill
  packs dense K/V straight into rung-16 slots, a decode step appends one token per row into the
  row's open block on the device, attention is ONE kernel call over the whole ragged batch (with
  the per-block softmax mass as a by-product), and maintenance runs the distortion, allocator and
  demotion kernels for all rows at once.

Free lists live on the host (numpy): a maintenance step reads the allocator's result back once,
for all rows (and, through :class:`PagedKVCache.maintain`, for all layers), which is the only
host synchronisation of the serving loop; decode steps in between launch kernels only.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Sequence

import numpy as np
import torch

from . import _lib

BLOCK = 64
LADDER = (16, 8, 4, 2, 1)
_LADDER_NP = np.array(LADDER, dtype=np.int32)
_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def _stream(dev):
    return torch.cuda.current_stream(dev).cuda_stream


def ladder_index_np(level: np.ndarray) -> np.ndarray:
    """Rungs (16, 8, 4, 2, 1) -> ladder indices 0..4."""
    lv = level.astype(np.int32)
    return (lv <= 8).astype(np.int32) + (lv <= 4) + (lv <= 2) + (lv <= 1)


class PoolExhausted(RuntimeError):
    pass


class PagedPool:
    """Byte pool with one free list per rung (host-side bookkeeping, device-side bytes)."""

    def __init__(self, capacity_bytes: int, D: int = 128, group: int = 32, device="cuda"):
        lib = _lib.load()
        self.D, self.group, self.device = D, group, torch.device(device)
        self.slot = {r: int(lib.gkv_paged_block_bytes(r, D, group)) for r in LADDER}
        if not all(self.slot.values()):
            raise ValueError(f"no paged layout for D={D}, group={group}")
        slab = 1
        for s in self.slot.values():
            slab = slab * s // math.gcd(slab, s)
        self.slab_bytes = slab if slab <= (8 << 20) else (2 << 20)
        self.n_slabs = int(capacity_bytes) // self.slab_bytes
        if self.n_slabs < 1:
            raise ValueError(f"capacity below one slab of {self.slab_bytes} bytes")
        self.data = torch.empty(self.n_slabs * self.slab_bytes, dtype=torch.uint8, device=self.device)
        self._free_slabs = list(range(self.n_slabs - 1, -1, -1))
        self._slab_rung = np.zeros(self.n_slabs, dtype=np.int32)           # 0 = unassigned
        self._slab_live = np.zeros(self.n_slabs, dtype=np.int64)
        self._stack = {r: np.empty(0, dtype=np.int64) for r in LADDER}     # free slot offsets per rung
        self._top = {r: 0 for r in LADDER}
        self.bytes_in_use = 0            # bytes of the slots handed out
        self.peak_bytes_in_use = 0

    # -- accounting ---------------------------------------------------------------------------
    @property
    def capacity_bytes(self) -> int:
        return self.n_slabs * self.slab_bytes

    @property
    def bytes_reserved(self) -> int:
        """Bytes of the slabs that currently belong to a rung (slot granularity is bytes_in_use)."""
        return (self.n_slabs - len(self._free_slabs)) * self.slab_bytes

    def slots_in_use(self, rung: int) -> int:
        return int(self._slab_live[self._slab_rung == rung].sum())

    # -- allocation ---------------------------------------------------------------------------
    def _push(self, rung: int, offs: np.ndarray) -> None:
        st, top = self._stack[rung], self._top[rung]
        if top + offs.size > st.size:
            grown = np.empty(max(2 * st.size, top + offs.size, 1024), dtype=np.int64)
            grown[:top] = st[:top]
            self._stack[rung] = st = grown
        st[top:top + offs.size] = offs
        self._top[rung] = top + offs.size

    def alloc(self, rung: int, n: int) -> np.ndarray:
        """Offsets of n free slots of a rung (int64)."""
        if n <= 0:
            return np.empty(0, dtype=np.int64)
        size = self.slot[rung]
        per_slab = self.slab_bytes // size
        while self._top[rung] < n:
            if not self._free_slabs:
                raise PoolExhausted(f"pool of {self.capacity_bytes} bytes exhausted asking for {n} slots of rung {rung} "
                                    f"({self.bytes_in_use} bytes in use)")
            s = self._free_slabs.pop()
            self._slab_rung[s] = rung
            # pushed high to low, so low addresses are handed out first
            self._push(rung, s * self.slab_bytes + np.arange(per_slab - 1, -1, -1, dtype=np.int64) * size)
        top = self._top[rung]
        out = self._stack[rung][top - n:top][::-1].copy()
        self._top[rung] = top - n
        np.add.at(self._slab_live, out // self.slab_bytes, 1)
        self.bytes_in_use += n * size
        self.peak_bytes_in_use = max(self.peak_bytes_in_use, self.bytes_in_use)
        return out

    def free(self, rung: int, offs: np.ndarray) -> None:
        """Give slots of a rung back; slabs left without a live slot return to the common list."""
        offs = np.asarray(offs, dtype=np.int64)
        if offs.size == 0:
            return
        slabs = offs // self.slab_bytes
        if np.any(self._slab_rung[slabs] != rung):
            raise ValueError("a freed offset does not belong to a slab of that rung")
        np.subtract.at(self._slab_live, slabs, 1)
        self.bytes_in_use -= offs.size * self.slot[rung]
        self._push(rung, offs)
        touched = np.unique(slabs)
        empty = touched[self._slab_live[touched] == 0]
        if empty.size:
            top = self._top[rung]
            st = self._stack[rung][:top]
            keep = st[~np.isin(st // self.slab_bytes, empty)]
            self._stack[rung][:keep.size] = keep
            self._top[rung] = keep.size
            self._slab_rung[empty] = 0
            self._free_slabs.extend(int(s) for s in empty[::-1])


class PagedLayerCache:
    """Block table of ONE layer over a :class:`PagedPool`: B sequences x Hkv heads, ragged lengths."""

    def __init__(self, pool: PagedPool, B: int, Hkv: int, cap_blocks: int = 64):
        self.pool, self.B, self.Hkv = pool, B, Hkv
        self.rows = B * Hkv
        self.D, self.group, self.device = pool.D, pool.group, pool.device
        self.lib = _lib.load()
        self.cap = 0
        self.len_h = np.zeros(B, dtype=np.int64)                     # tokens per sequence (host mirror)
        self.offs_h = np.full((self.rows, 0), -1, dtype=np.int64)
        self.level_h = np.zeros((self.rows, 0), dtype=np.int32)          # 0 = no block here
        self.offs = self.level = self.valid = self.mass = self.ek = self.ev = None
        self.lens = torch.zeros(self.rows, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._grow(cap_blocks)

    # -- tables ---------------------------------------------------------------------------------
    def _grow(self, cap: int) -> None:
        dev, rows, old = self.device, self.rows, self.cap
        def wider(t, fill, dtype):
            new = torch.full((rows, cap), fill, dtype=dtype, device=dev)
            if t is not None and old:
                new[:, :old] = t
            return new
        self.offs = wider(self.offs, -1, torch.int64)
        self.level = wider(self.level, 0, torch.int32)
        self.valid = wider(self.valid, 0, torch.int32)
        self.mass = wider(self.mass, 0.0, torch.float32)
        self.ek = wider(self.ek, 0.0, torch.float32)
        self.ev = wider(self.ev, 0.0, torch.float32)
        oh = np.full((rows, cap), -1, dtype=np.int64)
        lh = np.zeros((rows, cap), dtype=np.int32)
        oh[:, :old], lh[:, :old] = self.offs_h, self.level_h
        self.offs_h, self.level_h, self.cap = oh, lh, cap

    @property
    def nb(self) -> int:
        """Blocks of the longest row (the width the kernels are called with)."""
        return int((int(self.len_h.max()) + BLOCK - 1) // BLOCK) if self.B else 0

    def blocks_per_seq(self) -> np.ndarray:
        return (self.len_h + BLOCK - 1) // BLOCK

    def _row_blocks(self) -> np.ndarray:
        return np.repeat(self.blocks_per_seq(), self.Hkv)

    def _put(self, table: torch.Tensor, flat_idx: np.ndarray, values: np.ndarray) -> None:
        if flat_idx.size == 0:
            return
        idx = torch.from_numpy(flat_idx.astype(np.int64)).to(self.device, non_blocking=True)
        val = torch.from_numpy(np.ascontiguousarray(values)).to(self.device, non_blocking=True).to(table.dtype)
        table.view(-1).index_put_((idx,), val)

    # -- growth ---------------------------------------------------------------------------------
    def prefill(self, k: torch.Tensor, v: torch.Tensor, lengths: Sequence[int] | None = None) -> None:
        """Pack the prompts: k, v (B, Hkv, T, D) dense; sequence b keeps its first lengths[b] tokens.

        Every block enters at rung 16 (exact bf16), as in the reference (policies.py:690-700)."""
        B, Hkv, T, D = k.shape
        if (B, Hkv, D) != (self.B, self.Hkv, self.D) or int(self.len_h.max(initial=0)) != 0:
            raise ValueError("prefill needs an empty cache of matching shape")
        k, v = k.contiguous(), v.contiguous()
        lengths = np.full(B, T, dtype=np.int64) if lengths is None else np.asarray(lengths, dtype=np.int64)
        if lengths.shape != (B,) or int(lengths.min()) < 1 or int(lengths.max()) > T:
            raise ValueError("one length per sequence, between 1 and the number of token rows given")
        nblk = (lengths + BLOCK - 1) // BLOCK
        if int(nblk.max()) + 1 > self.cap:
            self._grow(int(nblk.max()) + 1 + 16)
        rows_b = np.repeat(np.arange(B), Hkv)
        row_nblk = np.repeat(nblk, Hkv)
        total = int(row_nblk.sum())
        row_of = np.repeat(np.arange(self.rows), row_nblk)                        # row of every block
        blk_of = np.arange(total) - np.repeat(np.cumsum(row_nblk) - row_nblk, row_nblk)
        slots = self.pool.alloc(16, total)
        src_off = (row_of * T + blk_of * BLOCK) * D
        nvalid = np.minimum(BLOCK, lengths[rows_b[row_of]] - blk_of * BLOCK).astype(np.int32)
        self.offs_h[row_of, blk_of] = slots
        self.level_h[row_of, blk_of] = 16
        self.len_h[:] = lengths
        flat = row_of * self.cap + blk_of
        self._put(self.offs, flat, slots)
        self._put(self.valid, flat, nvalid)
        self._put(self.level, flat, np.full(total, 16, dtype=np.int32))
        self.lens.copy_(torch.from_numpy(np.repeat(lengths, Hkv).astype(np.int32)), non_blocking=True)
        self.pack_blocks(k, v, src_off, D, nvalid, slots, np.full(total, 16, dtype=np.int32))

    def extend(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Append whole blocks to EVERY sequence: k, v (B, Hkv, n*64, D) dense; all sequences must
        stand at a block boundary (chunked prefill, or a serving loop that packs a block at a time)."""
        B, Hkv, T, D = k.shape
        if (B, Hkv, D) != (self.B, self.Hkv, self.D) or T % BLOCK or np.any(self.len_h % BLOCK):
            raise ValueError("extend appends whole blocks to sequences that stand at a block boundary")
        k, v = k.contiguous(), v.contiguous()
        n = T // BLOCK
        first = self.len_h // BLOCK
        if int(first.max()) + n + 1 > self.cap:
            self._grow(int(first.max()) + n + 1 + 63)
        row_of = np.repeat(np.arange(self.rows), n)
        blk_in = np.tile(np.arange(n), self.rows)
        blk_of = np.repeat(first, Hkv * n) + blk_in
        slots = self.offs_h[row_of, blk_of].copy()                      # slots reserved earlier are used first
        fresh = np.nonzero(slots < 0)[0]
        slots[fresh] = self.pool.alloc(16, fresh.size)
        self.offs_h[row_of, blk_of] = slots
        self.level_h[row_of, blk_of] = 16
        flat = row_of * self.cap + blk_of
        self._put(self.offs, flat, slots)
        self._put(self.level, flat, np.full(flat.size, 16, dtype=np.int32))
        self._put(self.valid, flat, np.full(flat.size, BLOCK, dtype=np.int32))
        for t in (self.mass, self.ek, self.ev):
            self._put(t, flat, np.zeros(flat.size, dtype=np.float32))
        self.len_h += T
        self.lens += T
        self.pack_blocks(k, v, (row_of * T + blk_in * BLOCK) * D, D, np.full(flat.size, BLOCK, np.int32), slots,
                         np.full(flat.size, 16, dtype=np.int32))

    def pack_blocks(self, k, v, src_off, token_stride, nvalid, slots, levels, radii: bool = False):
        """Quantise blocks from dense rows into given slots (element offsets into k and v)."""
        dev = self.device
        n = int(len(slots))
        up = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(dev, non_blocking=True).to(dt)
        so, nv, sl, lv = up(src_off, torch.int64), up(nvalid, torch.int32), up(slots, torch.int64), up(levels, torch.int32)
        ek = torch.zeros(n, dtype=torch.float32, device=dev) if radii else None
        ev = torch.zeros(n, dtype=torch.float32, device=dev) if radii else None
        with torch.cuda.device(dev):
            rc = self.lib.gkv_paged_pack_blocks(k.data_ptr(), v.data_ptr(), _DT[k.dtype], so.data_ptr(), int(token_stride),
                                                nv.data_ptr(), self.pool.data.data_ptr(), sl.data_ptr(), lv.data_ptr(),
                                                ek.data_ptr() if radii else None, ev.data_ptr() if radii else None,
                                                n, self.D, BLOCK, self.group, _stream(dev))
        _lib.check(rc, "gkv_paged_pack_blocks")
        return ek, ev

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
        """One more token for every sequence: k_new, v_new (B, Hkv, 1, D) or (B, Hkv, D)."""
        if np.any(self.len_h % BLOCK == 0):                               # some sequence opens a new block
            self.reserve(1)
        self.append_device(k_new, v_new)
        self.len_h += 1

    def reserve(self, tokens: int) -> None:
        """Give every row the rung-16 slots its next ``tokens`` appended tokens will need, so that that
        many :meth:`append_device` calls (e.g. replays of a captured step) need no host work."""
        first = (self.len_h + BLOCK - 1) // BLOCK                       # first block without a slot yet
        last = (self.len_h + tokens + BLOCK - 1) // BLOCK               # one past the last block needed
        cnt = np.maximum(last - first, 0)
        if int(cnt.sum()) == 0:
            return
        if int(last.max()) + 1 > self.cap:
            self._grow(int(last.max()) + 1 + 63)
        seq = np.repeat(np.arange(self.B), cnt)
        blk = np.arange(int(cnt.sum())) - np.repeat(np.cumsum(cnt) - cnt, cnt) + np.repeat(first, cnt)
        rows = (seq[:, None] * self.Hkv + np.arange(self.Hkv)[None]).reshape(-1)
        blks = np.repeat(blk, self.Hkv)
        have = self.offs_h[rows, blks] >= 0
        rows, blks = rows[~have], blks[~have]
        slots = self.pool.alloc(16, rows.size)
        self.offs_h[rows, blks] = slots
        self.level_h[rows, blks] = 16
        flat = rows * self.cap + blks
        self._put(self.offs, flat, slots)
        self._put(self.level, flat, np.full(rows.size, 16, dtype=np.int32))
        for t in (self.mass, self.ek, self.ev):
            self._put(t, flat, np.zeros(rows.size, dtype=np.float32))

    def sync_lengths(self) -> None:
        """Re-read the row lengths from the device (after append_device calls the host did not count)."""
        self.len_h[:] = self.lens.cpu().numpy().reshape(self.B, self.Hkv)[:, 0]

    def append_device(self, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
        """The device half of :meth:`append` (no host bookkeeping): safe inside a CUDA graph as long
        as no row crosses into a block without a slot — the status word says if one did."""
        k_new, v_new = k_new.reshape(self.rows, self.D), v_new.reshape(self.rows, self.D)
        if not (k_new.is_contiguous() and v_new.is_contiguous()):
            k_new, v_new = k_new.contiguous(), v_new.contiguous()
        dev = self.device
        with torch.cuda.device(dev):
            rc = self.lib.gkv_paged_append_token(k_new.data_ptr(), v_new.data_ptr(), _DT[k_new.dtype],
                                                 self.pool.data.data_ptr(), self.offs.data_ptr(), self.valid.data_ptr(),
                                                 self.lens.data_ptr(), self.status.data_ptr(), self.rows, self.cap,
                                                 self.D, BLOCK, _stream(dev))
        _lib.check(rc, "gkv_paged_append_token")

    # -- attention ------------------------------------------------------------------------------
    def attend(self, q: torch.Tensor, want_mass: bool = False, nb: int | None = None):
        """q (B, Hq, D) float32, already scaled -> out (B, Hq, D) [, mass (rows, table width)]: one kernel call."""
        from .cuda_ext import get_ext
        ext = get_ext()
        B, Hq, D = q.shape
        if B != self.B or D != self.D or q.dtype != torch.float32 or not q.is_contiguous():
            raise RuntimeError("q must be contiguous float32 (B, Hq, D) matching the cache")
        # by default the whole table goes in: entries beyond a row's blocks have valid = 0 and are never read
        nb = self.cap if nb is None else nb
        dev = self.device
        offs, level, valid = self.offs, self.level, self.valid
        if nb != self.cap:                                           # the kernel wants tables of width nb
            offs, level, valid = offs[:, :nb].contiguous(), level[:, :nb].contiguous(), valid[:, :nb].contiguous()
        lib = self.lib
        with torch.cuda.device(dev):
            need = (lib.gkv_decode_mass_workspace_bytes(B, Hq, self.Hkv, D, nb, self.group) if want_mass
                    else lib.gkv_decode_workspace_bytes(B, Hq, self.Hkv, D, nb))
            ws = ext._workspace(dev, need)
            out = torch.empty(B, Hq, D, dtype=torch.float32, device=dev)
            mass = torch.empty(self.rows, nb, dtype=torch.float32, device=dev) if want_mass else None
            rc = lib.gkv_paged_attn_decode(q.data_ptr(), self.pool.data.data_ptr(), self.pool.data.numel(), offs.data_ptr(),
                                           level.data_ptr(), valid.data_ptr(), out.data_ptr(),
                                           mass.data_ptr() if want_mass else None, None, ws.data_ptr(), ws.numel(),
                                           B, Hq, self.Hkv, D, nb, BLOCK, self.group, _stream(dev))
        _lib.check(rc, "gkv_paged_attn_decode")
        return (out, mass) if want_mass else out

    def observe(self, mass: torch.Tensor, decay: float) -> None:
        """Fold one step's per-block mass (rows, nb) into the running mass (policies.py:705-708)."""
        nb = mass.shape[1]
        self.mass[:, :nb].lerp_(mass, 1.0 - decay)

    # -- maintenance ----------------------------------------------------------------------------
    def hot_blocks(self, nb: int, sinks: int = 4, window: int = 128) -> torch.Tensor:
        """(rows, nb) uint8: blocks that must stay exact — sinks, the recent window, the block being
        written and its predecessor (policies.py:677-681), per row of the ragged batch."""
        lens = self.lens.to(torch.int64)[:, None]
        b = torch.arange(nb, device=self.device)[None]
        nbr = (lens + BLOCK - 1) // BLOCK
        hot = (b < max(1, (sinks + BLOCK - 1) // BLOCK)) | (b >= (lens - 1) // BLOCK - 1) | \
              (b >= nbr - max(1, (window + BLOCK - 1) // BLOCK))
        return (hot & (b < nbr)).to(torch.uint8).contiguous()

    def plan_demotion(self, budget_bits: float, sinks: int = 4, window: int = 128, mass_power: float = 1.0,
                      value_weight: float = 0.0, mass: torch.Tensor | None = None) -> torch.Tensor:
        """Run the distortion and allocator kernels over every row; returns the target ladder index
        (rows, nb) int32 ON THE DEVICE (nothing is read back here)."""
        from .policies import ladder_bits
        nb, dev, rows, D = self.nb, self.device, self.rows, self.D
        offs, level = self.offs[:, :nb].contiguous(), self.level[:, :nb].contiguous()
        E = torch.empty(rows, nb, 5, dtype=torch.float32, device=dev)
        m = (self.mass[:, :nb] if mass is None else mass).contiguous()
        idx = ((level <= 8).to(torch.int32) + (level <= 4).to(torch.int32) + (level <= 2).to(torch.int32)
               + (level <= 1).to(torch.int32)).contiguous()
        hot = self.hot_blocks(nb, sinks, window)
        nb_of = ((self.lens + (BLOCK - 1)) // BLOCK).to(torch.int32).contiguous()
        target = (nb_of.to(torch.float64) * (budget_bits * 2.0 * BLOCK * D)).contiguous()
        ratio = torch.empty(rows, nb, 4, dtype=torch.float32, device=dev)
        tgt = torch.empty(rows, nb, dtype=torch.int32, device=dev)
        bits = (C.c_float * 5)(*ladder_bits(BLOCK, D, self.group))
        with torch.cuda.device(dev):
            rc = self.lib.gkv_block_distortion(self.pool.data.data_ptr(), offs.data_ptr(), level.data_ptr(), E.data_ptr(),
                                               rows, nb, D, BLOCK, self.group, float(value_weight), 0, rows, _stream(dev))
            _lib.check(rc, "gkv_block_distortion")
            rc = self.lib.gkv_allocate_ragged(m.data_ptr(), E.data_ptr(), idx.data_ptr(), hot.data_ptr(), bits,
                                              target.data_ptr(), float(mass_power), ratio.data_ptr(), tgt.data_ptr(),
                                              nb_of.data_ptr(), rows, nb, _stream(dev))
            _lib.check(rc, "gkv_allocate_ragged")
        return tgt

    def apply_demotion(self, tgt_idx_host: np.ndarray) -> int:
        """Demote to the allocator's result (host array (rows, nb) of ladder indices): allocate the
        smaller slots, re-quantise on the device, free the larger slots.  Returns blocks demoted."""
        nb = tgt_idx_host.shape[1]
        cur = self.level_h[:, :nb]
        new = _LADDER_NP[np.clip(tgt_idx_host, 0, 4)]
        used = np.arange(nb)[None, :] < self._row_blocks()[:, None]
        r, b = np.nonzero((new < cur) & used & (self.offs_h[:, :nb] >= 0))
        n = int(r.size)
        if n == 0:
            return 0
        lv_old, lv_new = cur[r, b].copy(), new[r, b].astype(np.int32)
        off_old = self.offs_h[r, b].copy()
        off_new = np.empty(n, dtype=np.int64)
        for rung in LADDER[1:]:
            sel = np.nonzero(lv_new == rung)[0]
            if sel.size:
                off_new[sel] = self.pool.alloc(rung, sel.size)
        dev = self.device
        up = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a)).to(dev, non_blocking=True).to(dt)
        oo, lo, on, ln = up(off_old, torch.int64), up(lv_old, torch.int32), up(off_new, torch.int64), up(lv_new, torch.int32)
        ek = torch.zeros(n, dtype=torch.float32, device=dev)
        ev = torch.zeros(n, dtype=torch.float32, device=dev)
        pool = self.pool.data
        with torch.cuda.device(dev):
            rc = self.lib.gkv_paged_demote_blocks(pool.data_ptr(), oo.data_ptr(), lo.data_ptr(), pool.data_ptr(),
                                                  on.data_ptr(), ln.data_ptr(), ek.data_ptr(), ev.data_ptr(), n, self.D,
                                                  BLOCK, self.group, _stream(dev))
        _lib.check(rc, "gkv_paged_demote_blocks")
        flat = torch.from_numpy((r * self.cap + b).astype(np.int64)).to(dev, non_blocking=True)
        self.offs.view(-1).index_put_((flat,), on)
        self.level.view(-1).index_put_((flat,), ln)
        self.ek.view(-1).index_put_((flat,), ek, accumulate=True)
        self.ev.view(-1).index_put_((flat,), ev, accumulate=True)
        self.offs_h[r, b] = off_new
        self.level_h[r, b] = lv_new
        # the old slots are free for whatever is launched after the demotion kernel on this stream
        for rung in LADDER[:-1]:
            sel = np.nonzero(lv_old == rung)[0]
            if sel.size:
                self.pool.free(rung, off_old[sel])
        return n

    def maintain(self, budget_bits: float, **kw) -> int:
        """plan_demotion + one read-back + apply_demotion for this layer alone."""
        if budget_bits <= 0 or self.nb == 0:
            return 0
        return self.apply_demotion(self.plan_demotion(budget_bits, **kw).cpu().numpy())

    # -- accounting / debugging -----------------------------------------------------------------
    def bytes_in_pool(self) -> int:
        used = np.arange(self.cap)[None, :] < self._row_blocks()[:, None]
        lv = self.level_h[used]
        return int(sum(int((lv == r).sum()) * self.pool.slot[r] for r in LADDER))

    def bits_per_value(self) -> float:
        """Resident bits per cached value with the reference's accounting (policies.py:1582-1596)."""
        from .policies import ladder_bits
        used = np.arange(self.cap)[None, :] < self._row_blocks()[:, None]
        bits = np.array(ladder_bits(BLOCK, self.D, self.group))[ladder_index_np(self.level_h[used])]
        return float(bits.sum()) / max(1, int(used.sum()) * 2 * BLOCK * self.D)

    def release(self) -> None:
        """Give every slot back to the pool."""
        used = np.arange(self.cap)[None, :] < self._row_blocks()[:, None]
        for rung in LADDER:
            sel = used & (self.level_h == rung) & (self.offs_h >= 0)
            if sel.any():
                self.pool.free(rung, self.offs_h[sel])
        self.offs_h[:] = -1
        self.level_h[:] = 0
        self.len_h[:] = 0
        self.offs.fill_(-1)
        self.level.fill_(0)
        self.valid.zero_()
        self.mass.zero_()
        self.lens.zero_()

    def dequantise(self):
        """Exact fp32 K, V (rows, nb*64, D) of the cached tokens (tests, debugging); padding is zero."""
        nb, dev = self.nb, self.device
        k = torch.zeros(self.rows, nb, BLOCK, self.D, dtype=torch.float32, device=dev)
        v = torch.zeros_like(k)
        offs, level = self.offs[:, :nb].contiguous(), self.level[:, :nb].contiguous()
        with torch.cuda.device(dev):
            rc = self.lib.gkv_paged_unpack_blocks(self.pool.data.data_ptr(), offs.data_ptr(), level.data_ptr(),
                                                  k.data_ptr(), v.data_ptr(), self.rows * nb, self.D, BLOCK, self.group,
                                                  _stream(dev))
        _lib.check(rc, "gkv_paged_unpack_blocks")
        return k.view(self.rows, nb * BLOCK, self.D), v.view(self.rows, nb * BLOCK, self.D)
