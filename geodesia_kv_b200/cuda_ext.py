"""Loader and Python face of the decode-attention kernel.

Mirrors ``geodesia_kv/cuda_ext.py`` of the reference: ``get_ext()`` returns an
object whose ``mixed_attn_decode`` has the reference's signature
(geodesia_kv/cuda_ext.py:60-83, geodesia_kv_cuda/binding.cpp:3-13).  Instead of
JIT-compiling a torch extension it binds the prebuilt C-ABI library.

Differences a caller can rely on:
* ``get_ext()`` returns ``None`` only where the reference would — when
  ``GEODESIA_DISABLE_CUDA`` is set or the process has no CUDA device.  On a
  machine with a GPU a missing or broken library raises; nothing falls back to
  the CPU.
* GQA: ``data`` and the scale planes may have fewer heads than ``q``
  (``Hkv = data.size(1)`` dividing ``Hq = q.size(1)``); each cache row is read
  once for its whole group.  The reference needs the bytes replicated per query
  head, which still works (``Hkv == Hq``).
* ``offs`` / ``level`` / ``valid`` may be ``(B, Hkv, nb)`` to give each cache row
  its own rungs; ``(nb,)`` is the reference's shared form.
* Nothing is allocated per call in steady state: the scratch buffer is kept per
  (device, stream), and the rung-sorted block lists the kernel walks are kept per
  metadata triple and rebuilt only when ``offs`` / ``level`` / ``valid`` are other
  tensors or have been written to since (torch's version counters).  Code that
  writes those tensors through raw pointers calls ``invalidate_plans()``.
"""
from __future__ import annotations

import os
from collections import OrderedDict
from typing import Any, Optional

import torch

from . import _lib

_EXT: Any = None
_TRIED = False


def _ptr(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None or t.numel() == 0 else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class _Extension:
    """Stand-in for the reference's pybind module."""

    PLAN_CACHE_ENTRIES = 256

    def __init__(self) -> None:
        self.lib = _lib.load()
        self._plans: "OrderedDict[tuple, tuple]" = OrderedDict()
        self._workspaces: dict = {}

    # -- kernel choice (tensor-core kernel by shape, or always the CUDA-core kernel) ------
    def set_decode_kernel(self, which: str) -> None:
        _lib.check(self.lib.gkv_set_decode_kernel({"auto": 0, "generic": 1}[which]), "gkv_set_decode_kernel")

    def set_decode_item_blocks(self, blocks: int) -> None:
        """Blocks per work item of the tensor-core kernel (0 = chosen from the problem size)."""
        _lib.check(self.lib.gkv_set_decode_item_blocks(int(blocks)), "gkv_set_decode_item_blocks")

    def decode_status(self, device=None) -> int:
        """Status word of the last decode on the current stream of ``device`` (0 = normal; non-zero
        = a wait inside the kernel ran out and the output was filled with NaN).  Synchronises."""
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        ws = self._workspaces.get((dev.index, _stream(dev)))
        if ws is None:
            return 0
        import ctypes
        word = ctypes.c_int(0)
        with torch.cuda.device(dev):
            _lib.check(self.lib.gkv_decode_status(ws.data_ptr(), ctypes.byref(word), _stream(dev)), "gkv_decode_status")
        return int(word.value)

    # -- per-stream scratch and per-metadata block lists ------------------------------------
    def _workspace(self, dev, need: int) -> torch.Tensor:
        if torch.cuda.is_current_stream_capturing():
            return torch.empty(need, dtype=torch.uint8, device=dev)        # lives in the graph's own pool
        key = (dev.index, _stream(dev))
        ws = self._workspaces.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=dev)
            self._workspaces[key] = ws
        return ws

    def invalidate_plans(self) -> None:
        self._plans.clear()

    def _plan(self, offs, level, valid, meta_rows: int, nb: int):
        if nb == 0:
            return None
        key = (offs.data_ptr(), offs._version, level.data_ptr(), level._version, valid.data_ptr(), valid._version,
               meta_rows, nb)
        hit = self._plans.get(key)
        if hit is not None:
            # also while a CUDA graph is being captured: the graph then replays over the lists made for the
            # metadata as it stood at capture (whoever edits level/valid/offs in place captures again)
            self._plans.move_to_end(key)
            return hit[0]
        if torch.cuda.is_current_stream_capturing():
            return None                                                    # built inside the workspace by the call
        plan = torch.empty(self.lib.gkv_decode_plan_bytes(meta_rows, nb), dtype=torch.uint8, device=level.device)
        rc = self.lib.gkv_decode_build_plan(offs.data_ptr(), level.data_ptr(), valid.data_ptr(), plan.data_ptr(),
                                            meta_rows, nb, _stream(level.device))
        _lib.check(rc, "gkv_decode_build_plan")
        # the entry keeps the metadata tensors alive, so their addresses cannot be handed to other tensors
        self._plans[key] = (plan, offs, level, valid)
        while len(self._plans) > self.PLAN_CACHE_ENTRIES:
            self._plans.popitem(last=False)
        return plan

    # -- the reference entry point ------------------------------------------------
    def mixed_attn_decode(self, q, data, offs, klo, kstep, vlo, vstep, level, valid, block, group):
        out, _ = self._decode(q, data, offs, klo, kstep, vlo, vstep, level, valid, block, group, partial=False)
        return out

    # -- un-normalised (m, l, o) record per query head, for sequence-split decode ---
    def mixed_attn_decode_partial(self, q, data, offs, klo, kstep, vlo, vstep, level, valid, block, group):
        out, _ = self._decode(q, data, offs, klo, kstep, vlo, vstep, level, valid, block, group, partial=True)
        return out

    def mixed_attn_decode_with_mass(self, q, data, offs, klo, kstep, vlo, vstep, level, valid, block, group):
        """Attention output (B, Hq, D) and, as a by-product of the same kernel, the softmax mass of every
        block (B, Hkv, nb): mean over the cache row's query heads of the block's summed softmax weight."""
        return self._decode(q, data, offs, klo, kstep, vlo, vstep, level, valid, block, group, partial=False,
                            mass=True)

    def combine_partials(self, partials: torch.Tensor) -> torch.Tensor:
        """(parts, B, Hq, D+2) records -> (B, Hq, D) attention output."""
        if partials.dim() != 4 or partials.dtype != torch.float32 or not partials.is_cuda:
            raise RuntimeError("partials must be a CUDA fp32 tensor (parts, B, Hq, D+2)")
        partials = partials.contiguous()
        parts, B, Hq, D2 = partials.shape
        out = torch.empty(B, Hq, D2 - 2, dtype=torch.float32, device=partials.device)
        with torch.cuda.device(partials.device):
            rc = self.lib.gkv_combine_partials(partials.data_ptr(), out.data_ptr(), parts, B * Hq, D2 - 2,
                                               _stream(partials.device))
        _lib.check(rc, "gkv_combine_partials")
        return out

    def _decode(self, q, data, offs, klo, kstep, vlo, vstep, level, valid, block, group, partial, mass=False):
        if not (q.is_cuda and q.dim() == 3):
            raise RuntimeError("q must be a CUDA tensor of shape (B, H, D)")
        if int(block) != 64:
            raise RuntimeError("only 64-token blocks are supported")
        if q.dtype != torch.float32:
            raise RuntimeError("q must be float32 and already carry the softmax scale")
        B, Hq, D = q.shape
        if data.dim() != 3 or data.dtype != torch.uint8 or data.size(0) != B:
            raise RuntimeError("data must be uint8 of shape (B, Hkv, bytes)")
        Hkv = data.size(1)
        if Hkv == 0 or Hq % Hkv:
            raise RuntimeError(f"q heads ({Hq}) must be a multiple of cache heads ({Hkv})")
        nb = level.shape[-1]
        meta_rows = 1 if level.dim() == 1 else B * Hkv
        if level.dim() != 1 and tuple(level.shape) != (B, Hkv, nb):
            raise RuntimeError("level must be (nb,) or (B, Hkv, nb)")
        if offs.shape != level.shape or valid.shape != level.shape:
            raise RuntimeError("offs, level and valid must have the same shape")
        if offs.dtype != torch.int64 or level.dtype != torch.int32 or valid.dtype != torch.int32:
            raise RuntimeError("offs must be int64, level and valid int32")
        G, gv = (64 + group - 1) // group, (D + group - 1) // group
        for name, t, shp in (("klo", klo, (B, Hkv, nb, G, D)), ("kstep", kstep, (B, Hkv, nb, G, D)),
                             ("vlo", vlo, (B, Hkv, nb, 64, gv)), ("vstep", vstep, (B, Hkv, nb, 64, gv))):
            if t.dtype != torch.float16 or tuple(t.shape) != shp:
                raise RuntimeError(f"{name} must be float16 of shape {shp}, got {t.dtype} {tuple(t.shape)}")
        dev = q.device
        q, data, offs, level, valid = (t.contiguous() for t in (q, data, offs, level, valid))
        klo, kstep, vlo, vstep = (t.contiguous() for t in (klo, kstep, vlo, vstep))
        if mass:
            with torch.cuda.device(dev):
                need = self.lib.gkv_decode_mass_workspace_bytes(B, Hq, Hkv, D, nb, int(group))
                ws = self._workspace(dev, need)
                plan = self._plan(offs, level, valid, meta_rows, nb)
                out = torch.empty((B, Hq, D), dtype=torch.float32, device=dev)
                bm = torch.zeros((B, Hkv, nb), dtype=torch.float32, device=dev)
                rc = 0
                if nb:
                    rc = self.lib.gkv_mixed_attn_decode_mass(
                        q.data_ptr(), _ptr(data), _ptr(offs), _ptr(klo), _ptr(kstep), _ptr(vlo), _ptr(vstep),
                        _ptr(level), _ptr(valid), out.data_ptr(), bm.data_ptr(), _ptr(plan), ws.data_ptr(), ws.numel(),
                        B, Hq, Hkv, D, nb, int(block), int(group), data.size(-1), meta_rows, _stream(dev))
                else:
                    out.zero_()
            _lib.check(rc, "gkv_mixed_attn_decode_mass")
            return out, bm
        with torch.cuda.device(dev):
            need = self.lib.gkv_decode_workspace_bytes(B, Hq, Hkv, D, nb)
            ws = self._workspace(dev, need)
            plan = self._plan(offs, level, valid, meta_rows, nb)
            out = torch.empty((B, Hq, D + 2) if partial else (B, Hq, D), dtype=torch.float32, device=dev)
            rc = self.lib.gkv_mixed_attn_decode_planned(
                q.data_ptr(), _ptr(data), _ptr(offs), _ptr(klo), _ptr(kstep), _ptr(vlo), _ptr(vstep),
                _ptr(level), _ptr(valid), out.data_ptr(), _ptr(plan), 1 if partial else 0, ws.data_ptr(), ws.numel(),
                B, Hq, Hkv, D, nb, int(block), int(group), data.size(-1), meta_rows, _stream(dev))
        _lib.check(rc, "gkv_mixed_attn_decode")
        return out, ws


def get_ext() -> Any:
    """The kernel module, or ``None`` when CUDA is disabled or absent (as the reference does)."""
    global _EXT, _TRIED
    if _TRIED:
        return _EXT
    _TRIED = True
    if os.environ.get("GEODESIA_DISABLE_CUDA"):
        return None
    if not torch.cuda.is_available():
        return None
    _EXT = _Extension()          # raises if the library is missing: no silent fallback
    return _EXT


def mixed_attn_decode(q, data, offs, klo, kstep, vlo, vstep, level, valid, block=64, group=32):
    """Module-level form of the kernel call; raises if no CUDA device is usable."""
    ext = get_ext()
    if ext is None:
        raise RuntimeError("geodesia_kv_b200: CUDA is disabled or no device is present; there is no CPU path")
    return ext.mixed_attn_decode(q, data, offs, klo, kstep, vlo, vstep, level, valid, block, group)
