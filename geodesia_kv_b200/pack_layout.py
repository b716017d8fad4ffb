"""The byte layout the decode kernel reads, and its builders.

``build_layout`` mirrors ``geodesia_kv/pack_layout.py:14-54`` of the reference
(same arguments, same dict, byte-identical output) and, like it, works on any
torch device.  ``pack_cache`` is the batched device builder: dense K/V of every
cache row go through the CUDA pack kernel and come out as the same bytes, for
all rows at once, with no per-block Python.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from .packed import pack_bits

BLOCK = 64
LADDER = (16, 8, 4, 2, 1)


def block_nbytes(level: int, D: int, block: int = BLOCK) -> int:
    """Bytes of one packed block (K and V) at a rung."""
    half = D * 2 if level == 1 else block * D * 2 if level == 16 else block * D * level // 8
    return 2 * half


def build_layout(krec_q: dict, block: int, group: int, D: int, nb: int, levels: torch.Tensor,
                 valid: torch.Tensor, device):
    """Assemble (data, offs, klo, kstep, vlo, vstep) for ONE cache row.

    ``krec_q[b]`` holds ``{"k", "v"}`` — (P, D) values for rung 16, (1, D) centroids for rung 1,
    (P, D) integer codes plus ``klo, kstep`` (G, D) and ``vlo, vstep`` (P, gv) otherwise.
    """
    G, gv = (block + group - 1) // group, (D + group - 1) // group
    planes = {name: torch.zeros(nb, *shape, dtype=torch.float16, device=device)
              for name, shape in (("klo", (G, D)), ("kstep", (G, D)), ("vlo", (block, gv)), ("vstep", (block, gv)))}
    pieces, starts, cursor = [], [], 0
    for b in range(nb):
        rung, item = int(levels[b]), krec_q[b]
        if rung in (1, 16):
            store = torch.float16 if rung == 1 else torch.bfloat16
            halves = [item[key].reshape(-1).to(store).view(torch.uint8) for key in ("k", "v")]
        else:
            halves = [pack_bits(item[key].reshape(-1).to(torch.uint8), rung) for key in ("k", "v")]
            for name in planes:
                planes[name][b] = item[name]
        starts.append(cursor)
        for h in halves:
            pieces.append(h)
            cursor += h.numel()
    data = torch.cat(pieces) if pieces else torch.zeros(0, dtype=torch.uint8, device=device)
    scale_bytes = 2 * 2 * (planes["klo"].numel() + planes["vlo"].numel())
    return {"data": data, "offs": torch.tensor(starts, dtype=torch.long, device=device), **planes,
            "level": levels.to(torch.int32), "valid": valid.to(torch.int32),
            "nbytes": int(data.numel() + scale_bytes)}


@dataclass
class PackedCache:
    """Packed cache of one layer for B sequences x Hkv heads, in the kernel's layout."""
    data: torch.Tensor      # (B, Hkv, stride) uint8
    offs: torch.Tensor      # (B, Hkv, nb) int64
    klo: torch.Tensor       # (B, Hkv, nb, G, D) fp16
    kstep: torch.Tensor
    vlo: torch.Tensor       # (B, Hkv, nb, 64, gv) fp16
    vstep: torch.Tensor
    level: torch.Tensor     # (B, Hkv, nb) int32
    valid: torch.Tensor     # (B, Hkv, nb) int32
    group: int
    D: int

    @property
    def nb(self) -> int:
        return self.level.shape[-1]

    def kernel_args(self):
        return (self.data, self.offs, self.klo, self.kstep, self.vlo, self.vstep, self.level, self.valid,
                BLOCK, self.group)

    def algorithmic_bytes(self) -> int:
        """Bytes a decode step must read: block bytes + scale planes of quantised blocks
        + 16 B of metadata per block."""
        lv = self.level
        G, gv = self.klo.shape[-2], self.vlo.shape[-1]
        sizes = torch.zeros_like(lv, dtype=torch.int64)
        for rung in LADDER:
            sizes += (lv == rung).to(torch.int64) * block_nbytes(rung, self.D)
        quant = ((lv == 8) | (lv == 4) | (lv == 2)).to(torch.int64)
        scale = 4 * (G * self.D + BLOCK * gv)
        return int(sizes.sum() + quant.sum() * scale + lv.numel() * 16)


def layout_offsets(level: torch.Tensor, D: int, align: int = 1):
    """Contiguous block placement for rungs ``level`` (..., nb): (offs int64, bytes per row)."""
    sizes = torch.zeros_like(level, dtype=torch.int64)
    for rung in LADDER:
        sizes += (level == rung).to(torch.int64) * block_nbytes(rung, D)
    if align > 1:
        sizes = (sizes + align - 1) // align * align
    ends = sizes.cumsum(-1)
    return ends - sizes, ends[..., -1] if level.shape[-1] else ends.sum(-1)


def pack_cache(k: torch.Tensor, v: torch.Tensor, level: torch.Tensor, group: int = 32,
               valid: torch.Tensor | None = None) -> PackedCache:
    """Pack dense K, V (B, Hkv, T, D) on the GPU at per-block rungs ``level`` (B, Hkv, nb).

    T must fill ``nb`` blocks except for a ragged tail, which is given through ``valid``
    (defaults to all 64 with a short last block when T is not a multiple of 64).
    """
    if not k.is_cuda:
        raise RuntimeError("pack_cache packs on the GPU; there is no CPU path")
    B, Hkv, T, D = k.shape
    nb = (T + BLOCK - 1) // BLOCK
    level = level.to(device=k.device, dtype=torch.int32).expand(B, Hkv, nb).contiguous()
    if valid is None:
        valid = torch.full((B, Hkv, nb), BLOCK, dtype=torch.int32, device=k.device)
        if T % BLOCK:
            valid[..., -1] = T % BLOCK
    valid = valid.to(device=k.device, dtype=torch.int32).expand(B, Hkv, nb).contiguous()
    if T != nb * BLOCK:                       # the kernel indexes whole blocks
        pad = nb * BLOCK - T
        k = torch.nn.functional.pad(k, (0, 0, 0, pad))
        v = torch.nn.functional.pad(v, (0, 0, 0, pad))
    dt = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[k.dtype]
    k, v = k.contiguous(), v.contiguous()
    offs, row_bytes = layout_offsets(level, D)
    stride = int(row_bytes.max().item()) if nb else 0
    stride = (stride + 255) // 256 * 256
    G, gv = (BLOCK + group - 1) // group, (D + group - 1) // group
    dev = k.device
    data = torch.zeros(B, Hkv, stride, dtype=torch.uint8, device=dev)
    planes = [torch.empty(B, Hkv, nb, *s, dtype=torch.float16, device=dev)
              for s in ((G, D), (G, D), (BLOCK, gv), (BLOCK, gv))]
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.gkv_pack_blocks(k.data_ptr(), v.data_ptr(), dt, data.data_ptr(), offs.data_ptr(),
                                 *(p.data_ptr() for p in planes), level.data_ptr(), valid.data_ptr(),
                                 B * Hkv, nb, 0, nb, D, BLOCK, group, stride, B * Hkv,
                                 torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "gkv_pack_blocks")
    return PackedCache(data, offs, *planes, level, valid, group, D)


def unpack_cache(c: PackedCache):
    """Exact dequantisation of a packed cache -> fp32 K, V (B, Hkv, nb*64, D) (tests, debugging)."""
    B, Hkv, nb = c.level.shape
    dev = c.data.device
    k = torch.empty(B, Hkv, nb * BLOCK, c.D, dtype=torch.float32, device=dev)
    v = torch.empty_like(k)
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.gkv_unpack_blocks(c.data.data_ptr(), c.offs.data_ptr(), c.klo.data_ptr(), c.kstep.data_ptr(),
                                   c.vlo.data_ptr(), c.vstep.data_ptr(), c.level.data_ptr(), k.data_ptr(),
                                   v.data_ptr(), B * Hkv, nb, c.D, BLOCK, c.group, c.data.size(-1), B * Hkv,
                                   torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "gkv_unpack_blocks")
    return k, v
