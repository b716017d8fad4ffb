"""Sub-byte packing and the grouped-by-rung container ("format A").

Mirrors ``geodesia_kv/packed.py`` of the reference: same names, arguments and
return types.  ``pack_bits`` / ``unpack_bits`` (packed.py:23-49) define the
little-endian-in-byte code layout that the decode kernel reads.  ``PackedBlocks``
/ ``PackedKV`` / ``build_packed`` (packed.py:52-157) are the container the vLLM
manager stores; no attention kernel consumes it, it exists for ``nbytes()`` and
``dequantize()``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

_CODE_BITS = (2, 4, 8)


def pack_bits(q: torch.Tensor, bits: int) -> torch.Tensor:
    """Pack integers in [0, 2^bits) along the last dim: value i of a byte at bit i*bits."""
    assert bits in _CODE_BITS, f"unsupported bits: {bits}"
    if bits == 8:
        return q.contiguous()
    per = 8 // bits
    tail = (-q.shape[-1]) % per
    if tail:
        q = torch.nn.functional.pad(q, (0, tail))
    lanes = q.reshape(*q.shape[:-1], q.shape[-1] // per, per).to(torch.int32) & ((1 << bits) - 1)
    shifts = torch.arange(per, device=q.device, dtype=torch.int32) * bits
    return (lanes << shifts).sum(-1).to(torch.uint8)


def unpack_bits(p: torch.Tensor, bits: int, n: int) -> torch.Tensor:
    """Inverse of :func:`pack_bits`; ``n`` is the number of original values."""
    if bits == 8:
        return p[..., :n]
    per = 8 // bits
    shifts = torch.arange(per, device=p.device, dtype=torch.int32) * bits
    lanes = (p.to(torch.int32).unsqueeze(-1) >> shifts) & ((1 << bits) - 1)
    return lanes.to(torch.uint8).reshape(*p.shape[:-1], p.shape[-1] * per)[..., :n]


@dataclass
class PackedBlocks:
    """Blocks quantised at one bit width with per-group fp16 scales (packed.py:52-73)."""
    bits: int
    data: torch.Tensor
    lo: torch.Tensor
    step: torch.Tensor
    shape: tuple
    group: int
    per_channel: bool

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.data, self.lo, self.step))

    def dequantize(self) -> torch.Tensor:
        # Both K and V blocks are viewed as (nb, P/g, g, D) here, exactly as the reference's
        # dequantize does (packed.py:67-73); V scales therefore broadcast over channels.
        nb, p, d = self.shape
        g = min(self.group, p)
        codes = unpack_bits(self.data.reshape(-1), self.bits, nb * p * d).float()
        return (codes.reshape(nb, p // g, g, d) * self.step + self.lo).reshape(nb, p, d)


def quantize_packed(x: torch.Tensor, bits: int, group: int, per_channel: bool) -> PackedBlocks:
    """x (nb, P, D) -> packed codes; codes are taken against the fp32 scales, which are then
    stored as fp16 (packed.py:76-91)."""
    nb, p, d = x.shape
    g = min(group, p)
    xs = x.reshape(nb, p // g, g, d).float()
    axis = 2 if per_channel else 3
    lo = xs.amin(axis, keepdim=True)
    step = (xs.amax(axis, keepdim=True) - lo).clamp_min(1e-8) / (2 ** bits - 1)
    codes = ((xs - lo) / step).round().clamp_(0, 2 ** bits - 1).to(torch.uint8)
    return PackedBlocks(bits=bits, data=pack_bits(codes.reshape(-1), bits), lo=lo.to(torch.float16),
                        step=step.to(torch.float16), shape=(nb, p, d), group=g, per_channel=per_channel)


@dataclass
class PackedKV:
    """One layer's cache with mixed residency (packed.py:94-113)."""
    exact_k: torch.Tensor | None = None
    exact_v: torch.Tensor | None = None
    exact_idx: torch.Tensor | None = None
    quant: list = field(default_factory=list)      # [(idx, PackedBlocks K, PackedBlocks V)]
    cent_k: torch.Tensor | None = None
    cent_v: torch.Tensor | None = None
    cent_idx: torch.Tensor | None = None

    def nbytes(self) -> int:
        dense = (self.exact_k, self.exact_v, self.cent_k, self.cent_v, self.exact_idx, self.cent_idx)
        total = sum(t.numel() * t.element_size() for t in dense if t is not None)
        return total + sum(pk.nbytes() + pv.nbytes() for _, pk, pv in self.quant)


def build_packed(k: torch.Tensor, v: torch.Tensor, bits: torch.Tensor, centroid: torch.Tensor,
                 block: int, group: int) -> PackedKV:
    """k, v (T, D); bits (nb,) per block; centroid (nb,) bool mask (packed.py:116-157)."""
    from .policies import blockify
    kb, _ = blockify(k, block)
    vb, _ = blockify(v, block)
    out = PackedKV()

    def pick(mask):
        return mask.nonzero(as_tuple=True)[0]

    if centroid.any():
        idx = pick(centroid)
        out.cent_k = kb[idx].mean(1).to(torch.bfloat16).contiguous()
        out.cent_v = vb[idx].mean(1).to(torch.bfloat16).contiguous()
        out.cent_idx = idx.to(torch.int32)
    exact = ~centroid & (bits >= 16)
    if exact.any():
        idx = pick(exact)
        out.exact_k = kb[idx].to(torch.bfloat16).contiguous()
        out.exact_v = vb[idx].to(torch.bfloat16).contiguous()
        out.exact_idx = idx.to(torch.int32)
    todo = ~centroid & (bits < 16)
    known = torch.zeros_like(todo)
    for b in _CODE_BITS:
        sel = todo & (bits == b)
        known |= sel
        if sel.any():
            idx = pick(sel)
            out.quant.append((idx.to(torch.int32), quantize_packed(kb[idx], b, group, True),
                              quantize_packed(vb[idx], b, group, False)))
    odd = todo & ~known                    # widths off the ladder are stored at 8 bits
    if odd.any():
        idx = pick(odd)
        out.quant.append((idx.to(torch.int32), quantize_packed(kb[idx], 8, group, True),
                          quantize_packed(vb[idx], 8, group, False)))
    return out
