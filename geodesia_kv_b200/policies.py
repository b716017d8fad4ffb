"""Rung allocation and the attention hooks, with the reference's names.

Mirrors the part of ``geodesia_kv/policies.py`` that lies on the packed decode
path: the ladder constants and ``_level_bits`` (:1576-1596), ``blockify``
(:126-133), ``quant_grouped`` (:82-112), the Lagrangian allocator of
``Policy.attend`` (:810-868) and its hot mask (:677-681).  The allocator and the
distortion table run as CUDA kernels over whole batches of cache rows.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

SPECTRAL_LEVEL = 1.5
LEVELS = [16, 8, 4, 2, SPECTRAL_LEVEL, 1]
LADDER = (16, 8, 4, 2, 1)            # the rungs the packed format stores


def _level_bits(level, block: int, D: int, group: int, spectral_rank: int = 0) -> float:
    """Resident bits of one block at a rung, scales included."""
    if level >= 16:
        return 2.0 * block * D * 16.0
    if level == 1:
        return 2.0 * D * 16.0
    if level == SPECTRAL_LEVEL:
        rank = max(0, min(int(spectral_rank), block, D))
        return 2.0 * D * 16.0 * (1 + rank) + rank * 16.0
    token_groups = max(1, block // group)
    channel_groups = max(1, D // group)
    return 2.0 * level * block * D + token_groups * D * 32.0 + block * channel_groups * 32.0


def blockify(x: torch.Tensor, block: int):
    """(T, D) -> (nb, block, D), the tail padded by repeating the last row; returns (blocks, pad)."""
    t, d = x.shape
    nb = (t + block - 1) // block
    pad = nb * block - t
    if pad:
        x = torch.cat([x, x[-1:].expand(pad, -1)], 0)
    return x.view(nb, block, d), pad


def quant_grouped(x: torch.Tensor, bits: int, group: int, per_channel: bool):
    """Grouped min-max quantise -> dequantise of (nb, P, D) with fp32 scales; returns
    (reconstruction, largest step per block)."""
    nb, pp, d = x.shape
    if per_channel:
        g = min(group, pp)
        xs, axis = x.view(nb, pp // g, g, d), 2
    else:
        g = min(group, d)
        xs, axis = x.view(nb, pp, d // g, g), 3
    if bits >= 16:
        shape = (nb, d) if per_channel else (nb,)
        return x, torch.zeros(shape, device=x.device, dtype=x.dtype)
    lo = xs.amin(axis, keepdim=True)
    step = (xs.amax(axis, keepdim=True) - lo).clamp_min(1e-8) / (2 ** bits - 1)
    rec = (((xs - lo) / step).round().clamp_(0, 2 ** bits - 1) * step + lo).view(nb, pp, d)
    return rec, step.amax(dim=(1, 2) if per_channel else (1, 2, 3))


def hot_mask(nb: int, q_offset: int, block: int = 64, sinks: int = 4, window: int = 128,
             device=None) -> torch.Tensor:
    """Blocks that may never be demoted: sinks, the block being written and its
    predecessor, and the recent window (policies.py:677-681)."""
    hot = torch.zeros(nb, dtype=torch.bool, device=device)
    hot[: max(1, (sinks + block - 1) // block)] = True
    hot[max(0, q_offset // block - 1):] = True
    hot[-max(1, (window + block - 1) // block):] = True
    return hot


def ladder_bits(block: int, D: int, group: int) -> list[float]:
    return [_level_bits(L, block, D, group) for L in LADDER]


def allocate_rungs(mass: torch.Tensor, E: torch.Tensor, idx: torch.Tensor, hot: torch.Tensor,
                   budget_bits, block: int, D: int, group: int, mass_power: float = 1.0,
                   return_ratio: bool = False):
    """Target ladder index per block for every cache row at once.

    mass (..., nb) fp32, E (..., nb, 5) fp32, idx (..., nb) current ladder index,
    hot (..., nb) bool, all CUDA; ``budget_bits`` a float or a (...,) tensor of bits/value.
    Returns int32 (..., nb); bit-exact with the reference's allocation for the same inputs.
    """
    if not mass.is_cuda:
        raise RuntimeError("allocate_rungs runs on the GPU; there is no CPU path")
    lead, nb = mass.shape[:-1], mass.shape[-1]
    problems = 1
    for s in lead:
        problems *= s
    dev = mass.device
    mass = mass.to(torch.float32).contiguous()
    E = E.to(torch.float32).contiguous()
    idx = idx.to(torch.int32).contiguous()
    hot = hot.to(torch.uint8).contiguous()
    total_vals = 2.0 * nb * block * D
    target = (torch.as_tensor(budget_bits, dtype=torch.float64, device=dev) * total_vals).expand(lead).contiguous()
    ratio = torch.empty(*lead, nb, 4, dtype=torch.float32, device=dev)
    tgt = torch.empty(*lead, nb, dtype=torch.int32, device=dev)
    bits = (C.c_float * 5)(*ladder_bits(block, D, group))
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.gkv_allocate(mass.data_ptr(), E.data_ptr(), idx.data_ptr(), hot.data_ptr(), bits,
                              target.data_ptr(), float(mass_power), ratio.data_ptr(), tgt.data_ptr(),
                              problems, nb, torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "gkv_allocate")
    return (tgt, ratio) if return_ratio else tgt


def block_distortion(cache, value_weight: float = 0.0) -> torch.Tensor:
    """Distortion table E (B, Hkv, nb, 5) of a :class:`PackedCache`, from its rung-16 blocks."""
    B, Hkv, nb = cache.level.shape
    dev = cache.data.device
    E = torch.empty(B, Hkv, nb, 5, dtype=torch.float32, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.gkv_block_distortion(cache.data.data_ptr(), cache.offs.data_ptr(), cache.level.data_ptr(),
                                      E.data_ptr(), B * Hkv, nb, cache.D, 64, cache.group, float(value_weight),
                                      cache.data.size(-1), B * Hkv, torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "gkv_block_distortion")
    return E
