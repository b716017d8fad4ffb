"""Per-sequence compressed caches and their manager.

Same names, arguments and return values as ``geodesia_kv/vllm_plugin/kv_cache.py:15-104``.
On a CUDA tensor ``compress_sequence_kv`` also packs every layer into the decode kernel's
layout on the GPU (``kernel_layers``), so the result can be attended over directly; the
format-A containers (``layers``) are kept because the reference's callers read ``nbytes()``.

A manager that has been given a pool (``attach_pool``) additionally stores every sequence it
compresses in ONE paged byte pool with size-class free lists (``paged_layers``: a block table
per layer), so that what a sequence occupies is what its rungs cost and
``free_sequence_cache`` hands exactly those bytes back — the capacity the reference claims for
its plugin (README.md:243-248) but, keeping one Python object per sequence, never reclaims.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..packed import PackedKV, build_packed


@dataclass
class GeodesiaBlockCache:
    block_size: int = 64
    bits_per_value: float = 4.0
    group_size: int = 32
    layers: list[PackedKV] | None = None
    kernel_layers: list | None = None
    pool: object | None = None              # the manager's PagedPool, when it has one
    paged_layers: list | None = None        # PagedLayerCache per layer (block tables over the pool)

    def allocate_bits_for_blocks(self, nb: int, device) -> tuple[torch.Tensor, torch.Tensor]:
        """Threshold ladder of the reference (:23-42): one width for all blocks, last block 16-bit."""
        ladder = 2.0 if self.bits_per_value <= 2.5 else 4.0 if self.bits_per_value <= 4.5 else \
            8.0 if self.bits_per_value <= 8.5 else 16.0
        bits = torch.full((nb,), ladder, device=device, dtype=torch.float32)
        if nb > 0:
            bits[-1] = 16.0
        return bits, torch.zeros((nb,), device=device, dtype=torch.bool)

    def compress_sequence_kv(self, key_cache: torch.Tensor, value_cache: torch.Tensor) -> float:
        """(layers, T, heads, head_dim) dense K, V -> packed blocks; returns achieved bits/value."""
        num_layers, seq_len, num_heads, head_dim = key_cache.shape
        self.release()
        self.layers, self.kernel_layers, self.paged_layers = [], [], []
        total_bytes = 0
        total_values = num_layers * seq_len * num_heads * head_dim * 2
        nb = math.ceil(seq_len / self.block_size)
        for layer in range(num_layers):
            if nb == 0:
                continue
            k = key_cache[layer].reshape(seq_len, num_heads * head_dim)
            v = value_cache[layer].reshape(seq_len, num_heads * head_dim)
            bits, centroid = self.allocate_bits_for_blocks(nb, key_cache.device)
            packed_layer = build_packed(k=k, v=v, bits=bits, centroid=centroid, block=self.block_size,
                                        group=self.group_size)
            self.layers.append(packed_layer)
            total_bytes += packed_layer.nbytes()
            if key_cache.is_cuda and self.block_size == 64 and head_dim % 8 == 0 and head_dim <= 256:
                from ..pack_layout import pack_cache
                kk = key_cache[layer].permute(1, 0, 2).unsqueeze(0).contiguous()      # (1, H, T, Dh)
                vv = value_cache[layer].permute(1, 0, 2).unsqueeze(0).contiguous()
                self.kernel_layers.append(pack_cache(kk, vv, bits.to(torch.int32).view(1, 1, nb), self.group_size))
                if self.pool is not None and self.pool.D == head_dim and self.pool.group == self.group_size:
                    from ..paged import PagedLayerCache, ladder_index_np
                    pl = PagedLayerCache(self.pool, 1, num_heads, cap_blocks=nb + 1)
                    pl.prefill(kk, vv)                                            # exact blocks ...
                    tgt = ladder_index_np(bits.to(torch.int32).cpu().numpy())[None, :].repeat(num_heads, 0)
                    pl.apply_demotion(tgt)                                        # ... shrunk to their rung, the rest freed
                    self.paged_layers.append(pl)
        return (total_bytes * 8) / max(1, total_values)

    def release(self) -> None:
        """Give the pool slots of this sequence back."""
        for pl in self.paged_layers or []:
            pl.release()
        self.paged_layers = None

    def pool_bytes(self) -> int:
        return sum(pl.bytes_in_pool() for pl in self.paged_layers or [])


class GeodesiaKVCacheManager:
    def __init__(self, block_size: int = 64, target_bpv: float = 4.0, num_layers: int = 24):
        self.block_size = block_size
        self.target_bpv = target_bpv
        self.num_layers = num_layers
        self.active_caches: dict[int, GeodesiaBlockCache] = {}
        self.pool = None

    def attach_pool(self, capacity_bytes: int, head_dim: int = 128, group_size: int = 32, device="cuda"):
        """Give the manager ONE paged pool for all its sequences (not in the reference)."""
        from ..paged import PagedPool
        self.pool = PagedPool(capacity_bytes, head_dim, group_size, device)
        return self.pool

    def create_sequence_cache(self, seq_id: int) -> GeodesiaBlockCache:
        cache = GeodesiaBlockCache(block_size=self.block_size, bits_per_value=self.target_bpv, pool=self.pool)
        self.active_caches[seq_id] = cache
        return cache

    def get_cache(self, seq_id: int) -> GeodesiaBlockCache | None:
        return self.active_caches.get(seq_id)

    def free_sequence_cache(self, seq_id: int):
        cache = self.active_caches.pop(seq_id, None)
        if cache is not None:
            cache.release()
