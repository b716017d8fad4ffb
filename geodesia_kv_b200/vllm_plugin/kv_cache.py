"""Per-sequence compressed caches and their manager.

Same names, arguments and return values as ``geodesia_kv/vllm_plugin/kv_cache.py:15-104``.
On a CUDA tensor ``compress_sequence_kv`` also packs every layer into the decode kernel's
layout on the GPU (``kernel_layers``), so the result can be attended over directly; the
format-A containers (``layers``) are kept because the reference's callers read ``nbytes()``.
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
        self.layers, self.kernel_layers = [], []
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
        return (total_bytes * 8) / max(1, total_values)


class GeodesiaKVCacheManager:
    def __init__(self, block_size: int = 64, target_bpv: float = 4.0, num_layers: int = 24):
        self.block_size = block_size
        self.target_bpv = target_bpv
        self.num_layers = num_layers
        self.active_caches: dict[int, GeodesiaBlockCache] = {}

    def create_sequence_cache(self, seq_id: int) -> GeodesiaBlockCache:
        cache = GeodesiaBlockCache(block_size=self.block_size, bits_per_value=self.target_bpv)
        self.active_caches[seq_id] = cache
        return cache

    def get_cache(self, seq_id: int) -> GeodesiaBlockCache | None:
        return self.active_caches.get(seq_id)

    def free_sequence_cache(self, seq_id: int):
        self.active_caches.pop(seq_id, None)
