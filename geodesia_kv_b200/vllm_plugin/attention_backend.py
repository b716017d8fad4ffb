"""Attention-layer wrapper named as in the reference (attention_backend.py:14-36).  Like the
reference's it forwards to the wrapped layer; the manager it carries owns the packed caches."""
from __future__ import annotations

import torch.nn as nn

from .kv_cache import GeodesiaKVCacheManager


class GeodesiaAttentionWrapper(nn.Module):
    def __init__(self, orig_attn: nn.Module, layer_idx: int, manager: GeodesiaKVCacheManager):
        super().__init__()
        self.orig_attn = orig_attn
        self.layer_idx = layer_idx
        self.manager = manager

    def forward(self, query, key, value, kv_cache=None, attn_metadata=None, **kwargs):
        return self.orig_attn(query, key, value, kv_cache=kv_cache, attn_metadata=attn_metadata, **kwargs)
