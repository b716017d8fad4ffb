"""``register_geodesia_kv_plugin`` with the reference's contract (vllm_connector.py:17-43):
builds a manager, attaches it as ``geodesia_manager`` to the LLM (and its engine), returns it."""
from __future__ import annotations

import logging
from typing import Any

from .kv_cache import GeodesiaKVCacheManager

logger = logging.getLogger("geodesia_kv.vllm_plugin")


def register_geodesia_kv_plugin(engine_or_llm: Any, target_bpv: float = 4.0, block_size: int = 64) -> GeodesiaKVCacheManager:
    logger.info("Registering Geodesia-KV plugin with target %s bits-per-value, block_size=%s", target_bpv, block_size)
    manager = GeodesiaKVCacheManager(block_size=block_size, target_bpv=target_bpv)
    object.__setattr__(engine_or_llm, "geodesia_manager", manager)
    engine = getattr(engine_or_llm, "llm_engine", None)
    if engine is not None:
        try:
            object.__setattr__(engine, "geodesia_manager", manager)
        except Exception:            # some engine proxies refuse new attributes; the LLM handle keeps it
            pass
    return manager
