"""vLLM-facing names of the reference (geodesia_kv/vllm_plugin/__init__.py)."""
from .kv_cache import GeodesiaBlockCache, GeodesiaKVCacheManager
from .vllm_connector import register_geodesia_kv_plugin

__all__ = ["GeodesiaKVCacheManager", "GeodesiaBlockCache", "register_geodesia_kv_plugin"]
