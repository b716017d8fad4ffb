"""B200-native hot path of geodesia-kv: decode attention over a packed bit-ladder KV cache.

The sub-modules keep the reference package's names (``cuda_ext``, ``pack_layout``,
``packed``, ``policies``, ``vllm_plugin``) so that ``import geodesia_kv`` — a thin
alias package at the repository root — drops in for the reference.
"""
__version__ = "0.1.0"
__all__ = ["policies", "packed", "pack_layout", "cuda_ext"]
