"""Alias package: the reference's import names on top of ``geodesia_kv_b200``.

``import geodesia_kv.cuda_ext`` (``pack_layout``, ``packed``, ``policies``, ``vllm_plugin``)
resolves to the module of the same name in ``geodesia_kv_b200``, so code written against the
reference package runs unchanged.
"""
import importlib
import sys

import geodesia_kv_b200 as _impl

__version__ = _impl.__version__
__all__ = ["policies", "packed", "pack_layout", "cuda_ext"]

for _name in ("cuda_ext", "pack_layout", "packed", "policies", "vllm_plugin", "vllm_plugin.kv_cache",
              "vllm_plugin.vllm_connector", "vllm_plugin.attention_backend"):
    _mod = importlib.import_module(f"geodesia_kv_b200.{_name}")
    sys.modules[f"geodesia_kv.{_name}"] = _mod
    if "." not in _name:
        globals()[_name] = _mod
