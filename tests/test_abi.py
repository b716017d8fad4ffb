"""The C-ABI library: builds for sm_100a, loads, and exports exactly what the header declares."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "geodesia_kv_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gkv_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    from geodesia_kv_b200 import _lib, build
    so = build.build()
    assert so.exists()
    lib = ctypes.CDLL(str(so))
    names = declared_functions()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes signatures out of step with the header"


def test_host_only_calls_need_no_gpu():
    from geodesia_kv_b200 import _lib
    lib = _lib.load()
    assert lib.gkv_abi_version() == 1
    assert lib.gkv_error_string(-1) == b"only 64-token blocks are supported"
    assert lib.gkv_error_string(0) == b"ok"
    need = lib.gkv_decode_workspace_bytes(32, 32, 8, 128, 256)
    assert need > 0 and need % 256 == 0
    assert lib.gkv_decode_workspace_bytes(0, 1, 1, 128, 1) == 0
    assert lib.gkv_decode_kernel_launches(32, 32, 8, 128, 256, 32) == 3       # block lists, split kernel, one merge
    assert lib.gkv_decode_kernel_launches(1, 28, 4, 128, 16384, 32) == 4      # long rows: two merge levels
    assert lib.gkv_decode_kernel_launches(1, 4, 4, 96, 8, 32) == 2            # generic kernel + merge


def test_argument_validation_happens_before_any_cuda_call():
    from geodesia_kv_b200 import _lib
    lib = _lib.load()
    one = ctypes.c_void_p(256)      # never dereferenced: validation rejects the call first
    args = [one] * 10 + [one, 1 << 20]
    assert lib.gkv_mixed_attn_decode(*args, 1, 4, 4, 64, 8, 32, 32, 1024, 1, None) == -1      # block != 64
    assert lib.gkv_mixed_attn_decode(*args, 1, 5, 4, 64, 8, 64, 32, 1024, 1, None) == -2      # 5 % 4
    assert lib.gkv_mixed_attn_decode(*args, 1, 4, 4, 60, 8, 64, 32, 1024, 1, None) == -2      # D % 8
    assert lib.gkv_mixed_attn_decode(*args, 1, 4, 4, 64, 8, 64, 32, 1024, 3, None) == -2      # meta rows
    nul = [None] + [one] * 9 + [one, 1 << 20]
    assert lib.gkv_mixed_attn_decode(*nul, 1, 4, 4, 64, 8, 64, 32, 1024, 1, None) == -3
    small = [one] * 10 + [one, 16]
    assert lib.gkv_mixed_attn_decode(*small, 1, 4, 4, 64, 8, 64, 32, 1024, 1, None) == -4


def test_get_ext_follows_the_reference_contract(monkeypatch):
    import torch
    from geodesia_kv_b200 import cuda_ext
    monkeypatch.setattr(cuda_ext, "_TRIED", False)
    monkeypatch.setattr(cuda_ext, "_EXT", None)
    monkeypatch.setenv("GEODESIA_DISABLE_CUDA", "1")
    assert cuda_ext.get_ext() is None            # geodesia_kv/cuda_ext.py:66
    if not torch.cuda.is_available():
        import pytest
        with pytest.raises(RuntimeError, match="no CPU path"):
            cuda_ext.mixed_attn_decode(*([None] * 9))
