"""ctypes binding of ``libgeodesia_kv_b200.so`` (the C ABI in ``include/geodesia_kv_b200.h``).

There is no CPU fallback anywhere in this package: if the library cannot be
loaded the import of the first kernel entry point raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libgeodesia_kv_b200.so"

_lib = None

_vp, _i, _i64, _sz, _f = C.c_void_p, C.c_int, C.c_int64, C.c_size_t, C.c_float

# name -> (restype, argtypes); mirrors include/geodesia_kv_b200.h one to one
SIGNATURES = {
    "gkv_abi_version": (_i, []),
    "gkv_error_string": (C.c_char_p, [_i]),
    "gkv_last_cuda_error": (_i, []),
    "gkv_decode_workspace_bytes": (_sz, [_i] * 5),
    "gkv_decode_kernel_launches": (_i, [_i] * 6),
    "gkv_decode_launch_count": (_i, [_i] * 7),
    "gkv_set_decode_kernel": (_i, [_i]),
    "gkv_set_decode_item_blocks": (_i, [_i]),
    "gkv_decode_status": (_i, [_vp, C.POINTER(_i), _vp]),
    "gkv_decode_plan_bytes": (_sz, [_i, _i]),
    "gkv_decode_build_plan": (_i, [_vp] * 4 + [_i, _i, _vp]),
    "gkv_mixed_attn_decode_planned": (_i, [_vp] * 10 + [_vp, _i, _vp, _sz] + [_i] * 7 + [_i64, _i, _vp]),
    "gkv_mixed_attn_decode": (_i, [_vp] * 10 + [_vp, _sz] + [_i] * 7 + [_i64, _i, _vp]),
    "gkv_mixed_attn_decode_partial": (_i, [_vp] * 10 + [_vp, _sz] + [_i] * 7 + [_i64, _i, _vp]),
    "gkv_mixed_attn_decode_static": (_i, [_vp] * 10 + [_i] * 7 + [_i64, _i, _vp]),
    "gkv_decode_mass_workspace_bytes": (_sz, [_i] * 6),
    "gkv_mixed_attn_decode_mass": (_i, [_vp] * 10 + [_vp, _vp, _vp, _sz] + [_i] * 7 + [_i64, _i, _vp]),
    "gkv_exchange_inbox_bytes": (_sz, [_i, _i, _i]),
    "gkv_set_exchange_wait_ns": (_i, [C.c_ulonglong]),
    "gkv_mixed_attn_decode_exchange": (_i, [_vp] * 10 + [_vp, _vp, _sz] + [_i] * 7 + [_i64, _i] +
                                       [C.POINTER(_vp), _i, _i, _vp, _vp, _vp]),
    "gkv_combine_partials": (_i, [_vp, _vp, _i, _i, _i, _vp]),
    "gkv_pack_blocks": (_i, [_vp, _vp, _i, _vp, _vp] + [_vp] * 4 + [_vp, _vp] + [_i] * 7 + [_i64, _i, _vp]),
    "gkv_demote_blocks": (_i, [_vp] * 6 + [_vp] * 4 + [_i] * 5 + [_i64, _i64, _i, _vp]),
    "gkv_unpack_blocks": (_i, [_vp] * 7 + [_vp, _vp] + [_i] * 5 + [_i64, _i, _vp]),
    "gkv_maintenance_status": (_i, [C.POINTER(_i)]),
    "gkv_paged_block_bytes": (_sz, [_i, _i, _i]),
    "gkv_paged_pack_blocks": (_i, [_vp, _vp, _i, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _vp] + [_i] * 4 + [_vp]),
    "gkv_paged_demote_blocks": (_i, [_vp] * 8 + [_i] * 4 + [_vp]),
    "gkv_paged_unpack_blocks": (_i, [_vp] * 5 + [_i] * 4 + [_vp]),
    "gkv_paged_append_token": (_i, [_vp, _vp, _i] + [_vp] * 5 + [_i] * 4 + [_vp]),
    "gkv_paged_attn_decode": (_i, [_vp, _vp, _sz, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _sz] + [_i] * 7 + [_vp]),
    "gkv_allocate_ragged": (_i, [_vp] * 4 + [C.POINTER(_f), _vp, _f, _vp, _vp, _vp, _i, _i, _vp]),
    "gkv_allocate": (_i, [_vp] * 4 + [C.POINTER(_f), _vp, _f, _vp, _vp, _i, _i, _vp]),
    "gkv_block_distortion": (_i, [_vp] * 4 + [_i] * 5 + [_f, _i64, _i, _vp]),
}


class GkvError(RuntimeError):
    pass


def bind(path) -> C.CDLL:
    """Open a build of the library and attach the signatures of the header to it."""
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here = header and library disagree
        fn.restype, fn.argtypes = res, args
    return lib


def load():
    """Return the ctypes library, compiling it first when it is missing or was built from other
    sources than the ones in the tree (compared by content, so a copied tree is not rebuilt)."""
    global _lib
    if _lib is not None:
        return _lib
    import os
    path = Path(os.environ.get("GKV_LIBRARY", LIB_PATH))    # a differently tuned build can be swapped in
    if path == LIB_PATH:
        from . import build as _build
        _build.build()                   # returns at once when the library matches the sources
    _lib = bind(path)
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        lib = load()
        msg = lib.gkv_error_string(rc).decode()
        if rc == -5:
            msg += f" [cudaError {lib.gkv_last_cuda_error()}]"
        raise GkvError(f"{what}: {msg}")
