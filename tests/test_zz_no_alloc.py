"""The allocation-free decode entry point against the ordinary one (collected last on purpose).

`gkv_mixed_attn_decode_static` serves hosts that may not allocate device memory around the call:
its scratch is a fixed array inside the library.  It must give the same output as
`gkv_mixed_attn_decode` on the same inputs, call after call, whether this file runs alone in a
fresh process or after every other test has used the library.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import oracle_cache, to_torch

pytestmark = pytest.mark.gpu


def _call(lib, fn_static, q, t, c, out, ws=None):
    B, Hq, D = q.shape
    Hkv, nb = t["data"].shape[1], t["level"].shape[-1]
    ptrs = [q.data_ptr(), t["data"].data_ptr(), t["offs"].data_ptr(), t["klo"].data_ptr(), t["kstep"].data_ptr(),
            t["vlo"].data_ptr(), t["vstep"].data_ptr(), t["level"].data_ptr(), t["valid"].data_ptr(), out.data_ptr()]
    tail = [B, Hq, Hkv, D, nb, 64, c["group"], t["data"].size(-1), B * Hkv, torch.cuda.current_stream().cuda_stream]
    if fn_static:
        return lib.gkv_mixed_attn_decode_static(*ptrs, *tail)
    return lib.gkv_mixed_attn_decode(*ptrs, ws.data_ptr(), ws.numel(), *tail)


def test_static_scratch_entry_point_matches_the_ordinary_one(oracle):
    from geodesia_kv_b200 import _lib
    lib = _lib.load()
    B, Hq, Hkv, nb, D, group = 2, 8, 2, 40, 128, 32
    c = oracle_cache(oracle, 909, B, Hkv, nb, D, group, last_valid=33)
    t = to_torch(c, "cuda")
    rng = np.random.default_rng(17)
    need = lib.gkv_decode_workspace_bytes(B, Hq, Hkv, D, nb)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    for attempt in range(2):                                    # two calls in a row share the array
        q = torch.from_numpy(rng.standard_normal((B, Hq, D), dtype=np.float32) * np.float32(D ** -0.5)).cuda()
        want = torch.empty(B, Hq, D, device="cuda")
        got = torch.full((B, Hq, D), float("nan"), device="cuda")
        assert _call(lib, False, q, t, c, want, ws) == 0
        before = torch.cuda.memory_allocated()
        assert _call(lib, True, q, t, c, got) == 0
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before          # nothing went through torch's allocator
        assert torch.isfinite(got).all()
        assert (got - want).abs().max().item() <= 1e-6, attempt
        ref = oracle.mixed_attn_decode(q.cpu().numpy(), c["data"], c["offs"], c["klo"], c["kstep"], c["vlo"],
                                       c["vstep"], c["level"], c["valid"], 64, group)
        assert np.abs(got.cpu().numpy() - ref).max() < 2e-3


def test_static_scratch_rejects_problems_beyond_its_size(oracle):
    from geodesia_kv_b200 import _lib
    lib = _lib.load()
    # a shape whose split records cannot fit in the built-in array: refused before anything is launched
    B, Hq, Hkv, D, nb = 256, 64, 8, 128, 4096
    assert lib.gkv_decode_workspace_bytes(B, Hq, Hkv, D, nb) > (8 << 20)
    one = 256                                                   # never dereferenced
    rc = lib.gkv_mixed_attn_decode_static(*([one] * 10), B, Hq, Hkv, D, nb, 64, 32, 1 << 20, B * Hkv, None)
    assert rc == -7
    assert b"built-in scratch" in lib.gkv_error_string(rc)
