"""Host logic of the paged pool (size-class free lists over slabs); no GPU needed."""
from __future__ import annotations

import numpy as np
import pytest


def make_pool(mib=32, D=128, group=32):
    from geodesia_kv_b200.paged import PagedPool
    return PagedPool(mib << 20, D, group, device="cpu")


def test_slot_sizes_and_slab_geometry():
    pool = make_pool()
    assert pool.slot == {16: 32768, 8: 18432, 4: 10240, 2: 6144, 1: 512}
    assert pool.slab_bytes == 1474560 and all(pool.slab_bytes % s == 0 for s in pool.slot.values())
    small = make_pool(D=64)
    assert small.slot == {16: 16384, 8: 9216, 4: 5120, 2: 3072, 1: 256}


def test_slots_are_disjoint_and_aligned():
    pool = make_pool()
    got = []
    for rung, n in ((16, 50), (8, 90), (4, 10), (2, 300), (1, 3000), (16, 41)):
        offs = pool.alloc(rung, n)
        assert offs.dtype == np.int64 and offs.size == n and (offs % 512 == 0).all()
        got += [(int(o), int(o) + pool.slot[rung]) for o in offs]
    got.sort()
    assert all(a[1] <= b[0] for a, b in zip(got, got[1:]))
    assert got[-1][1] <= pool.capacity_bytes
    assert pool.bytes_in_use == 91 * 32768 + 90 * 18432 + 10 * 10240 + 300 * 6144 + 3000 * 512


def test_demotion_pattern_returns_bytes_and_slabs():
    pool = make_pool()
    big = pool.alloc(16, 90)                       # two slabs of rung 16
    assert pool.bytes_reserved == 2 * pool.slab_bytes
    small = pool.alloc(4, 90)
    freed_slab = int(big[0]) // pool.slab_bytes
    assert (big[:45] // pool.slab_bytes == freed_slab).all()
    pool.free(16, big[:45])                        # that slab empties and goes back
    assert pool.bytes_reserved == 2 * pool.slab_bytes
    assert pool.bytes_in_use == 45 * 32768 + 90 * 10240
    again = pool.alloc(2, 10)                      # reuses the returned slab for another rung
    assert (again // pool.slab_bytes == freed_slab).all()
    pool.free(16, big[45:])
    pool.free(4, small)
    pool.free(2, again)
    assert pool.bytes_in_use == 0 and pool.bytes_reserved == 0
    assert pool.peak_bytes_in_use == 90 * 32768 + 90 * 10240


def test_exhaustion_and_wrong_rung_are_errors():
    from geodesia_kv_b200.paged import PoolExhausted
    pool = make_pool(mib=3)                        # two slabs
    a = pool.alloc(16, 45)
    pool.alloc(8, 80)
    with pytest.raises(PoolExhausted):
        pool.alloc(4, 1)
    with pytest.raises(ValueError):
        pool.free(8, a[:1])
    pool.free(16, a)
    assert pool.alloc(4, 144).size == 144
