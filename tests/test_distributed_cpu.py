"""Host logic of the multi-GPU paths on CPU ranks (gloo, world size 2 and 3): the byte-balanced
block split and the gather-and-merge of per-rank softmax records.  The records are produced and
merged here by the test's own numpy/torch code (the product has no CPU path); what is under test
is the partition and the collective plumbing in geodesia_kv_b200.distributed."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def test_split_is_a_partition_and_balances_bytes():
    from geodesia_kv_b200.distributed import block_cost_bytes, split_blocks
    rng = np.random.default_rng(0)
    for world in (1, 2, 4, 8):
        for nb in (1, 3, 8, 500, 16384):
            lv = rng.choice([16, 8, 4, 2, 1], size=nb, p=[0.02, 0.08, 0.3, 0.4, 0.2])
            parts = split_blocks(lv, 128, 32, world)
            assert len(parts) == world and parts[0][0] == 0 and parts[-1][1] == nb
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            cost = np.asarray(block_cost_bytes(lv, 128, 32))
            if nb >= 500:
                per = [cost[a:b].sum() for a, b in parts]
                assert max(per) - min(per) <= 2 * cost.max()


def _records(oracle, c, q, lo, hi, P, D, group):
    """[m, l, o] of every query head over blocks [lo, hi) of row 0, from the oracle's de-quantiser."""
    Hq = q.shape[1]
    rec = np.zeros((1, Hq, D + 2), np.float32)
    ks, vs = [], []
    for b in range(lo, hi):
        o = int(c["offs"][0, 0, b])
        n = oracle.block_bytes(int(c["level"][0, 0, b]), P, D)
        kd, vd = oracle.dequant_block(c["data"][0, 0, o:o + n], int(c["level"][0, 0, b]), P, D, group, c["klo"][0, 0, b],
                                      c["kstep"][0, 0, b], c["vlo"][0, 0, b], c["vstep"][0, 0, b])
        nv = int(c["valid"][0, 0, b])
        ks.append(kd[:nv]); vs.append(vd[:nv])
    if not ks:
        rec[..., 0] = -np.inf
        return rec
    k, v = np.concatenate(ks).astype(np.float64), np.concatenate(vs).astype(np.float64)
    s = q[0].astype(np.float64) @ k.T
    m = s.max(-1)
    p = np.exp(s - m[:, None])
    rec[0, :, 0], rec[0, :, 1], rec[0, :, 2:] = m, p.sum(-1), p @ v
    return rec


def _combine(gathered: torch.Tensor) -> torch.Tensor:
    m = gathered[..., 0]
    mx = m.max(0).values
    w = torch.where(torch.isinf(m), torch.zeros_like(m), torch.exp(m - mx))
    l = (w * gathered[..., 1]).sum(0)
    return (w[..., None] * gathered[..., 2:]).sum(0) / l.clamp_min(1e-20)[..., None]


def _worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    for p in (str(ROOT), str(ROOT / "oracle"), str(ROOT / "tests")):
        sys.path.insert(0, p)
    import gkv_oracle
    from helpers import oracle_args, oracle_cache
    from geodesia_kv_b200.distributed import gather_and_combine, split_blocks
    dist.init_process_group("gloo", rank=rank, world_size=world)
    P, D, group, nb = 64, 64, 32, 23
    c = oracle_cache(gkv_oracle, 5, 1, 1, nb, D, group, last_valid=40)
    q = np.random.default_rng(9).standard_normal((1, 4, D), dtype=np.float32) * np.float32(D ** -0.5)
    lo, hi = split_blocks(c["level"][0, 0], D, group, world)[rank]
    partial = torch.from_numpy(_records(gkv_oracle, c, q, lo, hi, P, D, group))
    out = gather_and_combine(partial, _combine)
    want = gkv_oracle.mixed_attn_decode(q, *oracle_args(c))
    err = float(np.abs(out.numpy() - want).max())
    if rank == 0:
        Path(out_path).write_text(f"{err}")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_split_records_merge_across_gloo_ranks(tmp_path, world, oracle):
    out = tmp_path / "err.txt"
    port = 29500 + os.getpid() % 2000 + world
    mp.spawn(_worker, args=(world, port, str(out)), nprocs=world, join=True)
    assert float(out.read_text()) < 1e-5
