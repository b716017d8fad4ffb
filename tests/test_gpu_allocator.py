"""Allocator and distortion-table kernels through the C ABI."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_traced_reference_cases_are_reproduced_bit_for_bit(golden):
    """Inputs and outputs traced out of the reference's Policy.attend (policies.py:810-868)."""
    from geodesia_kv_b200 import policies
    g = golden("allocator")
    for c in range(int(g["ncases"])):
        P, D, group, nb, T = (int(x) for x in g[f"c{c}_meta"])
        cu = lambda a: torch.from_numpy(a).cuda()
        tgt, ratio = policies.allocate_rungs(cu(g[f"c{c}_mass"]), cu(g[f"c{c}_E"]), cu(g[f"c{c}_lvl_idx"]),
                                             cu(g[f"c{c}_hot"]), float(g[f"c{c}_budget"]), P, D, group,
                                             return_ratio=True)
        assert np.array_equal(ratio.cpu().numpy().view(np.uint32), g[f"c{c}_ratio"].view(np.uint32)), c
        assert np.array_equal(tgt.cpu().numpy(), g[f"c{c}_tgt_idx"]), c


def power_law_mass(nb, sink=0.1):
    dist = (nb - 1 - np.arange(nb)).astype(np.float64)
    m = (dist + 1.0) ** -1.2
    m /= m.sum()
    m[0] += sink
    return m.astype(np.float32)


def test_append_and_demote_scenario_against_the_oracle(oracle):
    """36 layers x 8 heads, one block appended per step (192 -> 256 blocks), budgets 2..5 bits:
    every step's rung assignment equals the oracle's, no block ever rises, and a block that has
    left rung 16 never moves again."""
    from geodesia_kv_b200 import policies
    P, D, group, probs = 64, 128, 32, 36 * 8
    rng = np.random.default_rng(2000)
    bits = np.asarray(policies.ladder_bits(P, D, group), np.float32)
    for budget in (2.0, 3.0, 4.0, 5.0):
        nb_max = 256
        # a synthetic but plausible distortion table: rises down the ladder, varies per block
        base = np.abs(rng.standard_normal((probs, nb_max, 1), dtype=np.float32)) + 0.5
        E = base * np.array([0.0, 0.02, 0.3, 1.5, 6.0], np.float32) * (1 + 0.2 * rng.random((probs, nb_max, 5), dtype=np.float32))
        E[..., 0] = 0.0
        idx = np.zeros((probs, 192), np.int32)
        for step, nb in enumerate(range(192, 257, 8)):
            if nb > idx.shape[1]:
                idx = np.concatenate([idx, np.zeros((probs, nb - idx.shape[1]), np.int32)], 1)
            mass = np.broadcast_to(power_law_mass(nb), (probs, nb)).copy()
            mass *= (1 + 0.1 * rng.random((probs, nb), dtype=np.float32))
            hot = policies.hot_mask(nb, nb * P - 1, P, 4, 128).numpy().astype(np.uint8)
            hotp = np.broadcast_to(hot, (probs, nb)).copy()
            cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
            tgt = policies.allocate_rungs(cu(mass), cu(E[:, :nb]), cu(idx), cu(hotp), budget, P, D, group).cpu().numpy()
            for pr in range(0, probs, 7):                       # oracle on a stride of the problems
                want, _ = oracle.allocate(mass[pr], E[pr, :nb], idx[pr], hotp[pr], bits, budget * 2.0 * nb * P * D)
                assert np.array_equal(tgt[pr], want), (budget, nb, pr)
            assert (tgt >= idx).all()
            assert np.array_equal(tgt[idx > 0], idx[idx > 0])
            assert (tgt[hotp > 0] == idx[hotp > 0]).all()
            idx = tgt


def test_million_token_row(oracle):
    """nb = 16384 (the 1M-token config): more candidates than fit in shared memory."""
    from geodesia_kv_b200 import policies
    P, D, group, nb = 64, 128, 32, 16384
    rng = np.random.default_rng(3000)
    E = (np.abs(rng.standard_normal((4, nb, 1), dtype=np.float32)) + 0.5) * np.array([0.0, 0.02, 0.3, 1.5, 6.0], np.float32)
    mass = np.broadcast_to(power_law_mass(nb), (4, nb)).copy()
    idx = np.zeros((4, nb), np.int32)
    hot = np.broadcast_to(policies.hot_mask(nb, nb * P - 1, P, 4, 128).numpy().astype(np.uint8), (4, nb)).copy()
    cu = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    tgt = policies.allocate_rungs(cu(mass), cu(E), cu(idx), cu(hot), 2.0, P, D, group).cpu().numpy()
    bits = np.asarray(policies.ladder_bits(P, D, group), np.float32)
    for pr in range(4):
        want, _ = oracle.allocate(mass[pr], E[pr], idx[pr], hot[pr], bits, 2.0 * 2.0 * nb * P * D)
        assert np.array_equal(tgt[pr], want)


def test_degenerate_budgets(oracle):
    from geodesia_kv_b200 import policies
    P, D, group, nb = 64, 64, 32, 40
    rng = np.random.default_rng(5)
    E = (np.abs(rng.standard_normal((1, nb, 1), dtype=np.float32)) + 0.5) * np.array([0.0, 0.02, 0.3, 1.5, 6.0], np.float32)
    mass = rng.random((1, nb), dtype=np.float32)
    idx = np.zeros((1, nb), np.int32)
    hot = np.zeros((1, nb), np.uint8)
    hot[0, -2:] = 1
    bits = np.asarray(policies.ladder_bits(P, D, group), np.float32)
    cu = lambda a: torch.from_numpy(a).cuda()
    for budget in (16.0, 100.0, 0.01, 0.25):       # already satisfied ... impossible to satisfy
        tgt = policies.allocate_rungs(cu(mass), cu(E), cu(idx), cu(hot), budget, P, D, group).cpu().numpy()
        want, _ = oracle.allocate(mass[0], E[0], idx[0], hot[0], bits, budget * 2.0 * nb * P * D)
        assert np.array_equal(tgt[0], want), budget
    # even a satisfied budget takes the cheapest available step (the reference's first candidate)
    tgt = policies.allocate_rungs(cu(mass), cu(E), cu(idx), cu(hot), 100.0, P, D, group).cpu().numpy()
    assert (tgt > 0).sum() >= 1


def test_distortion_table(oracle, golden, golden_inputs):
    from geodesia_kv_b200 import policies
    from geodesia_kv_b200.pack_layout import pack_cache
    g = golden("distortion")
    P, D, group, nb = (int(g[x]) for x in ("P", "D", "group", "nb"))
    k, v = golden_inputs.dense_inputs(int(g["seed"]), nb, P, D, outliers=int(g["outliers"]))
    # rung-16 blocks hold bf16: feed bf16-representable inputs so both sides see the same values
    kb = torch.from_numpy(k).to(torch.bfloat16)
    vb = torch.from_numpy(v).to(torch.bfloat16)
    level = torch.full((1, 1, nb), 16, dtype=torch.int32, device="cuda")
    level[0, 0, 2] = 4                               # a demoted block gets a zero row
    cache = pack_cache(kb.cuda().view(1, 1, -1, D), vb.cuda().view(1, 1, -1, D), level, group)
    E = policies.block_distortion(cache, float(g["value_weight"])).cpu().numpy()[0, 0]
    want = oracle.distortion(kb.float().numpy(), vb.float().numpy(), group, float(g["value_weight"]))
    keep = np.arange(nb) != 2
    assert np.array_equal(E[keep].view(np.uint32), want[keep].view(np.uint32))
    assert (E[2] == 0).all()
    # and, up to bf16 rounding of the inputs, the reference's table
    np.testing.assert_allclose(E[keep], g["E"][keep], rtol=2e-2)
