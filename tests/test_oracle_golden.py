"""The C oracle against fixtures produced by the reference's own Python (CPU only).

Each test names the reference code that produced the expected values; see
tests/golden/make_golden.py for how they were made.
"""
from __future__ import annotations

import numpy as np
import pytest


def h2f(u16):
    return np.asarray(u16, np.uint16).view(np.float16).astype(np.float32)


def test_pack_unpack_bits(oracle, golden):
    g = golden("pack_bits")                     # geodesia_kv/packed.py:23-49
    for bits in (2, 4, 8):
        for n in (64, 63, 130):
            codes, packed = g[f"codes_{bits}_{n}"], g[f"packed_{bits}_{n}"]
            assert np.array_equal(oracle.pack_bits(codes, bits), packed)
            assert np.array_equal(oracle.unpack_bits(packed, bits, n), codes)


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("per_channel", [True, False])
def test_quantize_codes_edge_cases(oracle, golden, bits, per_channel):
    g = golden("quantize_edge")                 # tests/test_cuda_kernel.py:18-33 of the reference
    P, D, group = int(g["P"]), int(g["D"]), int(g["group"])
    tag = f"{bits}_{'k' if per_channel else 'v'}"
    for b in range(g["x"].shape[0]):
        codes, lo, step = oracle.quantize_codes(g["x"][b], bits, group, per_channel)
        assert np.array_equal(lo.reshape(-1), g[f"lo_{tag}"][b].reshape(-1)), (b, "lo")
        assert np.array_equal(step.reshape(-1), g[f"step_{tag}"][b].reshape(-1)), (b, "step")
        assert np.array_equal(codes, g[f"codes_{tag}"][b]), (b, "codes")
        # reconstruction code*step16 + lo16 in fp32, bit for bit
        if per_channel:
            rec = (codes.reshape(P // group, group, D).astype(np.float32) * h2f(step)[:, None, :]
                   + h2f(lo)[:, None, :]).reshape(P, D)
        else:
            rec = (codes.reshape(P, D // group, group).astype(np.float32) * h2f(step)[:, :, None]
                   + h2f(lo)[:, :, None]).reshape(P, D)
        want = g[f"rec_{tag}"][b]
        finite = np.isfinite(want)
        assert np.array_equal(rec[finite].view(np.uint32), want[finite].view(np.uint32)), (b, "rec")


def _check_row_bytes(oracle, g, k, v, levels, group, sfx=""):
    """pack_row must reproduce build_layout's bytes; centroid halves within one fp16 ulp."""
    lay = oracle.pack_row(k, v, levels, group)
    P, D = k.shape[1:]
    assert np.array_equal(lay["offs"], g["offs" + sfx])
    assert int(lay["nbytes"]) == int(g["nbytes" + sfx])
    for key in ("klo", "kstep", "vlo", "vstep"):
        assert np.array_equal(lay[key], g[key + sfx]), key
    want = g["data" + sfx]
    assert lay["data"].size == want.size
    for b, lv in enumerate(levels):
        o, n = int(lay["offs"][b]), oracle.block_bytes(lv, P, D)
        got_b, want_b = lay["data"][o:o + n], want[o:o + n]
        if lv == 1:
            a = got_b.view(np.uint16).astype(np.int32)
            w = want_b.view(np.uint16).astype(np.int32)
            assert np.abs(a - w).max() <= 1, f"centroid block {b} off by more than one fp16 ulp"
        else:
            assert np.array_equal(got_b, want_b), f"block {b} rung {lv}"


def test_known_answer_config_bytes_dequant_and_output(oracle, golden, golden_inputs):
    g = golden("kat_mixed_d64")                 # tests/test_cuda_kernel.py:36-104 of the reference
    P, D, group, H = (int(g[x]) for x in ("P", "D", "group", "H"))
    levels = [int(x) for x in g["level"]]
    nb = len(levels)
    k, v = golden_inputs.dense_inputs(int(g["seed"]), nb, P, D)
    _check_row_bytes(oracle, g, k, v, levels, group)
    # dequantisation of the reference's bytes, bit for bit
    for b, lv in enumerate(levels):
        o, n = int(g["offs"][b]), oracle.block_bytes(lv, P, D)
        kd, vd = oracle.dequant_block(g["data"][o:o + n], lv, P, D, group, g["klo"][b], g["kstep"][b],
                                      g["vlo"][b], g["vstep"][b])
        assert np.array_equal(kd.view(np.uint32), g["krec"][b].view(np.uint32)), (b, lv)
        assert np.array_equal(vd.view(np.uint32), g["vrec"][b].view(np.uint32)), (b, lv)
    # attention: layout replicated per head as the reference's test does (:84-95)
    q = golden_inputs.query(int(g["seed"]), 1, H, D)
    rep = lambda a: np.broadcast_to(a[None, None], (1, H) + a.shape).copy()
    out = oracle.mixed_attn_decode(q, rep(g["data"]), g["offs"], rep(g["klo"]), rep(g["kstep"]),
                                   rep(g["vlo"]), rep(g["vstep"]), g["level"], g["valid"], P, group)
    rel = np.abs(out[0] - g["out"]).max() / np.abs(g["out"]).max()
    assert rel < 1e-5, rel                       # the reference's own bound is 1e-4 (:102-104)


def test_gqa_rows_with_ragged_tail(oracle, golden, golden_inputs):
    g = golden("gqa_d128")
    P, D, group, Hq, Hkv, nb = (int(g[x]) for x in ("P", "D", "group", "Hq", "Hkv", "nb"))
    rows = []
    for r in range(Hkv):
        k, v = golden_inputs.dense_inputs(int(g["seeds"][r]), nb, P, D, outliers=4)
        _check_row_bytes(oracle, g, k, v, [int(x) for x in g[f"level_{r}"]], group, sfx=f"_{r}")
        rows.append({key: g[f"{key}_{r}"] for key in
                     ("data", "offs", "klo", "kstep", "vlo", "vstep", "level", "valid")})
    # rows have different byte lengths: pad to a common stride
    stride = max(r["data"].size for r in rows)
    data = np.zeros((1, Hkv, stride), np.uint8)
    for r in range(Hkv):
        data[0, r, :rows[r]["data"].size] = rows[r]["data"]
    st = lambda key: np.stack([rows[r][key] for r in range(Hkv)])[None]
    valid = st("valid").copy()
    valid[..., -1] = int(g["last_valid"])
    q = golden_inputs.query(int(g["qseed"]), 1, Hq, D) * np.float32(D ** -0.5)
    out = oracle.mixed_attn_decode(q, data, st("offs"), st("klo"), st("kstep"), st("vlo"), st("vstep"),
                                   st("level"), valid, P, group)
    assert np.abs(out - g["out"]).max() < 2e-6


@pytest.mark.parametrize("group", [16, 64])
def test_other_group_sizes(oracle, golden, golden_inputs, group):
    g = golden(f"group{group}_d128")
    P, D = int(g["P"]), int(g["D"])
    levels = [int(x) for x in g["level"]]
    k, v = golden_inputs.dense_inputs(int(g["seed"]), len(levels), P, D, outliers=4)
    _check_row_bytes(oracle, g, k, v, levels, group)
    q = golden_inputs.query(int(g["seed"]), 1, 1, D) * np.float32(D ** -0.5)
    ex = lambda a: a[None, None]
    out = oracle.mixed_attn_decode(q, ex(g["data"]), g["offs"], ex(g["klo"]), ex(g["kstep"]), ex(g["vlo"]),
                                   ex(g["vstep"]), g["level"], g["valid"], P, group)
    assert np.abs(out - g["out"]).max() < 2e-6


def test_level_bits(oracle, golden):
    g = golden("allocator")                     # geodesia_kv/policies.py:1582-1596
    for c in range(int(g["ncases"])):
        P, D, group = (int(x) for x in g[f"c{c}_meta"][:3])
        got = [oracle.level_bits(L, P, D, group) for L in oracle.LADDER]
        assert np.array_equal(np.asarray(got, np.float32), g[f"c{c}_bits"])


def test_allocator_matches_traced_reference(oracle, golden):
    g = golden("allocator")                     # geodesia_kv/policies.py:810-868, traced
    moved = 0
    for c in range(int(g["ncases"])):
        tgt, ratio = oracle.allocate(g[f"c{c}_mass"], g[f"c{c}_E"], g[f"c{c}_lvl_idx"], g[f"c{c}_hot"],
                                     g[f"c{c}_bits"], float(g[f"c{c}_target"]))
        assert np.array_equal(ratio.view(np.uint32), g[f"c{c}_ratio"].view(np.uint32)), c
        assert np.array_equal(tgt, g[f"c{c}_tgt_idx"]), c
        after = np.asarray([oracle.LADDER[i] for i in tgt], np.float32)
        assert np.array_equal(after, g[f"c{c}_level_after"]), c
        moved += int((g[f"c{c}_level_after"] != g[f"c{c}_level_before"]).sum())
        # monotonic: no block rises, and one that has left rung 16 never moves again
        assert (g[f"c{c}_level_after"] <= g[f"c{c}_level_before"]).all()
        left16 = g[f"c{c}_level_before"] < 16
        assert np.array_equal(g[f"c{c}_level_after"][left16], g[f"c{c}_level_before"][left16])
    assert moved > 20                            # the fixtures really exercise demotion


def test_distortion_table(oracle, golden, golden_inputs):
    g = golden("distortion")                    # geodesia_kv/policies.py:774-808
    P, D, group, nb = (int(g[x]) for x in ("P", "D", "group", "nb"))
    k, v = golden_inputs.dense_inputs(int(g["seed"]), nb, P, D, outliers=int(g["outliers"]))
    E = oracle.distortion(k, v, group, float(g["value_weight"]))
    np.testing.assert_allclose(E, g["E"], rtol=2e-6, atol=0)


def test_empty_and_degenerate_inputs(oracle):
    P, D, group = 64, 64, 32
    q = np.ones((1, 2, D), np.float32)
    z16 = lambda *s: np.zeros(s, np.uint16)
    # no blocks at all: every slice is empty, the output is 0 (l clamps to 1e-20, mixed_attn.cu:198)
    out = oracle.mixed_attn_decode(q, np.zeros((1, 2, 0), np.uint8), np.zeros(0, np.int64),
                                   z16(1, 2, 0, 2, D), z16(1, 2, 0, 2, D), z16(1, 2, 0, P, 2),
                                   z16(1, 2, 0, P, 2), np.zeros(0, np.int32), np.zeros(0, np.int32), P, group)
    assert np.array_equal(out, np.zeros_like(out))
    # one block with a single valid token: the output is that token's V row
    rng = np.random.default_rng(1)
    k = rng.standard_normal((1, P, D), dtype=np.float32)
    v = rng.standard_normal((1, P, D), dtype=np.float32)
    lay = oracle.pack_row(k, v, [16], group)
    out = oracle.mixed_attn_decode(q[:, :1], lay["data"][None, None], lay["offs"], lay["klo"][None, None],
                                   lay["kstep"][None, None], lay["vlo"][None, None], lay["vstep"][None, None],
                                   lay["level"], np.array([1], np.int32), P, group)
    want = (v[0, 0].view(np.uint32) + 0x7FFF + ((v[0, 0].view(np.uint32) >> 16) & 1)) & 0xFFFF0000
    assert np.array_equal(out[0, 0].view(np.uint32), want.astype(np.uint32))
