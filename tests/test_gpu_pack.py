"""Pack / unpack / demote kernels through the C ABI: bit-exact against the CPU oracle."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import oracle_cache

pytestmark = pytest.mark.gpu


def pack_gpu(c, dtype=torch.float32):
    from geodesia_kv_b200.pack_layout import pack_cache
    B, Hkv, nb, P, D = c["k"].shape
    k = torch.from_numpy(c["k"]).cuda().view(B, Hkv, nb * P, D).to(dtype)
    v = torch.from_numpy(c["v"]).cuda().view(B, Hkv, nb * P, D).to(dtype)
    return pack_cache(k, v, torch.from_numpy(c["level"]).cuda(), c["group"])


def assert_cache_equal(cache, c, D):
    from geodesia_kv_b200.pack_layout import block_nbytes
    assert np.array_equal(cache.offs.cpu().numpy(), c["offs"])
    for key in ("klo", "kstep", "vlo", "vstep"):
        got = getattr(cache, key).cpu().view(torch.int16).numpy().view(np.uint16)
        assert np.array_equal(got, c[key]), key
    data = cache.data.cpu().numpy()
    B, Hkv, nb = c["level"].shape
    for b in range(B):
        for h in range(Hkv):
            for i in range(nb):
                o, n = int(c["offs"][b, h, i]), block_nbytes(int(c["level"][b, h, i]), D)
                assert np.array_equal(data[b, h, o:o + n], c["data"][b, h, o:o + n]), (b, h, i, int(c["level"][b, h, i]))


@pytest.mark.parametrize("D,group", [(128, 32), (128, 16), (128, 64), (64, 32), (256, 32)])
def test_pack_is_bit_exact_with_the_oracle(oracle, D, group):
    c = oracle_cache(oracle, 300 + D + group, 2, 2, 15, D, group)
    assert_cache_equal(pack_gpu(c), c, D)


def test_pack_reproduces_the_reference_bytes(oracle, golden, golden_inputs):
    """Bytes made by the reference's build_layout; centroid halves may differ by one fp16 ulp
    (torch's summation order is its own)."""
    from geodesia_kv_b200.pack_layout import block_nbytes, pack_cache
    g = golden("kat_mixed_d64")
    P, D, group = int(g["P"]), int(g["D"]), int(g["group"])
    levels = g["level"]
    k, v = golden_inputs.dense_inputs(int(g["seed"]), levels.size, P, D)
    cache = pack_cache(torch.from_numpy(k).cuda().view(1, 1, -1, D), torch.from_numpy(v).cuda().view(1, 1, -1, D),
                       torch.from_numpy(levels).cuda().view(1, 1, -1), group)
    data = cache.data.cpu().numpy()[0, 0]
    for b, lv in enumerate(levels):
        o, n = int(g["offs"][b]), block_nbytes(int(lv), D)
        if lv == 1:
            d = data[o:o + n].view(np.uint16).astype(np.int32) - g["data"][o:o + n].view(np.uint16).astype(np.int32)
            assert np.abs(d).max() <= 1
        else:
            assert np.array_equal(data[o:o + n], g["data"][o:o + n]), (b, int(lv))
    for key in ("klo", "kstep", "vlo", "vstep"):
        assert np.array_equal(getattr(cache, key).cpu().view(torch.int16).numpy().view(np.uint16)[0, 0], g[key])


def test_quantize_edge_cases_on_the_gpu(golden):
    """Constant groups, steps at the bottom of fp16, large values, exact .5 ties — the reference's
    quantize_codes outputs, reproduced bit for bit by the pack kernel."""
    from geodesia_kv_b200.pack_layout import pack_cache
    from geodesia_kv_b200.packed import unpack_bits
    g = golden("quantize_edge")
    P, D, group = int(g["P"]), int(g["D"]), int(g["group"])
    x = torch.from_numpy(g["x"]).cuda()                       # (4, P, D): used as both K and V
    nb = x.shape[0]
    for bits in (2, 4, 8):
        cache = pack_cache(x.view(1, 1, nb * P, D), x.view(1, 1, nb * P, D),
                           torch.full((1, 1, nb), bits, dtype=torch.int32, device="cuda"), group)
        data, offs = cache.data.cpu()[0, 0], cache.offs.cpu()[0, 0]
        half = P * D * bits // 8
        for b in range(nb):
            o = int(offs[b])
            kc = unpack_bits(data[o:o + half], bits, P * D).view(P, D).numpy()
            vc = unpack_bits(data[o + half:o + 2 * half], bits, P * D).view(P, D).numpy()
            assert np.array_equal(kc, g[f"codes_{bits}_k"][b]), (bits, b, "k codes")
            assert np.array_equal(vc, g[f"codes_{bits}_v"][b]), (bits, b, "v codes")
        u16 = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16)[0, 0]
        assert np.array_equal(u16(cache.klo).reshape(nb, -1), g[f"lo_{bits}_k"].reshape(nb, -1))
        assert np.array_equal(u16(cache.kstep).reshape(nb, -1), g[f"step_{bits}_k"].reshape(nb, -1))
        assert np.array_equal(u16(cache.vlo).reshape(nb, -1), g[f"lo_{bits}_v"].reshape(nb, -1))
        assert np.array_equal(u16(cache.vstep).reshape(nb, -1), g[f"step_{bits}_v"].reshape(nb, -1))


def test_unpack_is_bit_exact(oracle, golden):
    from geodesia_kv_b200.pack_layout import PackedCache, unpack_cache
    g = golden("kat_mixed_d64")
    P, D, group = int(g["P"]), int(g["D"]), int(g["group"])
    f16 = lambda a: torch.from_numpy(a.view(np.int16)).view(torch.float16).cuda()[None, None]
    i = lambda a: torch.from_numpy(a).cuda()[None, None]
    cache = PackedCache(i(g["data"]), i(g["offs"]), f16(g["klo"]), f16(g["kstep"]), f16(g["vlo"]), f16(g["vstep"]),
                        i(g["level"]), i(g["valid"]), group, D)
    k, v = unpack_cache(cache)
    assert np.array_equal(k.cpu().numpy().reshape(-1, P, D).view(np.uint32), g["krec"].view(np.uint32))
    assert np.array_equal(v.cpu().numpy().reshape(-1, P, D).view(np.uint32), g["vrec"].view(np.uint32))


def test_bf16_and_fp16_sources(oracle):
    c = oracle_cache(oracle, 411, 1, 2, 6, 128, 32)
    for dt in (torch.bfloat16, torch.float16):
        c2 = dict(c)
        c2["k"] = torch.from_numpy(c["k"]).to(dt).float().numpy()
        c2["v"] = torch.from_numpy(c["v"]).to(dt).float().numpy()
        rows = [oracle.pack_row(c2["k"][0, h], c2["v"][0, h], c["level"][0, h], 32) for h in range(2)]
        got = pack_gpu(c2, dt)
        for h in range(2):
            assert np.array_equal(got.data.cpu().numpy()[0, h, :rows[h]["data"].size], rows[h]["data"])


def test_ragged_tail_is_padded_with_the_last_row(oracle):
    from geodesia_kv_b200.pack_layout import pack_cache, unpack_cache
    T, D = 64 * 3 - 21, 64
    gen = torch.Generator(device="cuda").manual_seed(1)
    k = torch.randn(1, 1, T, D, device="cuda", generator=gen)
    v = torch.randn(1, 1, T, D, device="cuda", generator=gen)
    cache = pack_cache(k, v, torch.tensor([4, 2, 16], dtype=torch.int32, device="cuda").view(1, 1, 3), 32)
    assert cache.valid[0, 0].tolist() == [64, 64, 43]
    kk, vv = unpack_cache(cache)
    want = k[0, 0, -1].to(torch.bfloat16).float()
    assert torch.equal(kk[0, 0, T:], want.expand(21, D))


def test_demote_to_a_fresh_buffer(oracle):
    """policies.py:869-908: a demoted block is re-quantised from its CURRENT representation."""
    from geodesia_kv_b200 import _lib
    from geodesia_kv_b200.pack_layout import block_nbytes, layout_offsets
    D, group, nb = 128, 32, 10
    c = oracle_cache(oracle, 612, 1, 2, nb, D, group, levels=[16] * nb)
    cache = pack_gpu(c)
    targets = [16, 8, 4, 2, 1, 1, 2, 4, 8, 16]
    new_level = torch.tensor(targets, dtype=torch.int32, device="cuda").expand(1, 2, nb).contiguous()
    new_offs, row_bytes = layout_offsets(new_level, D)
    new_data = torch.zeros(1, 2, int(row_bytes.max()), dtype=torch.uint8, device="cuda")
    lib = _lib.load()
    rc = lib.gkv_demote_blocks(cache.data.data_ptr(), cache.offs.data_ptr(), cache.level.data_ptr(),
                               new_data.data_ptr(), new_offs.data_ptr(), new_level.data_ptr(),
                               cache.klo.data_ptr(), cache.kstep.data_ptr(), cache.vlo.data_ptr(), cache.vstep.data_ptr(),
                               2, nb, D, 64, group, cache.data.size(-1), new_data.size(-1), 2,
                               torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "demote")
    got = new_data.cpu().numpy()
    for h in range(2):
        # the current representation of a rung-16 block is its bf16 rounding
        kb = torch.from_numpy(c["k"][0, h]).to(torch.bfloat16).float().numpy()
        vb = torch.from_numpy(c["v"][0, h]).to(torch.bfloat16).float().numpy()
        want = oracle.pack_row(kb, vb, targets, group)
        for i, lv in enumerate(targets):
            if lv == 16:
                continue                       # unchanged blocks are not rewritten
            o, n = int(want["offs"][i]), block_nbytes(lv, D)
            assert np.array_equal(got[0, h, o:o + n], want["data"][o:o + n]), (h, i, lv)
            for key in ("klo", "kstep", "vlo", "vstep"):
                g = getattr(cache, key).cpu().view(torch.int16).numpy().view(np.uint16)[0, h, i]
                assert np.array_equal(g, want[key][i]), (key, i)


def test_demote_same_place_single_blocks(oracle):
    """In place: the new bytes start where the old block started (offs unchanged)."""
    from geodesia_kv_b200 import _lib
    from geodesia_kv_b200.pack_layout import block_nbytes, unpack_cache
    D, group, nb = 128, 32, 6
    c = oracle_cache(oracle, 700, 1, 1, nb, D, group, levels=[16] * nb)
    cache = pack_gpu(c)
    targets = [16, 4, 16, 2, 1, 8]
    new_level = torch.tensor(targets, dtype=torch.int32, device="cuda").view(1, 1, nb)
    lib = _lib.load()
    rc = lib.gkv_demote_blocks(cache.data.data_ptr(), cache.offs.data_ptr(), cache.level.data_ptr(),
                               cache.data.data_ptr(), cache.offs.data_ptr(), new_level.data_ptr(),
                               cache.klo.data_ptr(), cache.kstep.data_ptr(), cache.vlo.data_ptr(), cache.vstep.data_ptr(),
                               1, nb, D, 64, group, cache.data.size(-1), cache.data.size(-1), 1,
                               torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "demote")
    cache.level = new_level
    kb = torch.from_numpy(c["k"][0, 0]).to(torch.bfloat16).float().numpy()
    vb = torch.from_numpy(c["v"][0, 0]).to(torch.bfloat16).float().numpy()
    data = cache.data.cpu().numpy()[0, 0]
    for i, lv in enumerate(targets):
        want = oracle.pack_row(kb[i:i + 1], vb[i:i + 1], [lv], group)
        o = int(cache.offs[0, 0, i])
        assert np.array_equal(data[o:o + block_nbytes(lv, D)], want["data"]), (i, lv)
    # promotion is refused: asking for 16 on a demoted block leaves it untouched
    up = torch.full((1, 1, nb), 16, dtype=torch.int32, device="cuda")
    before = cache.data.clone()
    rc = lib.gkv_demote_blocks(cache.data.data_ptr(), cache.offs.data_ptr(), new_level.data_ptr(),
                               cache.data.data_ptr(), cache.offs.data_ptr(), up.data_ptr(),
                               cache.klo.data_ptr(), cache.kstep.data_ptr(), cache.vlo.data_ptr(), cache.vstep.data_ptr(),
                               1, nb, D, 64, group, cache.data.size(-1), cache.data.size(-1), 1,
                               torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "demote")
    assert torch.equal(before, cache.data)


def test_round_trip_error_bound_at_full_size():
    """encode -> decode on a 16k-token, 8-head, batch-4 slab: every element within step/2 of the
    source for quantised rungs, exact bf16 for rung 16 (quant_grouped's stated bound)."""
    from geodesia_kv_b200.pack_layout import pack_cache, unpack_cache
    B, Hkv, T, D, group = 4, 8, 16384, 128, 32
    gen = torch.Generator(device="cuda").manual_seed(3)
    k = torch.randn(B, Hkv, T, D, device="cuda", generator=gen)
    v = torch.randn(B, Hkv, T, D, device="cuda", generator=gen)
    nb = T // 64
    ladder = torch.tensor([16, 8, 4, 2], device="cuda", dtype=torch.int32)
    level = ladder[torch.randint(0, 4, (B, Hkv, nb), device="cuda", generator=gen)]
    cache = pack_cache(k, v, level, group)
    kk, vv = unpack_cache(cache)
    lv = level.repeat_interleave(64, dim=-1)[..., None].float()
    kstep = cache.kstep.float().repeat_interleave(group, dim=3).view(B, Hkv, T, D)
    vstep = cache.vstep.float().repeat_interleave(group, dim=4).view(B, Hkv, T, D)
    q = lv < 16
    # half a step, plus the fp16 rounding of lo (2^-11 relative) and of step
    kbound = torch.where(q, kstep * 0.5 * 1.002 + k.abs().amax() * 2 ** -10, k.abs() * 2 ** -8)
    vbound = torch.where(q, vstep * 0.5 * 1.002 + v.abs().amax() * 2 ** -10, v.abs() * 2 ** -8)
    assert bool(((kk - k).abs() <= kbound).all())
    assert bool(((vv - v).abs() <= vbound).all())
