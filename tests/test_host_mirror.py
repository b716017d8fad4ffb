"""Host-side mirrors of the reference's Python API against the reference-made fixtures (CPU)."""
from __future__ import annotations

import numpy as np
import torch

from geodesia_kv_b200 import pack_layout, packed, policies


def f16(u16):
    return torch.from_numpy(np.asarray(u16, np.uint16).view(np.int16)).view(torch.float16)


def test_pack_bits_matches_reference(golden):
    g = golden("pack_bits")
    for bits in (2, 4, 8):
        for n in (64, 63, 130):
            codes = torch.from_numpy(g[f"codes_{bits}_{n}"])
            pk = packed.pack_bits(codes, bits)
            assert np.array_equal(pk.numpy(), g[f"packed_{bits}_{n}"])
            assert packed.unpack_bits(pk, bits, n).equal(codes)


def test_build_layout_is_byte_identical(golden, golden_inputs, oracle):
    g = golden("kat_mixed_d64")
    P, D, group = int(g["P"]), int(g["D"]), int(g["group"])
    levels = [int(x) for x in g["level"]]
    nb = len(levels)
    k, v = golden_inputs.dense_inputs(int(g["seed"]), nb, P, D)
    items = {}
    for b, lv in enumerate(levels):
        kb, vb = torch.from_numpy(k[b]), torch.from_numpy(v[b])
        if lv == 16:
            items[b] = {"k": kb, "v": vb}
        elif lv == 1:
            items[b] = {"k": kb.mean(0, keepdim=True).to(torch.float16), "v": vb.mean(0, keepdim=True).to(torch.float16)}
        else:
            ck, klo, kstep = oracle.quantize_codes(k[b], lv, group, True)
            cv, vlo, vstep = oracle.quantize_codes(v[b], lv, group, False)
            items[b] = {"k": torch.from_numpy(ck), "v": torch.from_numpy(cv), "klo": f16(klo), "kstep": f16(kstep),
                        "vlo": f16(vlo), "vstep": f16(vstep)}
    lay = pack_layout.build_layout(items, P, group, D, nb, torch.tensor(levels), torch.full((nb,), P), "cpu")
    assert np.array_equal(lay["data"].numpy(), g["data"])
    assert np.array_equal(lay["offs"].numpy(), g["offs"])
    assert lay["nbytes"] == int(g["nbytes"])
    assert lay["level"].dtype == torch.int32 and lay["valid"].dtype == torch.int32
    for key in ("klo", "kstep", "vlo", "vstep"):
        assert np.array_equal(lay[key].view(torch.int16).numpy().view(np.uint16), g[key])
    # an all-2-bit layout really is smaller than half of bf16 (tests/test_cuda_kernel.py:107-128)
    assert pack_layout.block_nbytes(2, D) * nb + 4 * (lay["klo"].numel() + lay["vlo"].numel()) < 2 * nb * P * D * 2 / 2


def test_build_packed_matches_reference(golden, golden_inputs):
    g = golden("format_a")
    P, D, group = int(g["P"]), int(g["D"]), int(g["group"])
    k, v = golden_inputs.dense_inputs(int(g["seed"]), 6, P, D)
    bits = torch.tensor([16.0, 8.0, 4.0, 2.0, 3.0, 4.0])
    cent = torch.tensor([False, False, False, False, False, True])
    pk = packed.build_packed(torch.from_numpy(k.reshape(-1, D)), torch.from_numpy(v.reshape(-1, D)), bits, cent, P, group)
    assert pk.nbytes() == int(g["nbytes"])
    assert np.array_equal(pk.exact_idx.numpy(), g["exact_idx"]) and np.array_equal(pk.cent_idx.numpy(), g["cent_idx"])
    assert np.array_equal(pk.exact_k.view(torch.int16).numpy().view(np.uint16), g["exact_k"])
    assert np.abs(pk.cent_k.view(torch.int16).numpy().astype(np.int32) - g["cent_k"].view(np.int16).astype(np.int32)).max() <= 1
    assert len(pk.quant) == int(g["nquant"])
    for i, (idx, pkk, pvv) in enumerate(pk.quant):
        assert np.array_equal(idx.numpy(), g[f"q{i}_idx"]) and pkk.bits == int(g[f"q{i}_bits"])
        assert np.array_equal(pkk.data.numpy(), g[f"q{i}_kdata"]) and np.array_equal(pvv.data.numpy(), g[f"q{i}_vdata"])
        assert np.array_equal(pkk.lo.view(torch.int16).numpy().view(np.uint16), g[f"q{i}_klo"])
        assert np.array_equal(pvv.step.view(torch.int16).numpy().view(np.uint16), g[f"q{i}_vstep"])
        assert np.array_equal(pkk.dequantize().numpy(), g[f"q{i}_kdeq"])
        assert np.array_equal(pvv.dequantize().numpy(), g[f"q{i}_vdeq"])


def test_level_bits_and_hot_mask(golden):
    g = golden("allocator")
    for c in range(int(g["ncases"])):
        P, D, group, nb, T = (int(x) for x in g[f"c{c}_meta"])
        assert np.array_equal(np.asarray(policies.ladder_bits(P, D, group), np.float32), g[f"c{c}_bits"])
        hot = policies.hot_mask(nb, T - 1, P, sinks=4, window=128)
        assert np.array_equal(hot.numpy().astype(np.uint8), g[f"c{c}_hot"])


def test_blockify_pads_with_the_last_row():
    x = torch.arange(70 * 3, dtype=torch.float32).view(70, 3)
    blocks, pad = policies.blockify(x, 64)
    assert blocks.shape == (2, 64, 3) and pad == 58
    assert blocks[1, 6:].eq(x[-1]).all()


def test_quant_grouped_matches_reference(golden):
    """policies.py:82-112 on a reference-made fixture: every bit width, group size and both groupings."""
    import torch
    from geodesia_kv_b200.policies import quant_grouped
    g = golden("quant_grouped")
    x = torch.from_numpy(g["x"])
    for bits in (16, 8, 4, 2):
        for group in (16, 32):
            for pc in (True, False):
                rec, smax = quant_grouped(x.clone(), bits, group, pc)
                key = f"b{bits}_g{group}_pc{int(pc)}"
                assert rec.shape == x.shape
                assert np.array_equal(rec.numpy(), g["rec_" + key]), key
                assert np.array_equal(smax.numpy(), g["smax_" + key]), key
