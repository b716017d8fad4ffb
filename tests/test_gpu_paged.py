"""The paged pool on the GPU: blocks packed and demoted into size-class slots are the oracle's
bytes, demotion gives pool bytes back, and one kernel call attends over a ragged batch."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

P = 64
LADDER = (16, 8, 4, 2, 1)


def dense_batch(seed, B, Hkv, T, D, device="cuda"):
    gen = torch.Generator(device=device).manual_seed(seed)
    k = torch.randn(B, Hkv, T, D, device=device, generator=gen).to(torch.bfloat16)
    v = torch.randn(B, Hkv, T, D, device=device, generator=gen).to(torch.bfloat16)
    k[..., 5] *= 8.0                                            # an outlier channel
    return k, v


def rows_for_oracle(layer):
    """The paged cache as the row-form arrays the oracle takes (padding entries: valid 0, rung 16)."""
    pool = layer.pool.data.cpu().numpy()
    D, g = layer.D, layer.group
    G, gv = P // min(g, P), D // min(g, D)
    nb = layer.nb
    B, Hkv = layer.B, layer.Hkv
    valid = layer.valid.cpu().numpy()[:, :nb].reshape(B, Hkv, nb).copy()
    level = layer.level_h[:, :nb].reshape(B, Hkv, nb).copy()
    offs_p = layer.offs_h[:, :nb].reshape(B, Hkv, nb)
    sizes = np.where(level == 1, 4 * D, np.where(level == 16, 4 * P * D, np.where(level == 0, 0, 2 * P * D * level // 8)))
    stride = int(max(sizes.sum(-1).max(), 4 * P * D))
    out = {"data": np.zeros((B, Hkv, stride), np.uint8), "offs": np.zeros((B, Hkv, nb), np.int64),
           "klo": np.zeros((B, Hkv, nb, G, D), np.uint16), "kstep": np.zeros((B, Hkv, nb, G, D), np.uint16),
           "vlo": np.zeros((B, Hkv, nb, P, gv), np.uint16), "vstep": np.zeros((B, Hkv, nb, P, gv), np.uint16)}
    for b in range(B):
        for h in range(Hkv):
            cur = 0
            for i in range(nb):
                lv, n = int(level[b, h, i]), int(sizes[b, h, i])
                if lv == 0:
                    level[b, h, i], valid[b, h, i] = 16, 0
                    continue
                o = int(offs_p[b, h, i])
                out["data"][b, h, cur:cur + n] = pool[o:o + n]
                out["offs"][b, h, i] = cur
                cur += n
                if lv in (8, 4, 2):
                    s = pool[o + n:o + n + 4 * (G * D + P * gv)].view(np.uint16)
                    out["klo"][b, h, i] = s[:G * D].reshape(G, D)
                    out["kstep"][b, h, i] = s[G * D:2 * G * D].reshape(G, D)
                    out["vlo"][b, h, i] = s[2 * G * D:2 * G * D + P * gv].reshape(P, gv)
                    out["vstep"][b, h, i] = s[2 * G * D + P * gv:].reshape(P, gv)
    out["level"], out["valid"] = level.astype(np.int32), valid.astype(np.int32)
    return out


def power_law_mass(layer, exponent=1.2, sink=0.1):
    """Mass per block ~ (distance in blocks from the newest + 1)^-exponent, normalised, + a sink mass."""
    nbr = np.repeat(layer.blocks_per_seq(), layer.Hkv)
    nb = layer.nb
    b = np.arange(nb)[None, :]
    m = np.where(b < nbr[:, None], np.maximum(nbr[:, None] - b, 1).astype(np.float64) ** -exponent, 0.0)
    m /= m.sum(1, keepdims=True)
    m[:, 0] += sink
    return torch.from_numpy(m.astype(np.float32)).to(layer.device)


@pytest.mark.parametrize("D,group", [(128, 32), (64, 32), (128, 16), (128, 64)])
def test_blocks_packed_into_slots_are_the_oracles_bytes(oracle, D, group):
    from geodesia_kv_b200.paged import PagedLayerCache, PagedPool
    B, Hkv, nb = 2, 2, 11
    pool = PagedPool(64 << 20, D, group)
    layer = PagedLayerCache(pool, B, Hkv)
    k, v = dense_batch(5 + D + group, B, Hkv, nb * P, D)
    rng = np.random.default_rng(D + group)
    levels = rng.choice(np.array(LADDER), size=(B * Hkv, nb)).astype(np.int32)
    n = B * Hkv * nb
    slots = np.empty(n, dtype=np.int64)
    flat = levels.reshape(-1)
    for rung in LADDER:
        sel = np.nonzero(flat == rung)[0]
        slots[sel] = pool.alloc(rung, sel.size)
    assert len(set(slots.tolist())) == n and all(int(s) % 128 == 0 for s in slots)
    src = np.arange(n, dtype=np.int64) * P * D
    ek, ev = layer.pack_blocks(k, v, src, D, np.full(n, P, np.int32), slots, flat, radii=True)
    torch.cuda.synchronize()
    data = pool.data.cpu().numpy()
    kf, vf = k.float().cpu().numpy().reshape(B * Hkv, nb, P, D), v.float().cpu().numpy().reshape(B * Hkv, nb, P, D)
    G, gv = P // min(group, P), D // min(group, D)
    ek, ev = ek.cpu().numpy().reshape(B * Hkv, nb), ev.cpu().numpy().reshape(B * Hkv, nb)
    for r in range(B * Hkv):
        want = oracle.pack_row(kf[r], vf[r], levels[r], group)
        for i in range(nb):
            lv = int(levels[r, i])
            o, wo = int(slots[r * nb + i]), int(want["offs"][i])
            nbytes = oracle.block_bytes(lv, P, D)
            assert np.array_equal(data[o:o + nbytes], want["data"][wo:wo + nbytes]), (r, i, lv)
            if lv in (8, 4, 2):
                s = data[o + nbytes:o + nbytes + 4 * (G * D + P * gv)].view(np.uint16)
                assert np.array_equal(s[:G * D], want["klo"][i].reshape(-1)), (r, i, "klo")
                assert np.array_equal(s[G * D:2 * G * D], want["kstep"][i].reshape(-1))
                assert np.array_equal(s[2 * G * D:2 * G * D + P * gv], want["vlo"][i].reshape(-1))
                assert np.array_equal(s[2 * G * D + P * gv:], want["vstep"][i].reshape(-1))
            # error radii: max over tokens of |x - q(x)|
            kd, vd = oracle.dequant_block(want["data"][wo:wo + nbytes], lv, P, D, group, want["klo"][i], want["kstep"][i],
                                          want["vlo"][i], want["vstep"][i])
            rk = np.linalg.norm(kf[r, i] - kd, axis=-1).max()
            rv = np.linalg.norm(vf[r, i] - vd, axis=-1).max()
            assert abs(ek[r, i] - rk) <= 1e-4 * max(1.0, rk) and abs(ev[r, i] - rv) <= 1e-4 * max(1.0, rv), (r, i, lv)


def test_demotion_gives_pool_bytes_back_and_matches_the_oracle(oracle):
    from geodesia_kv_b200.paged import PagedLayerCache, PagedPool
    D, group, B, Hkv = 128, 32, 3, 2
    lengths = [64 * 40, 64 * 25 + 17, 64 * 33]
    pool = PagedPool(256 << 20, D, group)
    layer = PagedLayerCache(pool, B, Hkv)
    T = max(lengths)
    k, v = dense_batch(11, B, Hkv, T, D)
    layer.prefill(k, v, lengths)
    before = pool.bytes_in_use
    dense_bytes = sum((n + P - 1) // P for n in lengths) * Hkv * 4 * P * D
    assert before == dense_bytes == layer.bytes_in_pool()
    budget = 4.0
    n = layer.maintain(budget, mass=power_law_mass(layer))
    torch.cuda.synchronize()
    assert n > 0
    after = pool.bytes_in_use
    assert after < before and after == layer.bytes_in_pool()
    # resident bits respect the budget (the reference's accounting), and so do the pool bytes up to
    # the scale planes' share and the blocks that must stay exact
    assert layer.bits_per_value() <= budget + 1e-6
    assert after <= budget / 16.0 * dense_bytes * 1.05
    # every block now holds the oracle's bytes for its rung, made from the bf16 values
    c = rows_for_oracle(layer)
    for r in range(B * Hkv):
        b, h = divmod(r, Hkv)
        nbr = (lengths[b] + P - 1) // P
        kf = torch.nn.functional.pad(k[b, h, :lengths[b]].float(), (0, 0, 0, nbr * P - lengths[b]))
        vf = torch.nn.functional.pad(v[b, h, :lengths[b]].float(), (0, 0, 0, nbr * P - lengths[b]))
        kf, vf = kf.cpu().numpy().reshape(nbr, P, D), vf.cpu().numpy().reshape(nbr, P, D)
        tail = lengths[b] % P
        if tail:                                                # a short last block repeats its last row
            kf[-1, tail:] = kf[-1, tail - 1]
            vf[-1, tail:] = vf[-1, tail - 1]
        lv = c["level"][b, h, :nbr]
        want = oracle.pack_row(kf, vf, lv, group)
        for i in range(nbr):
            o, wo, nbytes = int(c["offs"][b, h, i]), int(want["offs"][i]), oracle.block_bytes(int(lv[i]), P, D)
            assert np.array_equal(c["data"][b, h, o:o + nbytes], want["data"][wo:wo + nbytes]), (r, i, int(lv[i]))
        for key in ("klo", "kstep", "vlo", "vstep"):
            assert np.array_equal(c[key][b, h, :nbr], want[key]), key
    assert (layer.ek.cpu().numpy()[layer.level_h != 16] >= 0).all()
    demoted = (layer.level_h != 16) & (layer.level_h != 0)
    assert (layer.ek.cpu().numpy()[demoted] > 0).all() and (layer.ev.cpu().numpy()[demoted] > 0).all()
    # a second pass at the same budget changes nothing; a tighter one never promotes (and, as in the
    # reference, a block that has left rung 16 is not moved again)
    lv0 = layer.level_h.copy()
    assert layer.maintain(budget, mass=power_law_mass(layer)) == 0
    layer.maintain(2.5, mass=power_law_mass(layer))
    assert (layer.level_h <= lv0).all() and pool.bytes_in_use <= after
    layer.release()
    assert pool.bytes_in_use == 0 and pool.bytes_reserved == 0


def test_pool_bytes_stay_within_budget_over_64_appended_blocks(oracle):
    """Blocks are appended one at a time (64 tokens each, one token per call) with maintenance after
    every closed block: the pool bytes in use stay under budget x dense bytes plus the blocks that
    must stay exact, although 64 exact blocks per row come in."""
    from geodesia_kv_b200.paged import PagedLayerCache, PagedPool
    D, group, B, Hkv, budget = 128, 32, 2, 2, 4.0
    pool = PagedPool(192 << 20, D, group)
    layer = PagedLayerCache(pool, B, Hkv)
    lengths = [64 * 16, 64 * 9]
    k, v = dense_batch(21, B, Hkv, max(lengths), D)
    layer.prefill(k, v, lengths)
    layer.maintain(budget, mass=power_law_mass(layer))
    gen = torch.Generator(device="cuda").manual_seed(3)
    exact_slack = B * Hkv * 5 * 4 * P * D                       # sinks, window, the open block and its predecessor
    fell = 0
    for blk in range(64):
        toks = torch.randn(64, B, Hkv, D, device="cuda", generator=gen).to(torch.bfloat16)
        for t in range(64):
            layer.append(toks[t], toks[t] * 0.5)
        in_use = pool.bytes_in_use
        layer.maintain(budget, mass=power_law_mass(layer))
        fell += pool.bytes_in_use < in_use
        dense = int(layer.blocks_per_seq().sum()) * Hkv * 4 * P * D
        assert pool.bytes_in_use <= budget / 16.0 * dense * 1.05 + exact_slack, blk
        assert layer.bits_per_value() <= budget + 16.0 * 5 / int(layer.blocks_per_seq().min()) + 1e-6
    assert fell >= 60 and int(layer.status.item()) == 0
    assert layer.len_h.tolist() == [64 * 80, 64 * 73] and layer.lens.cpu().tolist() == [64 * 80] * 2 + [64 * 73] * 2


@pytest.mark.parametrize("Hq,Hkv", [(16, 2), (8, 4)])
def test_ragged_batch_decode_matches_the_oracle(oracle, Hq, Hkv):
    from geodesia_kv_b200.paged import PagedLayerCache, PagedPool
    D, group = 128, 32
    lengths = [70, 64 * 30, 333, 64, 64 * 45 + 1, 1]
    B = len(lengths)
    pool = PagedPool(512 << 20, D, group)
    layer = PagedLayerCache(pool, B, Hkv)
    k, v = dense_batch(31 + Hq, B, Hkv, max(lengths), D)
    layer.prefill(k, v, lengths)
    layer.maintain(3.0, mass=power_law_mass(layer), window=64)
    gen = torch.Generator(device="cuda").manual_seed(9)
    q = (torch.randn(B, Hq, D, device="cuda", generator=gen) * D ** -0.5).contiguous()
    out, mass = layer.attend(q, want_mass=True)
    out2 = layer.attend(q)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    c = rows_for_oracle(layer)
    want = oracle.mixed_attn_decode(q.cpu().numpy(), c["data"], c["offs"], c["klo"], c["kstep"], c["vlo"], c["vstep"],
                                    c["level"], c["valid"], P, group)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-3       # the tolerance the reference's kernel test uses
    wm = oracle.block_mass(q.cpu().numpy(), c["data"], c["offs"], c["klo"], c["kstep"], c["vlo"], c["vstep"],
                           c["level"], c["valid"], P, group).reshape(B * Hkv, -1)
    got = mass.cpu().numpy()
    assert np.abs(got[:, :wm.shape[1]] - wm).max() <= 1e-5 and np.abs(got[:, wm.shape[1]:]).max(initial=0) == 0
    assert len(set(layer.level_h[layer.level_h > 0].tolist())) >= 3          # the batch really is mixed


def test_tokens_appended_on_the_device_are_attended(oracle):
    from geodesia_kv_b200.paged import PagedLayerCache, PagedPool
    D, group, B, Hkv, Hq = 128, 32, 3, 2, 8
    pool = PagedPool(64 << 20, D, group)
    layer = PagedLayerCache(pool, B, Hkv, cap_blocks=4)
    lengths = [130, 64, 5]
    k, v = dense_batch(41, B, Hkv, 200, D)
    layer.prefill(k, v, lengths)
    gen = torch.Generator(device="cuda").manual_seed(10)
    steps = 70
    new_k = torch.randn(steps, B, Hkv, 1, D, device="cuda", generator=gen).to(torch.bfloat16)
    new_v = torch.randn(steps, B, Hkv, 1, D, device="cuda", generator=gen).to(torch.bfloat16)
    for s in range(steps):
        layer.append(new_k[s], new_v[s])
    torch.cuda.synchronize()
    assert int(layer.status.item()) == 0
    kk, vv = layer.dequantise()
    for b in range(B):
        for h in range(Hkv):
            n = lengths[b]
            want_k = torch.cat([k[b, h, :n], new_k[:, b, h, 0]]).float()
            want_v = torch.cat([v[b, h, :n], new_v[:, b, h, 0]]).float()
            assert torch.equal(kk[b * Hkv + h, :n + steps], want_k) and torch.equal(vv[b * Hkv + h, :n + steps], want_v)
    q = (torch.randn(B, Hq, D, device="cuda", generator=gen) * D ** -0.5).contiguous()
    out = layer.attend(q)
    c = rows_for_oracle(layer)
    want = oracle.mixed_attn_decode(q.cpu().numpy(), c["data"], c["offs"], c["klo"], c["kstep"], c["vlo"], c["vstep"],
                                    c["level"], c["valid"], P, group)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-3
    # a row whose next block has no slot is reported, not written
    layer.offs[0, int(layer.len_h[0]) // P + 1:] = -1
    for _ in range(64):
        layer.append_device(new_k[0], new_v[0])
    torch.cuda.synchronize()
    assert int(layer.status.item()) == 1


@pytest.mark.parametrize("budget", [2.0, 3.0, 4.0, 5.0])
def test_one_block_per_step_for_64_steps_against_the_oracle(oracle, budget):
    """The maintenance scenario end to end on the packed cache: one 64-token block is appended to every
    row per step for 64 steps, the distortion, allocator and demotion kernels run after each, and every
    step is compared with the oracle — the rung of every block (bit-exact), the bytes and scale planes
    of every block demoted in the step (bit-exact), monotone demotion (policies.py:810-908)."""
    from geodesia_kv_b200 import policies
    from geodesia_kv_b200.paged import PagedLayerCache, PagedPool
    D, group, B, Hkv, nb0, steps = 128, 32, 2, 2, 8, 64
    rows = B * Hkv
    pool = PagedPool(192 << 20, D, group)
    layer = PagedLayerCache(pool, B, Hkv)
    gen = torch.Generator(device="cuda").manual_seed(int(2000 + budget))
    k = torch.randn(B, Hkv, (nb0 + steps) * P, D, device="cuda", generator=gen).to(torch.bfloat16)
    v = torch.randn(B, Hkv, (nb0 + steps) * P, D, device="cuda", generator=gen).to(torch.bfloat16)
    kf = k.float().cpu().numpy().reshape(rows, nb0 + steps, P, D)
    vf = v.float().cpu().numpy().reshape(rows, nb0 + steps, P, D)
    bits = np.asarray(policies.ladder_bits(P, D, group), np.float32)
    G, gv = P // group, D // group
    layer.extend(k[:, :, :nb0 * P], v[:, :, :nb0 * P])
    idx = np.zeros((rows, nb0), np.int32)
    E_all = np.stack([oracle.distortion(kf[r], vf[r], group, 0.0) for r in range(rows)])
    demoted_total = 0
    for step in range(steps + 1):
        nb = nb0 + step
        if step:
            layer.extend(k[:, :, (nb - 1) * P:nb * P], v[:, :, (nb - 1) * P:nb * P])
            idx = np.concatenate([idx, np.zeros((rows, 1), np.int32)], 1)
        mass = power_law_mass(layer)
        tgt = layer.plan_demotion(budget, mass=mass).cpu().numpy()
        hot = layer.hot_blocks(nb).cpu().numpy()
        assert np.array_equal(hot[0], policies.hot_mask(nb, nb * P - 1, P, 4, 128).numpy().astype(np.uint8))
        mh = mass.cpu().numpy()
        for r in range(rows):
            E = np.where((idx[r] == 0)[:, None], E_all[r, :nb], 0.0).astype(np.float32)   # demoted blocks carry a zero row
            want, _ = oracle.allocate(mh[r], E, idx[r], hot[r], bits, budget * 2.0 * nb * P * D)
            assert np.array_equal(tgt[r], want), (step, r)
        assert (tgt >= idx).all() and np.array_equal(tgt[idx > 0], idx[idx > 0])
        moved = np.argwhere(tgt > idx)
        assert layer.apply_demotion(tgt) == len(moved)
        demoted_total += len(moved)
        if len(moved):
            data = pool.data.cpu().numpy()
            for r, b in moved:
                lv = LADDER[tgt[r, b]]
                want = oracle.pack_row(kf[r, b:b + 1], vf[r, b:b + 1], [lv], group)
                o, nbytes = int(layer.offs_h[r, b]), oracle.block_bytes(lv, P, D)
                assert int(layer.level_h[r, b]) == lv
                assert np.array_equal(data[o:o + nbytes], want["data"]), (step, r, b, lv)
                if lv in (8, 4, 2):
                    s = data[o + nbytes:o + nbytes + 4 * (G * D + P * gv)].view(np.uint16)
                    got = (s[:G * D], s[G * D:2 * G * D], s[2 * G * D:2 * G * D + P * gv], s[2 * G * D + P * gv:])
                    for a, key in zip(got, ("klo", "kstep", "vlo", "vstep")):
                        assert np.array_equal(a, want[key].reshape(-1)), (step, r, b, key)
        idx = tgt
        assert pool.bytes_in_use == layer.bytes_in_pool()
    assert demoted_total >= rows * (steps - 4)
    assert layer.bits_per_value() <= budget + 16.0 * 5 / (nb0 + steps) + 1e-6
    # none of the pack/demote kernels' bounded waits ever ran out
    import ctypes
    word = ctypes.c_int(-1)
    assert layer.lib.gkv_maintenance_status(ctypes.byref(word)) == 0 and word.value == 0


def test_serving_manager_stores_sequences_in_one_pool_and_frees_them():
    """The reference's manager (vllm_plugin/kv_cache.py:85-104) with a pool attached: sequences of
    different lengths share it, each occupies what its rungs cost, freeing one gives that back."""
    from geodesia_kv_b200.vllm_plugin import GeodesiaKVCacheManager
    L, H, Dh = 3, 2, 128
    mgr = GeodesiaKVCacheManager(block_size=64, target_bpv=4.0, num_layers=L)
    pool = mgr.attach_pool(256 << 20, Dh, 32)
    gen = torch.Generator(device="cuda").manual_seed(8)
    used = {}
    for seq_id, T in ((7, 64 * 20), (8, 64 * 5 + 9), (9, 64 * 33)):
        c = mgr.create_sequence_cache(seq_id)
        k = torch.randn(L, T, H, Dh, device="cuda", generator=gen).to(torch.bfloat16)
        bpv = c.compress_sequence_kv(k, k * 0.5)
        assert 4.0 < bpv < 8.0                   # 4-bit blocks with their scales, the last block exact
        nb = (T + 63) // 64
        want = L * H * ((nb - 1) * pool.slot[4] + pool.slot[16])          # 4-bit ladder, last block exact
        assert c.pool_bytes() == want
        used[seq_id] = want
        # the pool copy attends like the row-form copy of the same sequence
        q = (torch.randn(1, 8, Dh, device="cuda", generator=gen) * Dh ** -0.5).contiguous()
        from geodesia_kv_b200.cuda_ext import get_ext
        a = c.paged_layers[1].attend(q)
        b = get_ext().mixed_attn_decode(q, *c.kernel_layers[1].kernel_args())
        assert (a - b).abs().max().item() < 1e-5
    assert pool.bytes_in_use == sum(used.values())
    mgr.free_sequence_cache(8)
    assert pool.bytes_in_use == used[7] + used[9] and 8 not in mgr.active_caches
    mgr.free_sequence_cache(7)
    mgr.free_sequence_cache(9)
    assert pool.bytes_in_use == 0 and pool.bytes_reserved == 0


@pytest.mark.parametrize("D,group,Hq,Hkv", [(64, 32, 8, 2), (128, 16, 4, 4), (64, 16, 14, 2), (128, 64, 16, 2)])
def test_other_shapes_through_the_pool(oracle, D, group, Hq, Hkv):
    """Head dim 64, groups 16 and 64, GQA widths 1, 2, 7, 8: prompts of odd lengths, demotion, tokens appended
    across block boundaries, then one call over the ragged batch against the oracle."""
    from geodesia_kv_b200.paged import PagedLayerCache, PagedPool
    lengths = [64 * 9 + 31, 5, 64 * 14]
    B = len(lengths)
    pool = PagedPool(128 << 20, D, group)
    layer = PagedLayerCache(pool, B, Hkv, cap_blocks=8)
    k, v = dense_batch(D + group + Hq, B, Hkv, max(lengths), D)
    layer.prefill(k, v, lengths)
    layer.maintain(3.5, mass=power_law_mass(layer), window=64)
    gen = torch.Generator(device="cuda").manual_seed(D)
    for _ in range(70):
        layer.append(torch.randn(B, Hkv, 1, D, device="cuda", generator=gen).to(torch.bfloat16),
                     torch.randn(B, Hkv, 1, D, device="cuda", generator=gen).to(torch.bfloat16))
    layer.maintain(3.5, mass=power_law_mass(layer), window=64)
    q = (torch.randn(B, Hq, D, device="cuda", generator=gen) * D ** -0.5).contiguous()
    out, mass = layer.attend(q, want_mass=True)
    torch.cuda.synchronize()
    assert int(layer.status.item()) == 0 and layer.len_h.tolist() == [n + 70 for n in lengths]
    c = rows_for_oracle(layer)
    args = (c["data"], c["offs"], c["klo"], c["kstep"], c["vlo"], c["vstep"], c["level"], c["valid"], P, group)
    want = oracle.mixed_attn_decode(q.cpu().numpy(), *args)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-3
    wm = oracle.block_mass(q.cpu().numpy(), *args).reshape(B * Hkv, -1)
    assert np.abs(mass.cpu().numpy()[:, :wm.shape[1]] - wm).max() <= 1e-5
    assert pool.bytes_in_use == layer.bytes_in_pool()
    assert (layer.level_h[layer.level_h > 0] < 16).any()
