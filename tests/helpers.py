"""Builders shared by the parity tests: seeded caches packed by the CPU oracle."""
from __future__ import annotations

import numpy as np


def categorical_levels(rng, nb, probs=(0.10, 0.20, 0.40, 0.20, 0.10), force_ends=True):
    lv = rng.choice(np.array([16, 8, 4, 2, 1]), size=nb, p=np.asarray(probs))
    if force_ends and nb:
        lv[0] = 16
        lv[-1] = 16
    return lv.astype(np.int32)


def oracle_cache(oracle, seed, B, Hkv, nb, D, group, probs=(0.10, 0.20, 0.40, 0.20, 0.10), outliers=4,
                 last_valid=64, shared_meta=False, levels=None):
    """Dense seeded K/V -> packed rows via the oracle.  Returns a dict of numpy arrays shaped
    like the kernel arguments plus the dense inputs."""
    rng = np.random.default_rng(seed)
    P = 64
    G, gv = (P + group - 1) // group, (D + group - 1) // group
    rows = []
    shared = categorical_levels(rng, nb, probs) if levels is None else np.asarray(levels, np.int32)
    kd = np.zeros((B, Hkv, nb, P, D), np.float32)
    vd = np.zeros((B, Hkv, nb, P, D), np.float32)
    for b in range(B):
        for h in range(Hkv):
            k = rng.standard_normal((nb, P, D), dtype=np.float32)
            v = rng.standard_normal((nb, P, D), dtype=np.float32)
            if outliers:
                k[:, :, rng.permutation(D)[:outliers]] *= 8.0
            lv = shared if (shared_meta or levels is not None) else categorical_levels(rng, nb, probs)
            kd[b, h], vd[b, h] = k, v
            rows.append(oracle.pack_row(k, v, lv, group))
    stride = max([r["data"].size for r in rows] + [0])
    stride = (stride + 255) // 256 * 256
    data = np.zeros((B, Hkv, stride), np.uint8)
    out = {"data": data, "k": kd, "v": vd}
    for key, shape, dt in (("klo", (G, D), np.uint16), ("kstep", (G, D), np.uint16),
                           ("vlo", (P, gv), np.uint16), ("vstep", (P, gv), np.uint16)):
        out[key] = np.zeros((B, Hkv, nb) + shape, dt)
    out["offs"] = np.zeros((B, Hkv, nb), np.int64)
    out["level"] = np.zeros((B, Hkv, nb), np.int32)
    out["valid"] = np.full((B, Hkv, nb), P, np.int32)
    for i, r in enumerate(rows):
        b, h = divmod(i, Hkv)
        data[b, h, :r["data"].size] = r["data"]
        for key in ("klo", "kstep", "vlo", "vstep", "offs", "level"):
            out[key][b, h] = r[key]
    if nb:
        out["valid"][..., -1] = last_valid
    if shared_meta:
        for key in ("offs", "level", "valid"):
            out[key] = out[key][0, 0].copy()
    out.update(P=P, D=D, group=group, B=B, Hkv=Hkv, nb=nb)
    return out


def to_torch(c, device):
    import torch
    t = {}
    for key in ("data", "offs", "level", "valid"):
        t[key] = torch.from_numpy(c[key]).to(device)
    for key in ("klo", "kstep", "vlo", "vstep"):
        t[key] = torch.from_numpy(c[key].view(np.int16)).view(torch.float16).to(device)
    return t


def kernel_args(t, c):
    return (t["data"], t["offs"], t["klo"], t["kstep"], t["vlo"], t["vstep"], t["level"], t["valid"],
            c["P"], c["group"])


def oracle_args(c):
    return (c["data"], c["offs"], c["klo"], c["kstep"], c["vlo"], c["vstep"], c["level"], c["valid"],
            c["P"], c["group"])
