"""ctypes front end of the CPU oracle (``gkv_oracle.c``).  TEST INFRASTRUCTURE ONLY.

The shipped package never imports this module: it is the checker used by the
tests, the smoke check and the CPU-baseline leg of the benchmark.  All arrays
are numpy; nothing here touches CUDA or torch.

The library is built by ``make -C oracle`` (or :func:`build`).
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB = None

LADDER = (16, 8, 4, 2, 1)          # geodesia_kv/policies.py:1576 without the spectral rung


def build(force: bool = False) -> Path:
    so = _HERE / "libgkv_oracle.so"
    src = _HERE / "gkv_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-B", "-C", str(_HERE)], check=True, capture_output=True)
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = _HERE / "libgkv_oracle.so"
        if not so.exists():
            build()
        _LIB = C.CDLL(str(so))
        _LIB.gkv_oracle_level_bits.restype = C.c_double
        _LIB.gkv_oracle_level_bits.argtypes = [C.c_int] * 4
        _LIB.gkv_oracle_block_bytes.restype = C.c_int64
        _LIB.gkv_oracle_pack_bits.restype = C.c_int64
        _LIB.gkv_oracle_pack_block.restype = C.c_int64
    return _LIB


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads() -> int:
    return int(lib().gkv_oracle_num_threads())


def set_threads(n: int) -> None:
    lib().gkv_oracle_set_threads(C.c_int(n))


def pack_bits(codes: np.ndarray, bits: int) -> np.ndarray:
    codes = _c(codes, np.uint8).reshape(-1)
    per = 8 // bits
    out = np.zeros((codes.size + per - 1) // per, np.uint8)
    lib().gkv_oracle_pack_bits(_p(codes), C.c_int64(codes.size), C.c_int(bits), _p(out))
    return out


def unpack_bits(packed: np.ndarray, bits: int, n: int) -> np.ndarray:
    packed = _c(packed, np.uint8).reshape(-1)
    out = np.zeros(n, np.uint8)
    lib().gkv_oracle_unpack_bits(_p(packed), C.c_int64(n), C.c_int(bits), _p(out))
    return out


def block_bytes(level: int, P: int, D: int) -> int:
    return int(lib().gkv_oracle_block_bytes(C.c_int(level), C.c_int(P), C.c_int(D)))


def level_bits(level: int, P: int, D: int, group: int) -> float:
    return float(lib().gkv_oracle_level_bits(level, P, D, group))


def quantize_codes(x: np.ndarray, bits: int, group: int, per_channel: bool):
    """x (P, D) fp32 -> (codes (P, D) u8, lo16, step16 as uint16 bit patterns)."""
    x = _c(x, np.float32)
    P, D = x.shape
    shape = (P // min(group, P), D) if per_channel else (P, D // min(group, D))
    codes = np.zeros((P, D), np.uint8)
    lo = np.zeros(shape, np.uint16)
    step = np.zeros(shape, np.uint16)
    lib().gkv_oracle_quantize_codes(_p(x), C.c_int(P), C.c_int(D), C.c_int(bits), C.c_int(group),
                                    C.c_int(int(per_channel)), _p(codes), _p(lo), _p(step))
    return codes, lo, step


def dequant_block(blk: np.ndarray, level: int, P: int, D: int, group: int, klo, kstep, vlo, vstep):
    """Bytes of one block (+ its scale planes as uint16) -> (K, V) fp32 (P, D)."""
    blk = _c(blk, np.uint8)
    k = np.zeros((P, D), np.float32)
    v = np.zeros((P, D), np.float32)
    klo, kstep, vlo, vstep = (_c(a, np.uint16) for a in (klo, kstep, vlo, vstep))
    lib().gkv_oracle_dequant_block(_p(blk), C.c_int(level), C.c_int(P), C.c_int(D), C.c_int(group),
                                   _p(klo), _p(kstep), _p(vlo), _p(vstep), _p(k), _p(v))
    return k, v


def pack_row(k: np.ndarray, v: np.ndarray, levels, group: int):
    """Dense (nb, P, D) fp32 K and V of ONE cache row -> the kernel byte layout.

    Returns a dict with the keys of the reference's ``build_layout``
    (geodesia_kv/pack_layout.py:14-54): data, offs, klo, kstep, vlo, vstep
    (uint16 bit patterns of fp16), level, valid (all 64), nbytes.
    """
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    nb, P, D = k.shape
    G, gv = (P + group - 1) // group, (D + group - 1) // group
    levels = [int(x) for x in levels]
    sizes = [block_bytes(lv, P, D) for lv in levels]
    offs = np.zeros(nb, np.int64)
    if nb:
        offs[1:] = np.cumsum(sizes)[:-1]
    data = np.zeros(int(sum(sizes)), np.uint8)
    klo = np.zeros((nb, G, D), np.uint16)
    kstep = np.zeros((nb, G, D), np.uint16)
    vlo = np.zeros((nb, P, gv), np.uint16)
    vstep = np.zeros((nb, P, gv), np.uint16)
    L = lib()
    for b, lv in enumerate(levels):
        blk = data[offs[b]: offs[b] + sizes[b]]
        L.gkv_oracle_pack_block(_p(k[b]), _p(v[b]), C.c_int(lv), C.c_int(P), C.c_int(D),
                                C.c_int(group), C.c_void_p(data.ctypes.data + int(offs[b])),
                                _p(klo[b]), _p(kstep[b]), _p(vlo[b]), _p(vstep[b]))
        del blk
    return {"data": data, "offs": offs, "klo": klo, "kstep": kstep, "vlo": vlo, "vstep": vstep,
            "level": np.asarray(levels, np.int32), "valid": np.full(nb, P, np.int32),
            "nbytes": int(data.size + klo.size * 4 + vlo.size * 4)}


def mixed_attn_decode(q, data, offs, klo, kstep, vlo, vstep, level, valid, P: int, group: int):
    """Oracle of ``mixed_attn_decode`` with the GQA / per-row-metadata supersets.

    q (B, Hq, D) fp32 pre-scaled; data (B, Hkv, nbytes) u8; klo/kstep
    (B, Hkv, nb, G, D) and vlo/vstep (B, Hkv, nb, P, gv) as uint16 fp16 bits;
    offs/level/valid either (nb,) shared or (B, Hkv, nb).  Returns (B, Hq, D) fp32.
    """
    q = _c(q, np.float32)
    data = _c(data, np.uint8)
    B, Hq, D = q.shape
    Hkv = data.shape[1]
    level = _c(level, np.int32)
    nb = level.shape[-1]
    meta_rows = 1 if level.ndim == 1 else B * Hkv
    offs = _c(offs, np.int64)
    valid = _c(valid, np.int32)
    klo, kstep, vlo, vstep = (_c(a, np.uint16) for a in (klo, kstep, vlo, vstep))
    out = np.zeros((B, Hq, D), np.float32)
    rc = lib().gkv_oracle_mixed_attn_decode(
        _p(q), _p(data), _p(offs), _p(klo), _p(kstep), _p(vlo), _p(vstep), _p(level), _p(valid),
        _p(out), C.c_int(B), C.c_int(Hq), C.c_int(Hkv), C.c_int(D), C.c_int(nb), C.c_int(P),
        C.c_int(group), C.c_int64(data.shape[-1]), C.c_int(meta_rows))
    if rc != 0:
        raise ValueError(f"oracle rejected the shapes (rc={rc})")
    return out


def block_mass(q, data, offs, klo, kstep, vlo, vstep, level, valid, P: int, group: int) -> np.ndarray:
    """Softmax mass per block: for every cache row the mean over its query heads of the summed softmax
    weight of each block's tokens, (B, Hkv, nb) fp32 — the `shared_mass` that the reference's hook gets
    from a dense softmax of the current query over all keys (geodesia_kv/policies.py:1497-1509), here
    over the de-quantised keys of the packed cache.  fp64 throughout; blocks without valid tokens get 0."""
    q = _c(q, np.float32)
    B, Hq, D = q.shape
    Hkv = data.shape[1]
    rep = Hq // Hkv
    level, valid, offs = np.asarray(level), np.asarray(valid), np.asarray(offs)
    nb = level.shape[-1]
    out = np.zeros((B, Hkv, nb), np.float32)
    for b in range(B):
        for h in range(Hkv):
            lv, va, of = (a if a.ndim == 1 else a[b, h] for a in (level, valid, offs))
            scores, owner = [], []
            for i in range(nb):
                n = int(va[i])
                if n <= 0:
                    continue
                nbytes = block_bytes(int(lv[i]), P, D)
                kd, _ = dequant_block(data[b, h, int(of[i]): int(of[i]) + nbytes], int(lv[i]), P, D, group,
                                      klo[b, h, i], kstep[b, h, i], vlo[b, h, i], vstep[b, h, i])
                scores.append(q[b, h * rep:(h + 1) * rep].astype(np.float64) @ kd[:n].astype(np.float64).T)
                owner += [i] * n
            if not scores:
                continue
            s = np.concatenate(scores, 1)
            w = np.exp(s - s.max(1, keepdims=True))
            w /= w.sum(1, keepdims=True)
            np.add.at(out[b, h], np.asarray(owner), w.mean(0))
    return out


def distortion(krec, vrec, group: int, value_weight: float = 0.0) -> np.ndarray:
    krec = _c(krec, np.float32)
    vrec = _c(vrec, np.float32)
    nb, P, D = krec.shape
    E = np.zeros((nb, 5), np.float32)
    lib().gkv_oracle_distortion(_p(krec), _p(vrec), C.c_int(nb), C.c_int(P), C.c_int(D),
                                C.c_int(group), C.c_float(value_weight), _p(E))
    return E


def allocate(mass, E, idx, hot, bits, target_bits: float, mass_power: float = 1.0):
    """Rung allocator.  Returns (target ladder index per block, ratio table (nb, 4))."""
    mass = _c(mass, np.float32)
    E = _c(E, np.float32)
    idx = _c(idx, np.int32)
    hot = _c(hot, np.uint8)
    bits = _c(bits, np.float32)
    nb = mass.shape[0]
    tgt = np.zeros(nb, np.int32)
    ratio = np.zeros((nb, 4), np.float32)
    lib().gkv_oracle_allocate(_p(mass), _p(E), _p(idx), _p(hot), C.c_int(nb), _p(bits),
                              C.c_double(target_bits), C.c_float(mass_power), _p(tgt), _p(ratio))
    return tgt, ratio
