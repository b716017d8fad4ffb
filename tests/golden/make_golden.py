"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE'S OWN PYTHON.

Run where a checkout of geodesia-ai/geodesia-kv is available:

    python tests/golden/make_golden.py --reference <path to the checkout>

Nothing from this repository's package is imported: every array written here
comes out of the reference's functions (``geodesia_kv.packed``,
``geodesia_kv.pack_layout``, ``geodesia_kv.policies`` and the ``quantize_codes``
helper of its ``tests/test_cuda_kernel.py``) on CPU.  Dense inputs are drawn
from ``numpy.random.default_rng(seed)`` so the tests can regenerate them without
storing them.  The fixtures are what pins the C oracle (``oracle/gkv_oracle.c``)
and, on a GPU, the CUDA kernels.
"""
from __future__ import annotations

import argparse
import os
import importlib.util
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def dense_inputs(seed: int, nb: int, P: int, D: int, outliers: int = 0):
    """K, V (nb, P, D) fp32.  ``outliers`` channels of K are scaled by 8."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal((nb, P, D), dtype=np.float32)
    v = rng.standard_normal((nb, P, D), dtype=np.float32)
    if outliers:
        ch = rng.permutation(D)[:outliers]
        k[:, :, ch] *= 8.0
    return k, v


def query(seed: int, *shape):
    rng = np.random.default_rng(seed + 7919)
    return rng.standard_normal(shape, dtype=np.float32)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("GEODESIA_REFERENCE"),
                    help="checkout of geodesia-ai/geodesia-kv (default: $GEODESIA_REFERENCE)")
    ap.add_argument("--only", default=None, help="write just this fixture (quant_grouped)")
    args = ap.parse_args()
    if not args.reference:
        raise SystemExit("pass --reference or set GEODESIA_REFERENCE to a checkout of the reference")
    ref = Path(args.reference)
    sys.path.insert(0, str(ref))
    import torch
    from geodesia_kv import packed as rpacked
    from geodesia_kv import policies as rpol
    from geodesia_kv.pack_layout import build_layout

    assert Path(rpacked.__file__).resolve().is_relative_to(ref.resolve()), "wrong geodesia_kv imported"
    spec = importlib.util.spec_from_file_location("ref_test_cuda_kernel", ref / "tests" / "test_cuda_kernel.py")
    rtest = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rtest)
    quantize_codes = rtest.quantize_codes
    torch.set_num_threads(1)

    def write_quant_grouped():
        """policies.py:82-112: grouped min-max quantise -> dequantise with fp32 scales, both groupings."""
        P, D = 64, 32
        k, _ = dense_inputs(900, 2, P, D, outliers=2)
        x = torch.from_numpy(k)
        x[1, :32, 5] = 0.25                       # a constant group: the step clamps at 1e-8
        blob = {}
        for bits in (16, 8, 4, 2):
            for group in (16, 32):
                for pc in (True, False):
                    rec, smax = rpol.quant_grouped(x.clone(), bits, group, pc)
                    blob[f"rec_b{bits}_g{group}_pc{int(pc)}"] = rec.numpy()
                    blob[f"smax_b{bits}_g{group}_pc{int(pc)}"] = smax.numpy()
        np.savez_compressed(HERE / "quant_grouped.npz", seed=900, P=P, D=D, nb=2, outliers=2, x=x.numpy(), **blob)

    if args.only == "quant_grouped":
        write_quant_grouped()
        return

    def build_row(k, v, levels, group):
        """tests/test_cuda_kernel.py:55-77 for one cache row, on CPU."""
        nb, P, D = k.shape
        G, gv = (P + group - 1) // group, (D + group - 1) // group
        items, krec, vrec = {}, [], []
        for b, lv in enumerate(levels):
            if lv == 16:
                items[b] = {"k": k[b], "v": v[b]}
                krec.append(k[b].to(torch.bfloat16).float())
                vrec.append(v[b].to(torch.bfloat16).float())
            elif lv == 1:
                kc = k[b].mean(0, keepdim=True).to(torch.float16)
                vc = v[b].mean(0, keepdim=True).to(torch.float16)
                items[b] = {"k": kc, "v": vc}
                krec.append(kc.float().expand(P, D))
                vrec.append(vc.float().expand(P, D))
            else:
                ck, rk, klo, kstep = quantize_codes(k[b:b + 1], lv, group, True)
                cv, rv, vlo, vstep = quantize_codes(v[b:b + 1], lv, group, False)
                items[b] = {"k": ck[0], "v": cv[0], "klo": klo.view(G, D), "kstep": kstep.view(G, D),
                            "vlo": vlo.view(P, gv), "vstep": vstep.view(P, gv)}
                krec.append(rk[0])
                vrec.append(rv[0])
        lay = build_layout(items, P, group, D, nb, torch.tensor(levels), torch.full((nb,), P), "cpu")
        return lay, torch.stack(krec), torch.stack(vrec)

    def lay_np(lay):
        out = {}
        for key in ("data", "offs", "level", "valid"):
            out[key] = lay[key].numpy()
        for key in ("klo", "kstep", "vlo", "vstep"):
            out[key] = lay[key].view(torch.int16).numpy().view(np.uint16)
        out["nbytes"] = np.int64(lay["nbytes"])
        return out

    # ---- A. the reference's known-answer configuration (tests/test_cuda_kernel.py:36-104)
    P, D, group = 64, 64, 32
    levels = [16, 8, 4, 2, 1, 4, 2, 8]
    nb, H = len(levels), 4
    k, v = dense_inputs(0, nb, P, D)
    lay, krec, vrec = build_row(torch.from_numpy(k), torch.from_numpy(v), levels, group)
    q = query(0, 1, H, D)
    refo = torch.softmax(torch.from_numpy(q).view(H, D) @ krec.view(-1, D).T, -1) @ vrec.view(-1, D)
    np.savez_compressed(HERE / "kat_mixed_d64.npz", seed=0, P=P, D=D, group=group, H=H,
                        krec=krec.numpy(), vrec=vrec.numpy(), out=refo.numpy(), **lay_np(lay))

    # ---- B. D=128, GQA 4:1, two cache rows with their own rungs, ragged last block
    P, D, group = 64, 128, 32
    Hq, Hkv = 8, 2
    nb = 10
    rows_levels = [[16, 2, 4, 8, 1, 4, 2, 1, 8, 16], [16, 4, 4, 1, 2, 8, 2, 4, 1, 16]]
    last_valid = 37
    q = query(1, 1, Hq, D) * (D ** -0.5)
    outs, rows = [], []
    for r, lv in enumerate(rows_levels):
        k, v = dense_inputs(100 + r, nb, P, D, outliers=4)
        lay, krec, vrec = build_row(torch.from_numpy(k), torch.from_numpy(v), lv, group)
        T = (nb - 1) * P + last_valid
        kk, vv = krec.view(-1, D)[:T], vrec.view(-1, D)[:T]
        qq = torch.from_numpy(q)[0, r * (Hq // Hkv):(r + 1) * (Hq // Hkv)]
        outs.append((torch.softmax(qq.double() @ kk.double().T, -1) @ vv.double()).float().numpy())
        rows.append(lay_np(lay))
    blob = {f"{key}_{r}": rows[r][key] for r in range(2) for key in rows[r]}
    np.savez_compressed(HERE / "gqa_d128.npz", P=P, D=D, group=group, Hq=Hq, Hkv=Hkv, nb=nb,
                        last_valid=last_valid, seeds=np.array([100, 101]), qseed=1,
                        out=np.concatenate(outs)[None], **blob)

    # ---- C. the other group sizes (Policy default 16, system_metrics 64)
    for group in (16, 64):
        P, D = 64, 128
        levels = [8, 1, 2, 16, 4]
        k, v = dense_inputs(200 + group, len(levels), P, D, outliers=4)
        lay, krec, vrec = build_row(torch.from_numpy(k), torch.from_numpy(v), levels, group)
        q = query(200 + group, 1, 1, D) * (D ** -0.5)
        refo = (torch.softmax(torch.from_numpy(q).view(1, D).double() @ krec.view(-1, D).double().T, -1)
                @ vrec.view(-1, D).double()).float()
        np.savez_compressed(HERE / f"group{group}_d128.npz", seed=200 + group, P=P, D=D, group=group,
                            out=refo.numpy()[None], **lay_np(lay))

    # ---- D. pack_bits / unpack_bits (geodesia_kv/packed.py:23-49)
    rng = np.random.default_rng(300)
    blob = {}
    for bits in (2, 4, 8):
        for n in (64, 63, 130):
            codes = rng.integers(0, 2 ** bits, size=n, dtype=np.uint8)
            pk = rpacked.pack_bits(torch.from_numpy(codes), bits)
            back = rpacked.unpack_bits(pk, bits, n)
            assert np.array_equal(back.numpy(), codes)
            blob[f"codes_{bits}_{n}"] = codes
            blob[f"packed_{bits}_{n}"] = pk.numpy()
    np.savez_compressed(HERE / "pack_bits.npz", **blob)

    # ---- E. quantize_codes on awkward blocks: constant groups, tiny and huge ranges, exact ties
    P, D, group = 64, 64, 32
    rng = np.random.default_rng(400)
    x = rng.standard_normal((4, P, D), dtype=np.float32)
    x[0, :32, :8] = 1.25                       # constant token groups (range clamps to 1e-8)
    x[0, 5, 32:] = -3.0                        # constant channel group
    x[1] *= 1e-6                               # steps near the bottom of fp16
    x[2] *= 3000.0                             # large values; fp16 rounding of lo visible
    x[3] = np.round(x[3] * 2) / 2              # many exact .5 quotients (half-to-even)
    blob = {"x": x}
    for bits in (2, 4, 8):
        for pc in (True, False):
            c, r, lo, st = quantize_codes(torch.from_numpy(x), bits, group, pc)
            tag = f"{bits}_{'k' if pc else 'v'}"
            blob[f"codes_{tag}"] = c.numpy()
            blob[f"rec_{tag}"] = r.numpy()
            blob[f"lo_{tag}"] = lo.view(torch.int16).numpy().view(np.uint16)
            blob[f"step_{tag}"] = st.view(torch.int16).numpy().view(np.uint16)
    np.savez_compressed(HERE / "quantize_edge.npz", P=P, D=D, group=group, **blob)

    # ---- F. allocator internals traced out of Policy.attend (geodesia_kv/policies.py:602-908)
    wanted = ("E", "ratio", "avail", "hot", "lvl_idx", "tgt_idx", "mass_cost", "target", "_lut")
    captured = {}

    def tracer(frame, event, arg):
        if frame.f_code is rpol.Policy.attend.__code__ and event == "call":
            def local(frame, event, arg):
                if event == "return":
                    for name in wanted:
                        if name in frame.f_locals:
                            val = frame.f_locals[name]
                            captured[name] = val.clone() if torch.is_tensor(val) else val
                return local
            return local
        return None

    blob, case = {}, 0
    for (P, D, group, nb0, steps, budget, seed) in [
            (64, 64, 32, 12, 3, 2.0, 500), (64, 64, 32, 12, 3, 3.0, 501), (64, 64, 16, 12, 3, 4.0, 502),
            (64, 64, 16, 12, 3, 5.0, 503), (64, 128, 32, 40, 4, 2.5, 504), (64, 128, 64, 40, 4, 0.75, 505),
            (64, 32, 16, 24, 2, 9.0, 506)]:
        pol = rpol.Policy(name="geodesia", budget_bits=budget, block=P, group=group, window=128,
                          sinks=4, mass_decay=0.0, validate=False)
        rng = np.random.default_rng(seed)
        kfull = rng.standard_normal(((nb0 + steps) * P, D), dtype=np.float32)
        vfull = rng.standard_normal(((nb0 + steps) * P, D), dtype=np.float32)
        for s in range(steps):
            nbs = nb0 + s
            T = nbs * P - (17 if s % 2 else 0)          # ragged tail on odd steps
            nbt = (T + P - 1) // P
            dist = (nbt - 1 - np.arange(nbt)).astype(np.float64)
            mass = (dist + 1.0) ** -1.2
            mass /= mass.sum()
            mass[0] += 0.1
            mass = mass.astype(np.float32)
            qv = rng.standard_normal((1, D), dtype=np.float32)
            st = pol.state.get((0, 0, 0))
            level_before = (st["level"].clone().numpy() if st is not None
                            else np.zeros(0, np.float32))
            captured.clear()
            sys.settrace(tracer)
            try:
                pol.attend(torch.from_numpy(qv), torch.from_numpy(kfull[:T]), torch.from_numpy(vfull[:T]),
                           D ** -0.5, q_offset=T - 1, hid=(0, 0, 0),
                           observed_mass=torch.from_numpy(mass))
            finally:
                sys.settrace(None)
            st = pol.state[(0, 0, 0)]
            tag = f"c{case}"
            blob[f"{tag}_meta"] = np.array([P, D, group, nbt, T], np.int64)
            blob[f"{tag}_budget"] = np.float64(budget)
            blob[f"{tag}_mass"] = st["mass"].numpy().copy()
            blob[f"{tag}_level_before"] = np.concatenate(
                [level_before, np.full(nbt - level_before.size, 16.0, np.float32)])
            blob[f"{tag}_level_after"] = st["level"].numpy().copy()
            blob[f"{tag}_E"] = captured["E"].numpy()
            blob[f"{tag}_ratio"] = captured["ratio"].numpy()
            blob[f"{tag}_hot"] = captured["hot"].numpy().astype(np.uint8)
            blob[f"{tag}_lvl_idx"] = captured["lvl_idx"].numpy().astype(np.int32)
            blob[f"{tag}_tgt_idx"] = captured["tgt_idx"].numpy().astype(np.int32)
            blob[f"{tag}_bits"] = captured["_lut"].numpy().astype(np.float32)
            blob[f"{tag}_target"] = np.float64(captured["target"])
            if case in (0, 4):                          # reconstructions, to pin the distortion table
                blob[f"{tag}_seed"] = np.int64(seed)
            case += 1
    blob["ncases"] = np.int64(case)
    np.savez_compressed(HERE / "allocator.npz", **blob)

    # ---- G. distortion table on fresh (all rung-16) blocks: E depends on K, V only
    P, D, group = 64, 64, 32
    k, v = dense_inputs(600, 6, P, D, outliers=2)
    pol = rpol.Policy(name="geodesia", budget_bits=3.0, block=P, group=group, window=64, sinks=4,
                      mass_decay=0.0, validate=False, alloc_value_weight=0.5)
    captured.clear()
    sys.settrace(tracer)
    try:
        pol.attend(torch.from_numpy(query(600, 1, D)), torch.from_numpy(k.reshape(-1, D)),
                   torch.from_numpy(v.reshape(-1, D)), D ** -0.5, q_offset=6 * P - 1, hid=(0, 0, 0),
                   observed_mass=torch.full((6,), 1.0 / 6))
    finally:
        sys.settrace(None)
    np.savez_compressed(HERE / "distortion.npz", seed=600, P=P, D=D, group=group, nb=6, outliers=2,
                        value_weight=0.5, E=captured["E"].numpy())

    # ---- H. format A (geodesia_kv/packed.py:52-157): quantize_packed / build_packed
    P, D, group = 64, 64, 32
    k, v = dense_inputs(700, 6, P, D)
    bits = torch.tensor([16.0, 8.0, 4.0, 2.0, 3.0, 4.0])
    cent = torch.tensor([False, False, False, False, False, True])
    pk = rpacked.build_packed(torch.from_numpy(k.reshape(-1, D)), torch.from_numpy(v.reshape(-1, D)),
                              bits, cent, P, group)
    blob = {"nbytes": np.int64(pk.nbytes()), "exact_idx": pk.exact_idx.numpy(),
            "cent_idx": pk.cent_idx.numpy(),
            "cent_k": pk.cent_k.view(torch.int16).numpy().view(np.uint16),
            "exact_k": pk.exact_k.view(torch.int16).numpy().view(np.uint16)}
    for i, (idx, pkk, pvv) in enumerate(pk.quant):
        blob[f"q{i}_idx"] = idx.numpy()
        blob[f"q{i}_bits"] = np.int64(pkk.bits)
        blob[f"q{i}_kdata"] = pkk.data.numpy()
        blob[f"q{i}_vdata"] = pvv.data.numpy()
        blob[f"q{i}_klo"] = pkk.lo.view(torch.int16).numpy().view(np.uint16)
        blob[f"q{i}_kstep"] = pkk.step.view(torch.int16).numpy().view(np.uint16)
        blob[f"q{i}_vlo"] = pvv.lo.view(torch.int16).numpy().view(np.uint16)
        blob[f"q{i}_vstep"] = pvv.step.view(torch.int16).numpy().view(np.uint16)
        blob[f"q{i}_kdeq"] = pkk.dequantize().numpy()
        blob[f"q{i}_vdeq"] = pvv.dequantize().numpy()
    blob["nquant"] = np.int64(len(pk.quant))
    np.savez_compressed(HERE / "format_a.npz", seed=700, P=P, D=D, group=group, **blob)

    # ---- I. a decode trajectory through Policy.attend (policies.py:602-908): rungs per step and outputs
    P, D, group = 64, 64, 32
    T0, steps, stride = 592, 32, 16      # T reaches every multiple of 64: the reference only refreshes the block being written
    rng = np.random.default_rng(800)
    bf = lambda a: torch.from_numpy(a).to(torch.bfloat16).float()           # bf16-representable inputs
    kfull = bf(rng.standard_normal((T0 + steps * stride, D), dtype=np.float32))
    vfull = bf(rng.standard_normal((T0 + steps * stride, D), dtype=np.float32))
    kfull[:, rng.permutation(D)[:2]] *= 8.0
    qall = bf(rng.standard_normal((steps, D), dtype=np.float32))
    pol = rpol.Policy(name="geodesia", budget_bits=3.0, block=P, group=group, window=128, sinks=4, validate=False)
    blob = {"meta": np.array([P, D, group, T0, steps, stride], np.int64), "budget": np.float64(3.0)}
    for s in range(steps):
        T = T0 + s * stride
        out = pol.attend(qall[s:s + 1], kfull[:T], vfull[:T], D ** -0.5, q_offset=T - 1, hid=(0, 0, 0))
        blob[f"level_{s}"] = pol.state[(0, 0, 0)]["level"].numpy().astype(np.int32)
        blob[f"out_{s}"] = out.numpy()
    blob["bits_per_value"] = np.float64(pol.report.bits_per_value)
    np.savez_compressed(HERE / "policy_decode.npz", seed=800, **blob)

    # ---- J. quant_grouped (geodesia_kv/policies.py:82-112)
    write_quant_grouped()

    for f in sorted(HERE.glob("*.npz")):
        print(f"{f.name:28s} {f.stat().st_size / 1024:8.1f} KiB")


if __name__ == "__main__":
    main()
