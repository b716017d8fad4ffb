"""The geodesia policy on the packed cache: rung trajectory against the reference's Policy.attend,
the HF attention-interface functions, the vLLM manager, and the reference's own CUDA kernel as a
second oracle when its build is present."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from helpers import kernel_args, oracle_cache, to_torch

pytestmark = pytest.mark.gpu


def bf16r(a):
    return torch.from_numpy(a).to(torch.bfloat16).float()


def test_decode_trajectory_matches_the_reference_policy(golden):
    """24 decode steps of policies.py:602-908 (run on CPU by the reference's code): the rung of
    every block after every step must be identical; outputs agree up to the scale precision of
    demoted blocks (the reference's simulation keeps fp32 scales, a packed cache stores fp16)."""
    from geodesia_kv_b200.policies import Policy
    g = golden("policy_decode")
    P, D, group, T0, steps, stride = (int(x) for x in g["meta"])
    rng = np.random.default_rng(int(g["seed"]))
    kfull = bf16r(rng.standard_normal((T0 + steps * stride, D), dtype=np.float32))
    vfull = bf16r(rng.standard_normal((T0 + steps * stride, D), dtype=np.float32))
    kfull[:, rng.permutation(D)[:2]] *= 8.0
    qall = bf16r(rng.standard_normal((steps, D), dtype=np.float32))
    kfull, vfull, qall = kfull.cuda(), vfull.cuda(), qall.cuda()
    pol = Policy(name="geodesia", budget_bits=float(g["budget"]), block=P, group=group, window=128, sinks=4,
                 validate=False)
    demoted = 0
    for s in range(steps):
        T = T0 + s * stride
        out = pol.attend(qall[s:s + 1], kfull[:T], vfull[:T], D ** -0.5, q_offset=T - 1, hid=(0, 0, 0))
        level = pol.state[(0, 0, 0)].view((T + P - 1) // P).level[0, 0].cpu().numpy()
        assert np.array_equal(level, g[f"level_{s}"]), f"step {s}"
        demoted = int((level < 16).sum())
        want = g[f"out_{s}"]
        assert np.abs(out.cpu().numpy() - want).max() < 5e-3, f"step {s}"
    assert demoted >= 5
    assert abs(pol.report.bits_per_value - float(g["bits_per_value"])) < 1e-6


def test_policy_attention_hook_gqa_decode():
    """policy_attention on a random GQA decode step: one packed cache per KV head, outputs within
    the budgeted error of exact attention, state keyed (layer, batch, kv head)."""
    from types import SimpleNamespace
    from geodesia_kv_b200 import policies as P
    gen = torch.Generator(device="cuda").manual_seed(0)
    B, H, Hkv, T, D = 2, 8, 2, 1500, 128
    key = torch.randn(B, Hkv, T, D, device="cuda", dtype=torch.bfloat16, generator=gen)
    val = torch.randn(B, Hkv, T, D, device="cuda", dtype=torch.bfloat16, generator=gen)
    qry = torch.randn(B, H, 1, D, device="cuda", dtype=torch.bfloat16, generator=gen)
    module = SimpleNamespace(layer_idx=3)
    P.ACTIVE = P.Policy(name="geodesia", budget_bits=16.0, group=32)          # budget 16: nothing is demoted
    try:
        out, _ = P.policy_attention(module, qry, key, val, None, D ** -0.5)
        assert out.shape == (B, 1, H, D) and out.dtype == qry.dtype
        exact = torch.nn.functional.scaled_dot_product_attention(
            qry.float(), key.float().repeat_interleave(H // Hkv, 1), val.float().repeat_interleave(H // Hkv, 1))
        assert (out.float().transpose(1, 2) - exact).abs().max().item() < 2e-2      # bf16 output rounding
        assert set(P.ACTIVE.state) == {(3, b, hk) for b in range(B) for hk in range(Hkv)}
        # a tight budget demotes cold blocks and the result stays close
        P.ACTIVE = P.Policy(name="geodesia", budget_bits=4.0, group=32, mass_decay=0.0)
        out2, _ = P.policy_attention(module, qry, key, val, None, D ** -0.5)
        lv = P.ACTIVE.state[(3, 0, 0)].view((T + 63) // 64).level
        assert int((lv < 16).sum()) > 0 and int(lv[0, 0, 0]) == 16 and int(lv[0, 0, -1]) == 16
        assert (out2.float().transpose(1, 2) - exact).abs().max().item() < 0.15
        assert P.ACTIVE.report.bits_per_value < 8.0
    finally:
        P.ACTIVE = None


def test_vllm_manager_packs_for_the_kernel():
    """tests/test_vllm_geodesia_plugin.py:26-58 of the reference, plus attending over the result."""
    from geodesia_kv.vllm_plugin import GeodesiaKVCacheManager, register_geodesia_kv_plugin
    from geodesia_kv_b200.cuda_ext import get_ext

    class Dummy:
        pass

    llm = Dummy()
    mgr = register_geodesia_kv_plugin(llm, target_bpv=4.0, block_size=64)
    assert isinstance(mgr, GeodesiaKVCacheManager) and llm.geodesia_manager is mgr
    cache = mgr.create_sequence_cache(7)
    gen = torch.Generator(device="cuda").manual_seed(1)
    kc = torch.randn(3, 1024, 4, 64, device="cuda", dtype=torch.bfloat16, generator=gen)
    vc = torch.randn(3, 1024, 4, 64, device="cuda", dtype=torch.bfloat16, generator=gen)
    bpv = cache.compress_sequence_kv(kc, vc)
    assert bpv <= 5.5 and 1.0 - bpv / 16.0 > 0.6
    assert len(cache.layers) == 3 and len(cache.kernel_layers) == 3
    lay = cache.kernel_layers[1]
    q = torch.randn(1, 8, 64, device="cuda", generator=gen) * 64 ** -0.5
    out = get_ext().mixed_attn_decode(q, *lay.kernel_args())
    kk = kc[1].permute(1, 0, 2).float().repeat_interleave(2, 0)
    vv = vc[1].permute(1, 0, 2).float().repeat_interleave(2, 0)
    exact = torch.softmax(torch.einsum("hd,htd->ht", q[0], kk), -1)
    exact = torch.einsum("ht,htd->hd", exact, vv)
    assert (out[0] - exact).abs().max().item() < 0.1            # 4-bit cache vs exact
    mgr.free_sequence_cache(7)
    assert mgr.get_cache(7) is None


def test_against_the_reference_cuda_kernel(oracle):
    """The reference's own mixed_attn.cu, compiled unmodified for sm_100a, on the same tensors
    (bytes replicated per query head, as it requires)."""
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "oracle"))
    import build_ref
    ref = build_ref.load()
    if ref is None:
        pytest.skip("oracle/_ref has not been built (needs a checkout of the reference)")
    from geodesia_kv_b200.cuda_ext import get_ext
    for D, group, nb in ((128, 32, 40), (64, 32, 9), (128, 64, 12)):
        c = oracle_cache(oracle, 77 + D + group, 1, 4, nb, D, group, shared_meta=True)
        t = to_torch(c, "cuda")
        q = torch.randn(1, 4, D, device="cuda") * D ** -0.5
        ours = get_ext().mixed_attn_decode(q, *kernel_args(t, c))
        theirs = ref.mixed_attn_decode(q, *kernel_args(t, c))
        assert (ours - theirs).abs().max().item() < 2e-3
        assert (ours - theirs).abs().max().item() < 5e-5
