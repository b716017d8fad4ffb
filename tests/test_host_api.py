"""CPU tests of the reference-facing Python surface: alias package, Policy bookkeeping, plugin."""
from __future__ import annotations

import pytest
import torch


def test_alias_package_exposes_the_reference_names():
    import geodesia_kv
    import geodesia_kv.cuda_ext as ce
    import geodesia_kv.pack_layout as pl
    import geodesia_kv.packed as pk
    import geodesia_kv.policies as po
    from geodesia_kv.vllm_plugin import GeodesiaBlockCache, GeodesiaKVCacheManager, register_geodesia_kv_plugin
    assert geodesia_kv.__all__ == ["policies", "packed", "pack_layout", "cuda_ext"]
    for mod, names in ((ce, ["get_ext", "mixed_attn_decode"]), (pl, ["build_layout"]),
                       (pk, ["pack_bits", "unpack_bits", "quantize_packed", "PackedBlocks", "PackedKV", "build_packed"]),
                       (po, ["Policy", "Report", "policy_attention", "observation_attention", "ACTIVE", "OBSERVER",
                             "LEVELS", "_level_bits", "blockify", "quant_grouped"])):
        for n in names:
            assert hasattr(mod, n), (mod.__name__, n)
    assert GeodesiaBlockCache and GeodesiaKVCacheManager and register_geodesia_kv_plugin


def test_full_policy_is_exact_and_causal():
    from geodesia_kv.policies import Policy
    torch.manual_seed(0)
    q, k, v = torch.randn(3, 16), torch.randn(40, 16), torch.randn(40, 16)
    pol = Policy(name="full")
    out = pol.attend(q, k, v, 0.25, q_offset=37)
    for i in range(3):
        w = torch.softmax((q[i] @ k[:38 + i].T) * 0.25, -1)
        assert torch.allclose(out[i], w @ v[:38 + i], atol=1e-6)
    assert pol.report.bits_per_value == 16.0
    pol.reset_state()
    assert not pol.state and not pol.observations


def test_policy_rejects_what_it_does_not_implement():
    from geodesia_kv.policies import Policy
    with pytest.raises(ValueError):
        Policy(name="snapkv")
    with pytest.raises(ValueError):
        Policy(name="geodesia", block=32)
    with pytest.raises(ValueError):
        Policy(name="geodesia", spectral_rank=2)
    pol = Policy(name="geodesia", budget_bits=2.0, layer_budget_bits=(2.0, 3.0))
    assert pol._budget_for((1, 0, 0)) == 3.0
    with pytest.raises(ValueError):
        pol._budget_for((5, 0, 0))
    with pytest.raises(RuntimeError, match="no CPU path"):
        pol.attend(torch.randn(1, 64), torch.randn(128, 64), torch.randn(128, 64), 0.125, q_offset=127, hid=(0, 0, 0))


def test_vllm_manager_on_cpu_like_the_reference_test():
    """tests/test_vllm_geodesia_plugin.py:26-58: synthetic (24, 1024, 14, 64) bf16 cache."""
    from geodesia_kv.vllm_plugin import GeodesiaKVCacheManager
    mgr = GeodesiaKVCacheManager(block_size=64, target_bpv=4.0, num_layers=24)
    cache = mgr.create_sequence_cache(0)
    torch.manual_seed(0)
    kc = torch.randn(4, 1024, 14, 64, dtype=torch.bfloat16)
    vc = torch.randn(4, 1024, 14, 64, dtype=torch.bfloat16)
    bpv = cache.compress_sequence_kv(kc, vc)
    assert bpv <= 5.5
    assert 1.0 - bpv / 16.0 > 0.60
    bits, cent = cache.allocate_bits_for_blocks(5, "cpu")
    assert bits.tolist() == [4.0, 4.0, 4.0, 4.0, 16.0] and not cent.any()
    assert mgr.get_cache(0) is cache


def test_observation_attention_records_block_mass():
    from types import SimpleNamespace
    import geodesia_kv.policies as P
    torch.manual_seed(0)
    B, H, Hkv, T, D = 1, 4, 2, 200, 16
    q, k, v = torch.randn(B, H, T, D), torch.randn(B, Hkv, T, D), torch.randn(B, Hkv, T, D)
    P.OBSERVER = P.Policy(name="geodesia", budget_bits=3.0, group=16)
    try:
        out, _ = P.observation_attention(SimpleNamespace(layer_idx=1, training=False, is_causal=True, num_key_value_groups=H // Hkv), q, k, v, None, D ** -0.5,
                                         is_causal=True)
        assert out.shape[0] == B
        m = P.OBSERVER.observations[(1, 0, 1)]["block_mass"]
        assert m.shape == (4,) and abs(float(m.sum()) - 1.0) < 1e-5
    finally:
        P.OBSERVER = None
