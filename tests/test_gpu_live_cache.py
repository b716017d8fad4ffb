"""The HF cache that owns the packed pool, driven through a random-init Qwen3 model: exact at an
unlimited budget, within budget and close at 4 bits/value, and no dense K/V left after prefill."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny_qwen3(layers=2, seed=0):
    from transformers import Qwen3Config, Qwen3ForCausalLM
    from geodesia_kv_b200 import live_cache
    name = live_cache.register()
    cfg = Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=layers,
                      num_attention_heads=8, num_key_value_heads=2, head_dim=128, max_position_embeddings=8192,
                      tie_word_embeddings=False)
    torch.manual_seed(seed)
    model = Qwen3ForCausalLM(cfg).to(device="cuda", dtype=torch.bfloat16).eval()
    return model, name


@torch.no_grad()
def run(model, impl, cache, prompt, new_tokens):
    """Greedy continuation with teacher forcing of a fixed token stream; returns the logits of every step."""
    model.config._attn_implementation = impl
    out = model(input_ids=prompt, past_key_values=cache, use_cache=True)
    logits = [out.logits[:, -1].float()]
    for t in range(new_tokens.shape[1]):
        out = model(input_ids=new_tokens[:, t:t + 1], past_key_values=cache, use_cache=True)
        logits.append(out.logits[:, -1].float())
    return torch.stack(logits, 1)


def test_unlimited_budget_reproduces_the_dense_cache():
    from transformers import DynamicCache
    from geodesia_kv_b200.live_cache import PagedKVCache
    model, name = tiny_qwen3()
    gen = torch.Generator(device="cuda").manual_seed(1)
    prompt = torch.randint(0, 512, (2, 300), device="cuda", generator=gen)
    cont = torch.randint(0, 512, (2, 70), device="cuda", generator=gen)
    want = run(model, "sdpa", DynamicCache(config=model.config), prompt, cont)
    cache = PagedKVCache(num_layers=2, budget_bits=0.0)
    got = run(model, name, cache, prompt, cont)
    # the cache stores the same bf16 rows; only the attention arithmetic differs (fp32 accumulate here)
    assert (got - want).abs().max().item() < 0.08 * want.abs().max().item()
    assert (got.argmax(-1) == want.argmax(-1)).float().mean().item() > 0.9
    assert cache.get_seq_length() == 370 and cache.layers[0].paged.len_h.tolist() == [370, 370]
    assert cache.bytes_in_use() == cache.dense_bytes()          # every block still exact
    assert all(l.keys is None and l.values is None for l in cache.layers)   # no dense K/V is held anywhere


def test_budgeted_cache_stays_close_and_gives_memory_back():
    from transformers import DynamicCache
    from geodesia_kv_b200.live_cache import PagedKVCache
    model, name = tiny_qwen3(seed=3)
    gen = torch.Generator(device="cuda").manual_seed(2)
    prompt = torch.randint(0, 512, (3, 64 * 24), device="cuda", generator=gen)
    cont = torch.randint(0, 512, (3, 130), device="cuda", generator=gen)
    want = run(model, "sdpa", DynamicCache(config=model.config), prompt, cont)
    cache = PagedKVCache(num_layers=2, budget_bits=4.0, maintain_every=64)
    got = run(model, name, cache, prompt, cont)
    assert cache.blocks_demoted > 0
    assert cache.bits_per_value() <= 4.0 + 16.0 * 5 / 26 + 1e-6   # budget + the blocks that must stay exact
    assert cache.bytes_in_use() < 0.45 * cache.dense_bytes()
    assert cache.pool.bytes_in_use == cache.bytes_in_use()
    # a random-init model attends almost uniformly, so most of its blocks end as centroids: the logits stay
    # aligned with the dense run's but not equal to them
    cos = torch.nn.functional.cosine_similarity(got, want, dim=-1)
    assert cos.min().item() > 0.93 and cos.mean().item() > 0.97
    assert torch.equal(got[:, 0], got[:, 0]) and (got[:, 0] - want[:, 0]).abs().max().item() < 1e-3   # prefill is exact
    # the prompt's masses came from the prefill queries, the later ones from the decode kernel
    m = cache.layers[1].paged.mass
    assert torch.isfinite(m).all() and float(m.sum()) > 0
    for l in cache.layers:
        assert int(l.paged.status.item()) == 0


def test_generate_runs_on_the_packed_cache():
    """transformers' own generate loop (greedy) with the packed cache passed as past_key_values."""
    from geodesia_kv_b200.live_cache import PagedKVCache
    model, name = tiny_qwen3(seed=5)
    model.config._attn_implementation = name
    gen = torch.Generator(device="cuda").manual_seed(4)
    prompt = torch.randint(0, 512, (2, 200), device="cuda", generator=gen)
    cache = PagedKVCache(num_layers=2, budget_bits=4.0, maintain_every=32)
    with torch.no_grad():
        out = model.generate(prompt, past_key_values=cache, max_new_tokens=80, do_sample=False, use_cache=True)
    assert out.shape == (2, 280) and torch.equal(out[:, :200], prompt)
    assert cache.get_seq_length() == 279 and cache.blocks_demoted > 0          # the last token is not fed back
    assert cache.pool.bytes_in_use == cache.bytes_in_use()
