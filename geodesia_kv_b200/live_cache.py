"""A transformers ``Cache`` that owns the packed pool, and the attention function that reads it.

The reference's resident-memory cache (``geodesia_kv/live_cache.py:52-162``) closes chunks of a dense
tail into uniformly quantised ``PackedBlocks`` and, at every layer of every step, de-quantises the whole
layer back to dense K/V for SDPA (``_materialize``, :113-142); its bit-ladder policy
(``policies.py:1459-1519``) keeps the dense K/V in the HF cache and simulates the compression.  Here the
packed pool IS the cache:

* prefill: the prompt's K/V of a layer are packed into rung-16 slots of a :class:`PagedPool` as they
  arrive, attended exactly by SDPA (they are in hand anyway), the block masses of the last ``obs``
  queries seed the allocator (``policies.py:1393-1456``), and the layer is demoted to its budget before
  the next layer runs — after prefill no dense K/V remains anywhere;
* decode: the step's single K/V row per sequence is appended to the row's open block on the device,
  ONE kernel call attends over all (sequence, KV head) rows of the layer and hands back the per-block
  softmax mass as a by-product, which is folded into the running mass; every ``maintain_every``
  tokens the distortion, allocator and demotion kernels run for all layers with one read-back.

Unlike the reference's simulation, a demotion decided from the masses of step t takes effect for step
t+1 (the masses come out of the attention call itself), and the masses are those of the packed keys.
"""
from __future__ import annotations

import numpy as np
import torch
from transformers.cache_utils import Cache, CacheLayerMixin

from .paged import BLOCK, PagedLayerCache, PagedPool

ACTIVE_CACHE: "PagedKVCache | None" = None      # the cache whose layer was updated last (set by update())
ATTENTION_NAME = "geodesia_paged"


class PagedCacheLayer(CacheLayerMixin):
    """One layer of a :class:`PagedKVCache`: a block table over the shared pool."""

    is_sliding = False
    is_compileable = False

    def __init__(self, owner: "PagedKVCache", idx: int):
        super().__init__()
        self.owner, self.idx = owner, idx
        self.paged: PagedLayerCache | None = None
        self.seen = 0

    def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        B, Hkv, T, D = key_states.shape
        self.dtype, self.device = key_states.dtype, key_states.device
        pool = self.owner.pool_for(B, Hkv, D, key_states.device, T)
        self.paged = PagedLayerCache(pool, B, Hkv, cap_blocks=(T + BLOCK - 1) // BLOCK + 64)
        self.is_initialized = True

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, *args, **kwargs):
        """Take the step's K/V rows into the pool and hand the SAME rows back: the prompt at prefill (the
        attention function attends it exactly, nothing keeps it), one row per sequence afterwards (the
        attention function ignores it and reads the pool)."""
        global ACTIVE_CACHE
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        T = key_states.shape[-2]
        if self.seen == 0:
            self.paged.prefill(key_states, value_states)
        elif T == 1:
            self.paged.append(key_states, value_states)
        else:
            raise NotImplementedError("the packed cache takes a prompt once and then one token per step")
        self.seen += T
        ACTIVE_CACHE = self.owner
        return key_states, value_states

    def get_seq_length(self) -> int:
        return self.seen

    def get_mask_sizes(self, query_length: int) -> tuple[int, int]:
        return self.seen + query_length, 0

    def get_max_cache_shape(self) -> int:
        return -1

    def reset(self) -> None:
        if self.paged is not None:
            self.paged.release()
        self.seen = 0

    def offload(self):
        raise NotImplementedError("the packed pool stays on its GPU")

    prefetch = offload

    def reorder_cache(self, beam_idx):
        raise NotImplementedError("beam search is not supported on the packed cache")


class PagedKVCache(Cache):
    """HF cache whose storage is the packed pool (no dense K/V after prefill).

    ``budget_bits`` is the resident budget in bits per cached value (0 keeps every block exact);
    ``layer_budget_bits`` overrides it per layer.  ``pool`` shares one pool between caches;
    otherwise ``pool_bytes`` (or a size derived from the first prompt and ``max_new_tokens``) is
    allocated on first use.  A batch is B sequences of the SAME prompt length (no padding tokens:
    ragged batches go through :class:`PagedLayerCache` directly, which takes per-sequence lengths);
    the prompt arrives in one forward pass, then one token per step.  Everything runs on the
    current stream.  The remaining fields are the reference policy's
    (``policies.py:227-272``): sinks, window, obs, mass_decay, alloc_mass_power, alloc_value_weight.
    """

    def __init__(self, num_layers: int, budget_bits: float = 4.0, group: int = 32, pool: PagedPool | None = None,
                 pool_bytes: int | None = None, max_new_tokens: int = 4096, sinks: int = 4, window: int = 128, obs: int = 32,
                 mass_decay: float = 0.9, alloc_mass_power: float = 1.0, alloc_value_weight: float = 0.0,
                 maintain_every: int = BLOCK, layer_budget_bits: tuple = ()):
        super().__init__(layers=[PagedCacheLayer(self, i) for i in range(num_layers)])
        self.budget_bits, self.layer_budget_bits, self.group = budget_bits, tuple(layer_budget_bits), group
        self.pool, self.pool_bytes, self.max_new_tokens = pool, pool_bytes, max_new_tokens
        self.sinks, self.window, self.obs = sinks, window, obs
        self.mass_decay, self.alloc_mass_power, self.alloc_value_weight = mass_decay, alloc_mass_power, alloc_value_weight
        self.maintain_every = maintain_every
        self.steps = 0
        self.blocks_demoted = 0

    # -- storage ----------------------------------------------------------------------------------
    def pool_for(self, B: int, Hkv: int, D: int, device, prompt_tokens: int) -> PagedPool:
        if self.pool is None:
            if self.pool_bytes is None:
                # every layer's final share plus one layer exact (the one being prefilled), with slack
                L = len(self.layers)
                dense_layer = B * Hkv * (prompt_tokens + self.max_new_tokens + BLOCK) * D * 4
                share = min(1.0, (self.budget_bits if self.budget_bits > 0 else 16.0) / 16.0 * 1.3 + 0.05)
                self.pool_bytes = int(L * dense_layer * share + 2 * dense_layer) + (64 << 20)
            self.pool = PagedPool(self.pool_bytes, D, self.group, device)
        return self.pool

    def budget_for(self, idx: int) -> float:
        return float(self.layer_budget_bits[idx]) if self.layer_budget_bits else float(self.budget_bits)

    # -- maintenance ------------------------------------------------------------------------------
    def _plan(self, layer: PagedCacheLayer):
        return layer.paged.plan_demotion(self.budget_for(layer.idx), sinks=self.sinks, window=self.window,
                                         mass_power=self.alloc_mass_power, value_weight=self.alloc_value_weight)

    def maintain(self, layers=None) -> int:
        """Distortion + allocator kernels for the given layers (default: all), ONE read-back, then the
        demotion kernels.  Returns the number of blocks demoted."""
        todo = [l for l in (self.layers if layers is None else layers)
                if l.paged is not None and l.seen and self.budget_for(l.idx) > 0]
        if not todo:
            return 0
        plans = [self._plan(l) for l in todo]
        width = max(p.shape[1] for p in plans)
        if any(p.shape[1] != width for p in plans):
            plans = [torch.nn.functional.pad(p, (0, width - p.shape[1])) for p in plans]
        host = torch.stack(plans).cpu().numpy()                  # the one synchronisation
        n = 0
        for l, tgt in zip(todo, host):
            n += l.paged.apply_demotion(tgt[:, :l.paged.nb])
        self.blocks_demoted += n
        return n

    def after_layer(self, layer: PagedCacheLayer, prefill: bool) -> None:
        if prefill:
            self.maintain([layer])                              # the prompt of this layer shrinks before the next one is packed
        elif layer.idx == len(self.layers) - 1:
            self.steps += 1
            if self.maintain_every and self.steps % self.maintain_every == 0:
                self.maintain()

    # -- accounting -------------------------------------------------------------------------------
    def bits_per_value(self) -> float:
        vals = [l.paged.bits_per_value() for l in self.layers if l.paged is not None]
        return float(np.mean(vals)) if vals else 0.0

    def bytes_in_use(self) -> int:
        return sum(l.paged.bytes_in_pool() for l in self.layers if l.paged is not None)

    def dense_bytes(self) -> int:
        return sum(int(l.paged.blocks_per_seq().sum()) * l.paged.Hkv * 4 * BLOCK * l.paged.D for l in self.layers if l.paged is not None)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self.layers[layer_idx].get_seq_length() if layer_idx < len(self.layers) else 0


def _prompt_block_mass(query, key, scaling, obs: int):
    """Mass per block of the last ``obs`` prompt queries, averaged over them and over the query heads of
    each KV head (policies.py:1421-1451): (B*Hkv, nb)."""
    B, H, Q, D = query.shape
    Hkv, T = key.shape[1], key.shape[-2]
    reps = H // Hkv
    n_obs = min(obs, Q)
    q_start = T - n_obs
    causal = torch.arange(T, device=key.device)[None, :] <= (q_start + torch.arange(n_obs, device=key.device))[:, None]
    nb = (T + BLOCK - 1) // BLOCK
    qo = query[:, :, -n_obs:].float().reshape(B, Hkv, reps * n_obs, D)
    sc = (qo @ key.float().transpose(-1, -2)) * scaling
    cmask = causal[None].expand(reps, -1, -1).reshape(reps * n_obs, T)
    w = torch.softmax(sc.masked_fill(~cmask, float("-inf")), -1)
    if nb * BLOCK != T:
        w = torch.nn.functional.pad(w, (0, nb * BLOCK - T))
    return w.view(B, Hkv, reps * n_obs, nb, BLOCK).sum(-1).mean(2).reshape(B * Hkv, nb)


def paged_attention(module, query, key, value, attention_mask, scaling=None, dropout=0.0, **kwargs):
    """Attention function for ``ALL_ATTENTION_FUNCTIONS`` over a :class:`PagedKVCache`
    (replaces ``policy_attention``, policies.py:1459-1519, and ``live_cache._materialize`` + SDPA)."""
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    cache = ACTIVE_CACHE
    idx = getattr(module, "layer_idx", 0)
    layer = cache.layers[idx] if cache is not None and idx < len(cache.layers) else None
    B, H, Q, D = query.shape
    if scaling is None:
        scaling = D ** -0.5
    if layer is None or layer.paged is None or key.shape[-2] == layer.seen or Q > 1:
        out = ALL_ATTENTION_FUNCTIONS["sdpa"](module, query, key, value, attention_mask, dropout=dropout, scaling=scaling, **kwargs)
        if layer is not None and layer.paged is not None:
            with torch.no_grad():
                nb = layer.paged.nb
                layer.paged.mass[:, :nb] = _prompt_block_mass(query, key, scaling, cache.obs)
            cache.after_layer(layer, prefill=True)
        return out
    q = (query[:, :, 0].float() * scaling).contiguous()
    out, mass = layer.paged.attend(q, want_mass=True)
    layer.paged.observe(mass, cache.mass_decay)
    cache.after_layer(layer, prefill=False)
    return out.to(query.dtype)[:, None], None


def register() -> str:
    """Make ``attn_implementation="geodesia_paged"`` available to transformers models."""
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS
    ALL_ATTENTION_FUNCTIONS.register(ATTENTION_NAME, paged_attention)
    try:        # masks as SDPA builds them (only the prefill uses one)
        ALL_MASK_ATTENTION_FUNCTIONS.register(ATTENTION_NAME, ALL_MASK_ATTENTION_FUNCTIONS["sdpa"])
    except Exception:
        pass
    return ATTENTION_NAME
