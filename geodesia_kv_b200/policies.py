"""Rung allocation and the attention hooks, with the reference's names.

Mirrors the part of ``geodesia_kv/policies.py`` that lies on the packed decode
path: the ladder constants and ``_level_bits`` (:1576-1596), ``blockify``
(:126-133), ``quant_grouped`` (:82-112), the Lagrangian allocator of
``Policy.attend`` (:810-868) and its hot mask (:677-681).  The allocator and the
distortion table run as CUDA kernels over whole batches of cache rows.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

SPECTRAL_LEVEL = 1.5
LEVELS = [16, 8, 4, 2, SPECTRAL_LEVEL, 1]
LADDER = (16, 8, 4, 2, 1)            # the rungs the packed format stores


def _level_bits(level, block: int, D: int, group: int, spectral_rank: int = 0) -> float:
    """Resident bits of one block at a rung, scales included."""
    if level >= 16:
        return 2.0 * block * D * 16.0
    if level == 1:
        return 2.0 * D * 16.0
    if level == SPECTRAL_LEVEL:
        rank = max(0, min(int(spectral_rank), block, D))
        return 2.0 * D * 16.0 * (1 + rank) + rank * 16.0
    token_groups = max(1, block // group)
    channel_groups = max(1, D // group)
    return 2.0 * level * block * D + token_groups * D * 32.0 + block * channel_groups * 32.0


def blockify(x: torch.Tensor, block: int):
    """(T, D) -> (nb, block, D), the tail padded by repeating the last row; returns (blocks, pad)."""
    t, d = x.shape
    nb = (t + block - 1) // block
    pad = nb * block - t
    if pad:
        x = torch.cat([x, x[-1:].expand(pad, -1)], 0)
    return x.view(nb, block, d), pad


def quant_grouped(x: torch.Tensor, bits: int, group: int, per_channel: bool):
    """Grouped min-max quantise -> dequantise of (nb, P, D) with fp32 scales; returns
    (reconstruction, largest step per block)."""
    nb, pp, d = x.shape
    if per_channel:
        g = min(group, pp)
        xs, axis = x.view(nb, pp // g, g, d), 2
    else:
        g = min(group, d)
        xs, axis = x.view(nb, pp, d // g, g), 3
    if bits >= 16:
        shape = (nb, d) if per_channel else (nb,)
        return x, torch.zeros(shape, device=x.device, dtype=x.dtype)
    lo = xs.amin(axis, keepdim=True)
    step = (xs.amax(axis, keepdim=True) - lo).clamp_min(1e-8) / (2 ** bits - 1)
    rec = (((xs - lo) / step).round().clamp_(0, 2 ** bits - 1) * step + lo).view(nb, pp, d)
    return rec, step.amax(dim=(1, 2) if per_channel else (1, 2, 3))


def hot_mask(nb: int, q_offset: int, block: int = 64, sinks: int = 4, window: int = 128,
             device=None) -> torch.Tensor:
    """Blocks that may never be demoted: sinks, the block being written and its
    predecessor, and the recent window (policies.py:677-681)."""
    hot = torch.zeros(nb, dtype=torch.bool, device=device)
    hot[: max(1, (sinks + block - 1) // block)] = True
    hot[max(0, q_offset // block - 1):] = True
    hot[-max(1, (window + block - 1) // block):] = True
    return hot


def ladder_bits(block: int, D: int, group: int) -> list[float]:
    return [_level_bits(L, block, D, group) for L in LADDER]


def allocate_rungs(mass: torch.Tensor, E: torch.Tensor, idx: torch.Tensor, hot: torch.Tensor,
                   budget_bits, block: int, D: int, group: int, mass_power: float = 1.0,
                   return_ratio: bool = False):
    """Target ladder index per block for every cache row at once.

    mass (..., nb) fp32, E (..., nb, 5) fp32, idx (..., nb) current ladder index,
    hot (..., nb) bool, all CUDA; ``budget_bits`` a float or a (...,) tensor of bits/value.
    Returns int32 (..., nb); bit-exact with the reference's allocation for the same inputs.
    """
    if not mass.is_cuda:
        raise RuntimeError("allocate_rungs runs on the GPU; there is no CPU path")
    lead, nb = mass.shape[:-1], mass.shape[-1]
    problems = 1
    for s in lead:
        problems *= s
    dev = mass.device
    mass = mass.to(torch.float32).contiguous()
    E = E.to(torch.float32).contiguous()
    idx = idx.to(torch.int32).contiguous()
    hot = hot.to(torch.uint8).contiguous()
    total_vals = 2.0 * nb * block * D
    target = (torch.as_tensor(budget_bits, dtype=torch.float64, device=dev) * total_vals).expand(lead).contiguous()
    ratio = torch.empty(*lead, nb, 4, dtype=torch.float32, device=dev)
    tgt = torch.empty(*lead, nb, dtype=torch.int32, device=dev)
    bits = (C.c_float * 5)(*ladder_bits(block, D, group))
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.gkv_allocate(mass.data_ptr(), E.data_ptr(), idx.data_ptr(), hot.data_ptr(), bits,
                              target.data_ptr(), float(mass_power), ratio.data_ptr(), tgt.data_ptr(),
                              problems, nb, torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "gkv_allocate")
    return (tgt, ratio) if return_ratio else tgt


def block_distortion(cache, value_weight: float = 0.0) -> torch.Tensor:
    """Distortion table E (B, Hkv, nb, 5) of a :class:`PackedCache`, from its rung-16 blocks."""
    B, Hkv, nb = cache.level.shape
    dev = cache.data.device
    E = torch.empty(B, Hkv, nb, 5, dtype=torch.float32, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.gkv_block_distortion(cache.data.data_ptr(), cache.offs.data_ptr(), cache.level.data_ptr(),
                                      E.data_ptr(), B * Hkv, nb, cache.D, 64, cache.group, float(value_weight),
                                      cache.data.size(-1), B * Hkv, torch.cuda.current_stream(dev).cuda_stream)
    _lib.check(rc, "gkv_block_distortion")
    return E


# --------------------------------------------------------------------------- #
# Policy: the packed cache of one KV head, grown block by block
# --------------------------------------------------------------------------- #
from dataclasses import dataclass, field  # noqa: E402


@dataclass
class Report:
    """Accounting of one attention call (policies.py:188-224 of the reference)."""
    resident_bits: float = 0.0
    read_bits: float = 0.0
    total_values: int = 0
    cert_bound: float = 0.0
    true_err: float = 0.0
    n_certified: int = 0
    n_violations: int = 0
    gate_candidate_blocks: int = 0
    gate_selected_blocks: int = 0

    def merge(self, o: "Report") -> None:
        for name in ("resident_bits", "read_bits", "total_values", "cert_bound", "true_err", "n_certified",
                     "n_violations", "gate_candidate_blocks", "gate_selected_blocks"):
            setattr(self, name, getattr(self, name) + getattr(o, name))

    @property
    def bits_per_value(self) -> float:
        return self.resident_bits / max(self.total_values, 1)

    @property
    def read_bits_per_value(self) -> float:
        return self.read_bits / max(self.total_values, 1)

    @property
    def gate_keep_fraction(self) -> float:
        return 1.0 if not self.gate_candidate_blocks else self.gate_selected_blocks / self.gate_candidate_blocks


class _RowCache:
    """Packed cache of ONE cache row (one layer, sequence, KV head) that grows by whole blocks.

    Every block owns a fixed slot of the rung-16 size, so demotion rewrites a block in place at
    the start of its slot and the decode kernel then reads only the bytes of its current rung.
    """

    def __init__(self, D: int, group: int, device, capacity: int = 64):
        from .pack_layout import PackedCache, block_nbytes
        self.D, self.group, self.device = D, group, device
        self.slot = block_nbytes(16, D)
        self.n = 0
        self.cap = 0
        self.cache: PackedCache | None = None
        self.mass = torch.zeros(0, dtype=torch.float32, device=device)
        self._grow(capacity)

    def _grow(self, cap: int) -> None:
        from .pack_layout import PackedCache
        D, g, dev = self.D, self.group, self.device
        G, gv = (64 + g - 1) // g, (D + g - 1) // g
        new = PackedCache(
            torch.zeros(1, 1, cap * self.slot, dtype=torch.uint8, device=dev),
            (torch.arange(cap, device=dev, dtype=torch.int64) * self.slot).view(1, 1, cap),
            torch.zeros(1, 1, cap, G, D, dtype=torch.float16, device=dev),
            torch.zeros(1, 1, cap, G, D, dtype=torch.float16, device=dev),
            torch.zeros(1, 1, cap, 64, gv, dtype=torch.float16, device=dev),
            torch.zeros(1, 1, cap, 64, gv, dtype=torch.float16, device=dev),
            torch.full((1, 1, cap), 16, dtype=torch.int32, device=dev),
            torch.full((1, 1, cap), 64, dtype=torch.int32, device=dev), g, D)
        mass = torch.zeros(cap, dtype=torch.float32, device=dev)
        if self.cache is not None and self.n:
            n, old = self.n, self.cache
            new.data[..., : n * self.slot] = old.data[..., : n * self.slot]
            for name in ("klo", "kstep", "vlo", "vstep"):
                getattr(new, name)[:, :, :n] = getattr(old, name)[:, :, :n]
            new.level[..., :n] = old.level[..., :n]
            new.valid[..., :n] = old.valid[..., :n]
            mass[:n] = self.mass[:n]
        self.cache, self.mass, self.cap = new, mass, cap

    def view(self, n: int):
        """The first n blocks as a PackedCache (views, no copies)."""
        from .pack_layout import PackedCache
        c = self.cache
        return PackedCache(c.data, c.offs[..., :n], c.klo[:, :, :n], c.kstep[:, :, :n], c.vlo[:, :, :n],
                           c.vstep[:, :, :n], c.level[..., :n], c.valid[..., :n], c.group, c.D)

    def append(self, k: torch.Tensor, v: torch.Tensor, first: int, T: int) -> None:
        """(Re)pack blocks [first, ceil(T/64)) at rung 16 from the dense rows k, v (T, D)."""
        nb = (T + 63) // 64
        if nb > self.cap:
            self._grow(max(nb, 2 * self.cap))
        c, D = self.cache, self.D
        cnt = nb - first
        pad = nb * 64 - T
        ks, vs = k[first * 64:].float(), v[first * 64:].float()
        if pad:
            ks = torch.nn.functional.pad(ks, (0, 0, 0, pad))
            vs = torch.nn.functional.pad(vs, (0, 0, 0, pad))
        ks, vs = ks.contiguous(), vs.contiguous()
        c.level[..., first:nb] = 16
        c.valid[..., first:nb] = 64
        if pad:
            c.valid[..., nb - 1] = 64 - pad
        lib = _lib.load()
        sub = lambda t: t[:, :, first:nb].contiguous() if t.dim() > 3 else t[..., first:nb].contiguous()
        klo, kstep, vlo, vstep = (sub(t) for t in (c.klo, c.kstep, c.vlo, c.vstep))
        offs, level, valid = sub(c.offs), sub(c.level), sub(c.valid)
        with torch.cuda.device(self.device):
            rc = lib.gkv_pack_blocks(ks.data_ptr(), vs.data_ptr(), 0, c.data.data_ptr(), offs.data_ptr(),
                                     klo.data_ptr(), kstep.data_ptr(), vlo.data_ptr(), vstep.data_ptr(),
                                     level.data_ptr(), valid.data_ptr(), 1, cnt, 0, cnt, D, 64, self.group,
                                     c.data.size(-1), 1, torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(rc, "gkv_pack_blocks")
        for dst, src in ((c.klo, klo), (c.kstep, kstep), (c.vlo, vlo), (c.vstep, vstep)):
            dst[:, :, first:nb] = src
        self.n = nb

    def demote(self, new_level: torch.Tensor) -> None:
        """In-place demotion of the first n blocks to ``new_level`` (int32 (n,)); never promotes."""
        c, n = self.cache, self.n
        old = c.level[..., :n].contiguous()
        new = new_level.view(1, 1, n).to(torch.int32).contiguous()
        offs = c.offs[..., :n].contiguous()
        planes = [t[:, :, :n].contiguous() for t in (c.klo, c.kstep, c.vlo, c.vstep)]
        lib = _lib.load()
        with torch.cuda.device(self.device):
            rc = lib.gkv_demote_blocks(c.data.data_ptr(), offs.data_ptr(), old.data_ptr(), c.data.data_ptr(),
                                       offs.data_ptr(), new.data_ptr(), *(p.data_ptr() for p in planes), 1, n,
                                       self.D, 64, self.group, c.data.size(-1), c.data.size(-1), 1,
                                       torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(rc, "gkv_demote_blocks")
        for dst, src in zip((c.klo, c.kstep, c.vlo, c.vstep), planes):
            dst[:, :, :n] = src
        c.level[..., :n] = torch.minimum(old, new)


@dataclass
class Policy:
    """Cache policy.  ``name == "geodesia"`` is the packed bit-ladder cache (the reference's
    production design, policies.py:602-908); ``"full"`` attends exactly.  The other names of the
    reference are comparison baselines and are not provided here.

    Fields keep the reference's names and defaults (policies.py:227-272); the default-off
    research knobs are accepted and must stay at their defaults.
    """
    name: str = "full"
    sinks: int = 4
    window: int = 128
    block: int = 64
    obs: int = 32
    group: int = 16
    validate: bool = True
    budget_bits: float = 0.0
    layer_budget_bits: tuple = ()
    alloc_value_weight: float = 0.0
    alloc_mass_power: float = 1.0
    mass_decay: float = 0.9
    query_keep_frac: float = 1.0
    query_cold_bias: float = 0.0
    query_gate: str = "mass"
    protected_frac: float = 0.0
    token_protected_frac: float = 0.0
    spectral_rank: int = 0
    cumulant_strength: float = 0.0
    state: dict = field(default_factory=dict)
    observations: dict = field(default_factory=dict)
    report: Report = field(default_factory=Report)

    def __post_init__(self):
        if self.name not in ("full", "fullpath", "geodesia"):
            raise ValueError(f"policy '{self.name}' is a comparison baseline of the reference and is not built here")
        if self.name == "geodesia":
            if self.block != 64:
                raise ValueError("the packed format defines 64-token blocks only")
            if (self.query_keep_frac != 1.0 or self.protected_frac or self.token_protected_frac
                    or self.spectral_rank or self.cumulant_strength):
                raise ValueError("query gates, protected tokens, spectral rung and cumulant are research knobs "
                                 "of the reference that the packed path does not implement")

    def reset_state(self) -> None:
        """Forget the caches and the prompt observations (between two different prompts)."""
        self.state.clear()
        self.observations.clear()

    def reset_runtime(self) -> None:
        """Forget the caches but keep the prompt observations."""
        self.state.clear()

    def _budget_for(self, hid) -> float:
        if not self.layer_budget_bits:
            return self.budget_bits
        if hid is None:
            raise ValueError("layer_budget_bits needs an identifier hid")
        layer = int(hid[0])
        if not 0 <= layer < len(self.layer_budget_bits):
            raise ValueError(f"layer {layer} outside the profile of {len(self.layer_budget_bits)} layers")
        budget = float(self.layer_budget_bits[layer])
        if budget <= 0:
            raise ValueError("every per-layer budget must be positive")
        return budget

    # -- the reference's per-head entry point ---------------------------------------------------
    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scaling: float, q_offset: int = 0,
               hid=None, allow_demote: bool = True, observed_mass: torch.Tensor | None = None) -> torch.Tensor:
        """q (Q, D), k/v (T, D) of ONE head -> (Q, D).  Query i sees keys 0..q_offset+i."""
        return self.attend_group(q[None], k, v, scaling, q_offset, hid, allow_demote, observed_mass)[0]

    # -- all query heads that share one KV head, in one kernel call -------------------------------
    def attend_group(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scaling: float, q_offset: int = 0,
                     hid=None, allow_demote: bool = True, observed_mass: torch.Tensor | None = None) -> torch.Tensor:
        """q (R, Q, D) for the R query heads of a GQA group, k/v (T, D) -> (R, Q, D)."""
        R, Q, D = q.shape
        T = k.shape[0]
        self.report.total_values += 2 * T * D * R
        if self.name in ("full", "fullpath"):
            self.report.resident_bits += 2 * T * D * 16 * R
            self.report.read_bits += 2 * T * D * 16 * R
            return _exact_attention(q, k, v, scaling, q_offset)
        if not k.is_cuda:
            raise RuntimeError("the geodesia policy runs on the GPU; there is no CPU path")
        P = self.block
        nb = (T + P - 1) // P
        st = self.state.get(hid)
        if st is None:
            st = self.state[hid] = _RowCache(D, self.group, k.device, capacity=max(64, nb))
            prior = self.observations.get(hid, {}).get("block_mass")
        else:
            prior = None
        # new blocks enter exact; the block still being written is re-packed from the dense rows
        first = max(0, min(st.n - 1, nb - 1)) if st.n else 0
        old_n = st.n
        st.append(k, v, first, T)
        if prior is not None:
            npri = min(int(prior.numel()), nb)
            st.mass[:npri] = prior[:npri].to(device=k.device, dtype=torch.float32)
        if old_n and nb > old_n:
            st.mass[old_n:nb] = 0.0
        hot = hot_mask(nb, q_offset, P, self.sinks, self.window, device=k.device)
        if allow_demote:
            mass = observed_mass
            if mass is None:
                mass = _block_mass(q, st.view(nb), k, scaling, q_offset, nb, P)
            st.mass[:nb] = self.mass_decay * st.mass[:nb] + (1.0 - self.mass_decay) * mass.to(torch.float32)
        budget = self._budget_for(hid)
        cache = st.view(nb)
        if budget > 0 and allow_demote:
            E = block_distortion(cache, self.alloc_value_weight)[0, 0]
            idx = _ladder_index(cache.level[0, 0])
            tgt = allocate_rungs(st.mass[:nb], E, idx, hot, budget, P, D, self.group, self.alloc_mass_power)
            if bool((tgt != idx).any()):
                st.demote(_LADDER_T.to(k.device)[tgt.long()])
                cache = st.view(nb)
        bits = torch.tensor(ladder_bits(P, D, self.group), device=k.device)[_ladder_index(cache.level[0, 0]).long()]
        cache_bits = float(bits.sum()) * R
        self.report.resident_bits += cache_bits
        self.report.read_bits += cache_bits
        return _packed_attention(q, cache, scaling, q_offset, T)


_LADDER_T = torch.tensor(LADDER, dtype=torch.int32)


def _ladder_index(level: torch.Tensor) -> torch.Tensor:
    """Rung ids (16, 8, 4, 2, 1) -> ladder indices 0..4."""
    lv = level.to(torch.int32)
    return ((lv <= 8).to(torch.int32) + (lv <= 4).to(torch.int32) + (lv <= 2).to(torch.int32)
            + (lv <= 1).to(torch.int32))


def _exact_attention(q, k, v, scaling, q_offset):
    R, Q, D = q.shape
    T = k.shape[0]
    s = (q.float() @ k.float().T) * scaling
    kpos = torch.arange(T, device=k.device)
    qpos = q_offset + torch.arange(Q, device=k.device)
    s = s.masked_fill(~(kpos[None, :] <= qpos[:, None])[None], float("-inf"))
    return torch.softmax(s, -1) @ v.float()


def _block_mass(q, cache, k, scaling, q_offset, nb, P):
    """Attention mass per block of the first query position, averaged over the R heads of the group
    (policies.py:1497-1509 of the reference, which takes a dense softmax over all keys).

    A single decode query that sees the whole cache gets it as a by-product of the decode kernel over
    the packed blocks — one kernel call, no dense scores; any other call (a chunk of queries, a query
    that sees only part of the keys) is a prefill-style call and falls back to the dense softmax."""
    R, Q, D = q.shape
    T = k.shape[0]
    if Q == 1 and q_offset >= T - 1 and D in (64, 128) and cache.group in (16, 32, 64) and R <= 8:
        from .cuda_ext import get_ext
        qi = (q[:, 0].float() * scaling).view(1, R, D).contiguous()
        return get_ext().mixed_attn_decode_with_mass(qi, *cache.kernel_args())[1][0, 0]
    s = (q[:, 0].float() @ k.float().T) * scaling
    s = s.masked_fill(~(torch.arange(T, device=k.device) <= q_offset)[None], float("-inf"))
    w = torch.softmax(s, -1)
    if nb * P != T:
        w = torch.nn.functional.pad(w, (0, nb * P - T))
    return w.view(w.shape[0], nb, P).sum(-1).mean(0)


def _packed_attention(q, cache, scaling, q_offset, T):
    """Decode kernel over one packed row for R heads; one call per query position (each sees
    the keys up to its own position through the per-block valid counts)."""
    from .cuda_ext import get_ext
    ext = get_ext()
    R, Q, D = q.shape
    nb = cache.level.shape[-1]
    outs = []
    base = torch.arange(nb, device=q.device, dtype=torch.int32) * 64
    for i in range(Q):
        seen = min(q_offset + i + 1, T)
        valid = (seen - base).clamp_(0, 64).view(1, 1, nb)
        valid = torch.minimum(valid, cache.valid)
        qi = (q[:, i].float() * scaling).view(1, R, D).contiguous()
        outs.append(ext.mixed_attn_decode(qi, cache.data, cache.offs, cache.klo, cache.kstep, cache.vlo, cache.vstep,
                                          cache.level, valid.contiguous(), 64, cache.group)[0])
    return torch.stack(outs, 1)


# --------------------------------------------------------------------------- #
# transformers attention-interface functions
# --------------------------------------------------------------------------- #
ACTIVE: Policy | None = None
OBSERVER: Policy | None = None
MIN_CTX = 512


def _sdpa(module, query, key, value, attention_mask, scaling, dropout, **kwargs):
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS
    return ALL_ATTENTION_FUNCTIONS["sdpa"](module, query, key, value, attention_mask, dropout=dropout,
                                           scaling=scaling, **kwargs)


def observation_attention(module, query, key, value, attention_mask, scaling, dropout=0.0, **kwargs):
    """Exact prefill that records, per (layer, sequence, KV head), the attention mass per block of
    the last ``obs`` queries of the whole GQA group (policies.py:1393-1456); returns SDPA."""
    pol = OBSERVER
    if pol is not None and pol.name == "geodesia":
        B, H, Q, D = query.shape
        T, Hkv = key.shape[-2], key.shape[1]
        reps = H // Hkv
        n_obs = min(pol.obs, Q)
        q_start = T - Q + (Q - n_obs)
        causal = torch.arange(T, device=key.device)[None, :] <= (q_start + torch.arange(n_obs, device=key.device))[:, None]
        layer = getattr(module, "layer_idx", 0)
        nb = (T + pol.block - 1) // pol.block
        pad = nb * pol.block - T
        with torch.no_grad():
            qo = query[:, :, -n_obs:].float().reshape(B, Hkv, reps * n_obs, D)
            sc = (qo @ key.float().transpose(-1, -2)) * scaling                       # (B, Hkv, reps*n_obs, T)
            cmask = causal[None].expand(reps, -1, -1).reshape(reps * n_obs, T)
            w = torch.softmax(sc.masked_fill(~cmask, float("-inf")), -1)
            if pad:
                w = torch.nn.functional.pad(w, (0, pad))
            mass = w.view(B, Hkv, reps * n_obs, nb, pol.block).sum(-1).mean(2)        # (B, Hkv, nb)
            for b in range(B):
                for hk in range(Hkv):
                    pol.observations.setdefault((layer, b, hk), {})["block_mass"] = mass[b, hk].detach()
    return _sdpa(module, query, key, value, attention_mask, scaling, dropout, **kwargs)


def policy_attention(module, query, key, value, attention_mask, scaling, dropout=0.0, **kwargs):
    """Attention function for ``ALL_ATTENTION_FUNCTIONS`` (policies.py:1459-1519): one packed
    cache per (layer, sequence, KV head), demoted once per call with the mass of the whole GQA
    group, attended by all the group's query heads in one kernel call."""
    pol = ACTIVE
    if pol is None:
        return _sdpa(module, query, key, value, attention_mask, scaling, dropout, **kwargs)
    B, H, Q, D = query.shape
    T, Hkv = key.shape[-2], key.shape[1]
    reps = H // Hkv
    q_offset = T - Q
    layer = getattr(module, "layer_idx", 0)
    out = torch.empty(B, H, Q, D, dtype=torch.float32, device=query.device)
    for b in range(B):
        for hk in range(Hkv):
            qg = query[b, hk * reps:(hk + 1) * reps].float()
            # the mass the allocator is fed with comes out of the decode kernel (see _block_mass)
            out[b, hk * reps:(hk + 1) * reps] = pol.attend_group(qg, key[b, hk], value[b, hk], scaling, q_offset,
                                                                (layer, b, hk), True, None)
    return out.to(query.dtype).transpose(1, 2).contiguous(), None
