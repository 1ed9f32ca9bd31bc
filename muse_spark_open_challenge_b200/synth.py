"""Seeded synthetic weights and inputs with the reference's dict schema.

`generate_weights` / `generate_input` of the reference (muse_prefill_layer/reference.py:89-128,
244-326) build one hard-coded model shard.  The functions here emit the same keys, dtypes and
layouts for any `LayerShape`, including the benchmark configurations (ragged request lengths, a
layer without pooler/unpooler, a BF16 shared expert, Zipf-skewed expert load).  They are plain
torch and run on any device; nothing here is on the timed path.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace

import torch

FP8 = torch.float8_e4m3fn
QK_SCALE_FACTOR = 5.4730064863875     # reference.py:36
ROUTER_MULTIPLIER = 0.1767766952966369


@dataclass(frozen=True)
class LayerShape:
    hidden: int = 8192
    hq: int = 16
    hkv: int = 2
    head_dim: int = 64
    n_experts: int = 256
    local_experts: int = 32
    top_k: int = 8
    moe_width: int = 4096      # experts' input/output width
    inter: int = 4096          # experts' intermediate size
    pooled: bool = True        # pooler/unpooler + pre-expert norm
    shared_inter: int = 0      # BF16 shared expert's intermediate size, 0 = none
    window: int = 0
    rope_theta: float = 0.0

    @property
    def q_size(self):
        return self.hq * self.head_dim

    @property
    def kv_size(self):
        return self.hkv * self.head_dim

    @property
    def qkv_size(self):
        return 2 * self.q_size + 2 * self.kv_size


# The reference's native per-GPU shard (reference.py:29-58).
NATIVE = LayerShape()
# Benchmark configurations.
TINY = LayerShape(hidden=512, hq=8, hkv=2, head_dim=64, n_experts=16, local_experts=16, top_k=4, moe_width=256,
                  inter=256, pooled=True, rope_theta=1e6)
MID = LayerShape(hidden=4096, hq=32, hkv=8, head_dim=128, n_experts=128, local_experts=128, top_k=8,
                 moe_width=4096, inter=1536, pooled=False, shared_inter=4096, rope_theta=1e6)
MOE_ONLY = replace(MID, shared_inter=0)
LONG_EP = replace(MID, n_experts=256, local_experts=32)


def _nvfp4_bank(gen, device, leading, rows, k, std):
    """Random NVFP4 weights: uniform 4-bit codes, log-normal E4M3 block scales (log2 ~ N(7, .4),
    clamped to [8, 448]) and a global scale that gives dequantised values of deviation `std`
    (the construction of muse_prefill_layer/nvfp4.py:105-131, with the target deviation free)."""
    packed = torch.randint(0, 256, (*leading, rows, k // 2), dtype=torch.uint8, generator=gen, device=device)
    z = torch.randn((*leading, rows, k // 16), generator=gen, device=device)
    sf = torch.exp2(7.0 + 0.4 * z).clamp(8.0, 448.0).to(FP8)
    mean_sq = 4.0 ** 7.0 * math.exp(2 * (math.log(2) * 0.4) ** 2)
    gs = std / math.sqrt(8.6 * mean_sq)
    gs = gs * torch.exp(0.5 * torch.randn(leading, generator=gen, device=device))   # per-expert spread
    return packed, sf, gs.float()


def make_weights(shape: LayerShape, seed: int = 0, device: str = "cpu", std: float = 0.02,
                 router_bias_std: float = 0.055, expert_offsets: torch.Tensor | None = None) -> dict:
    """Weights ~ N(0, std) in the reference's layouts (baseline.py:66-86).  `expert_offsets`
    [n_experts] is added to the router bias AND returned under "route_offsets" so a caller can
    skew the load; the skew lives in the router rows (see `skew_router`)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    s = shape

    def dense(n, k):
        return (std * torch.randn((n, k), generator=gen, device=device)).to(torch.bfloat16)

    def vec(n, dev):
        return (dev * torch.randn((n,), generator=gen, device=device)).to(torch.bfloat16)

    w = {
        "qkv_gate": dense(s.qkv_size, s.hidden),
        "o": dense(s.hidden, s.q_size),
        "attn_residual_gate": vec(s.hidden, 0.3),
        "pre_ffn_norm": vec(s.hidden, 0.1),
        "router": (0.045 * torch.randn((s.n_experts, s.hidden), generator=gen, device=device)).contiguous(),
        "router_bias": (router_bias_std * torch.randn((s.n_experts,), generator=gen, device=device)).contiguous(),
    }
    if s.pooled:
        w["pooler"] = dense(s.moe_width, s.hidden)
        w["pre_expert_norm"] = vec(s.moe_width, 0.1)
    w["w13"], w["w13_sf"], w["w13_gs"] = _nvfp4_bank(gen, device, (s.local_experts,), 2 * s.inter, s.moe_width,
                                                     1.0 / math.sqrt(s.moe_width))
    w["w2"], w["w2_sf"], w["w2_gs"] = _nvfp4_bank(gen, device, (s.local_experts,), s.moe_width, s.inter,
                                                  1.0 / math.sqrt(s.inter))
    w["post_expert_norm"] = vec(s.moe_width, 0.1)
    if s.pooled:
        w["unpooler"] = dense(s.hidden, s.moe_width)
    if s.shared_inter:
        w["shared_w13"] = dense(2 * s.shared_inter, s.moe_width)
        w["shared_w2"] = dense(s.moe_width, s.shared_inter)
    w["post_ffn_norm"] = vec(s.hidden, 0.1)
    w["ffn_residual_gate"] = vec(s.hidden, 0.3)
    w["next_pre_attn_norm"] = vec(s.hidden, 0.1)
    return w


def config_of(shape: LayerShape, batch: int, tokens: int, q_len: int, page: int, kv_scale: float) -> dict:
    """The per-call config dict (reference.py:308-325)."""
    return {"batch": batch, "q_len": q_len, "tokens": tokens, "hidden": shape.hidden, "num_q_heads": shape.hq,
            "num_kv_heads": shape.hkv, "head_dim": shape.head_dim, "page_size": page, "window": shape.window,
            "rope_theta": shape.rope_theta, "qk_scale_factor": QK_SCALE_FACTOR, "sm_scale": shape.head_dim ** -0.5,
            "kv_scale": kv_scale, "n_experts": shape.n_experts, "top_k": shape.top_k,
            "local_experts": shape.local_experts}


def make_input(shape: LayerShape, new_lens, ctx_lens, seed: int = 0, page: int = 64, kv_scale: float = 1.0,
               local_start: int = 0, device: str = "cpu", fill_cache: bool = True) -> dict:
    """One prefill step: request b adds new_lens[b] tokens after ctx_lens[b] cached ones.
    Same keys as reference.generate_input; `q_len` in the config is the longest request, and
    `cu_seqlens_q` carries the (possibly ragged) lengths.  Pages are scattered through the pool
    by a seeded permutation (reference.py:261-266)."""
    gen = torch.Generator(device=device).manual_seed(seed)
    s = shape
    new_lens, ctx_lens = list(new_lens), list(ctx_lens)
    batch, tokens = len(new_lens), sum(new_lens)
    pages_per = [(c + n + page - 1) // page for c, n in zip(ctx_lens, new_lens)]
    max_pages = max(pages_per)
    total = sum(pages_per)
    perm = torch.randperm(total, generator=gen, device=device).to(torch.int32)
    page_table = torch.full((batch, max_pages), -1, dtype=torch.int32, device=device)
    at = 0
    for b, n in enumerate(pages_per):
        page_table[b, :n] = perm[at:at + n]
        at += n
    positions = torch.cat([c + torch.arange(n, device=device) for c, n in zip(ctx_lens, new_lens)]).long()
    req = torch.cat([torch.full((n,), b, dtype=torch.long, device=device) for b, n in enumerate(new_lens)])
    cache_loc = page_table.long()[req, positions // page] * page + positions % page
    cshape = (total, page, s.hkv, s.head_dim)
    if fill_cache:
        k_cache = (torch.randn(cshape, generator=gen, device=device) / kv_scale).to(FP8)
        v_cache = (torch.randn(cshape, generator=gen, device=device) / kv_scale).to(FP8)
    else:
        k_cache = torch.zeros(cshape, dtype=FP8, device=device)
        v_cache = torch.zeros(cshape, dtype=FP8, device=device)
    stream = torch.randn((tokens, s.hidden), generator=gen, device=device)
    attn_input = (stream * torch.rsqrt(stream.pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16)
    cu = torch.zeros(batch + 1, dtype=torch.int32, device=device)
    cu[1:] = torch.cumsum(torch.tensor(new_lens, device=device), 0).to(torch.int32)
    seq_lens = torch.tensor(ctx_lens, dtype=torch.int32, device=device)
    return {
        "stream": stream, "attn_input": attn_input, "positions": positions, "cache_loc": cache_loc,
        "cache_seqlens": seq_lens + torch.tensor(new_lens, dtype=torch.int32, device=device),
        "cu_seqlens_q": cu, "scheduler_metadata": None, "k_cache": k_cache, "v_cache": v_cache,
        "k_scale": torch.tensor(kv_scale, dtype=torch.float32, device=device),
        "v_scale": torch.tensor(kv_scale, dtype=torch.float32, device=device),
        "page_table": page_table, "seq_lens": seq_lens,
        "local_start": torch.tensor([local_start], dtype=torch.int32, device=device),
        "config": config_of(s, batch, tokens, max(new_lens), page, kv_scale),
    }


def uniform_lengths(batch: int, lo: int, hi: int, seed: int = 0) -> list[int]:
    """Lengths lo + floor(u * (hi - lo + 1)) from a seeded CPU generator."""
    u = torch.rand((batch,), generator=torch.Generator().manual_seed(seed))
    return (lo + (u * (hi - lo + 1)).floor().long()).clamp(max=hi).tolist()


def zipf_targets(n_experts: int, routes: int, s: float = 1.1, cap: int = 3000, n_empty: int = 2) -> torch.Tensor:
    """Target routes per expert: proportional to rank^-s, clipped at `cap` with the excess
    re-spread over the unclipped ranks, the last `n_empty` ranks at zero."""
    live = n_experts - n_empty
    w = torch.arange(1, live + 1, dtype=torch.float64).pow(-s)
    t = torch.zeros(live, dtype=torch.float64)
    free = torch.ones(live, dtype=torch.bool)
    left = float(routes)
    for _ in range(live):
        share = w * free
        t = torch.where(free, share / share.sum() * left, t)
        over = free & (t > cap)
        if not over.any():
            break
        t[over] = cap
        free &= ~over
        left = routes - float(cap) * int((~free).sum())
    return torch.cat([t, torch.zeros(n_empty, dtype=torch.float64)])


def skew_router(weights: dict, h: torch.Tensor, targets: torch.Tensor, top_k: int, iters: int = 40,
                sample: int = 4096, seed: int = 0, identity: bool = False) -> torch.Tensor:
    """Shift `router_bias` per expert, in place, until the top-k routing of `h` [T, H] (a sample
    of it) has per-expert counts close to `targets` (a permutation of them over experts, seeded).
    Experts with target 0 get a bias so low they are never chosen.  Returns the permutation."""
    e = weights["router"].shape[0]
    g = torch.Generator().manual_seed(seed)
    perm = torch.arange(e) if identity else torch.randperm(e, generator=g)     # identity: target i is expert i's
    tgt = torch.empty(e, dtype=torch.float64)
    tgt[perm] = targets
    idx = torch.randperm(h.shape[0], generator=g)[:sample].to(h.device)
    hs = h[idx].float()
    scores = torch.sigmoid((hs @ weights["router"].float().T) * ROUTER_MULTIPLIER).cpu().double()
    base = weights["router_bias"].double().cpu()
    off = torch.zeros(e, dtype=torch.float64)
    want = tgt / tgt.sum() * (hs.shape[0] * top_k)
    dead = tgt <= 0
    for _ in range(iters):
        biased = scores + base + off
        biased[:, dead] = -10.0
        ids = biased.topk(top_k, dim=-1).indices
        got = torch.bincount(ids.flatten(), minlength=e).double()
        off += 0.08 * torch.log((want + 0.5) / (got + 0.5))
        off.clamp_(-3.0, 3.0)
    off[dead] = -10.0
    weights["router_bias"] = (base + off).float().to(weights["router_bias"].device).contiguous()
    return perm
