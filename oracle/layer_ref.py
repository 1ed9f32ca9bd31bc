"""TEST INFRASTRUCTURE ONLY: CPU restatement of the reference's MoE decoder layer at prefill.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the
product path never does and fails loudly without its CUDA library.

The reference (muse_prefill_layer/reference.py) hard-codes one model shard in module globals.
This restatement follows the same arithmetic, operation by operation, but reads every size from
a `Dims` record, so the same oracle serves the reference's native shard and the synthetic
benchmark configurations.  Three things have no counterpart in the reference and are defined
here (and nowhere else): a per-request number of new tokens (`cu_seqlens_q`), a layer without
pooler/unpooler (`Dims.pooled == False`: the experts read the FFN input directly and their sum
is the FFN branch), and a dense BF16 shared expert added to the routed sum.

Parity pin: `oracle/check_against_reference.py` runs this file and the unmodified reference on
the same seeded inputs in a container that holds the reference and requires identical tensors;
`tests/golden/` stores reference-made input/output vectors that `tests/test_oracle_golden.py`
replays anywhere.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

FP8 = torch.float8_e4m3fn
RMS_EPS = 1e-5            # reference.py:38
POST_NORM_EPS = 1e-8      # reference.py:39
ROUTER_MULTIPLIER = 0.1767766952966369   # reference.py:51
ROUTE_EPS = 1e-15         # reference.py:53
SLICED_MAX_TOKENS = 8      # reference.py:58
RESIDUAL_TEMPERATURE = 0.3   # reference.py:54
RESIDUAL_GATE_EPS = 1e-3     # reference.py:55
QUERY_CHUNK = 2048
NVFP4_BLOCK = 16
_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


@dataclass(frozen=True)
class Dims:
    hidden: int
    hq: int
    hkv: int
    head_dim: int
    n_experts: int
    local_experts: int
    top_k: int
    moe_width: int        # the experts' input/output width (reference: D_EXPERT)
    inter: int            # the experts' intermediate size (reference: D_EXPERT as well)
    pooled: bool          # pooler/unpooler + pre-expert norm present (reference: always)
    shared_inter: int     # 0 = no shared expert (reference: none)

    @property
    def q_size(self):
        return self.hq * self.head_dim

    @property
    def kv_size(self):
        return self.hkv * self.head_dim


def dims_of(weights: dict, config: dict) -> Dims:
    """Sizes from the weight shapes and the per-call config (reference.py:29-58 as globals)."""
    el, two_i, half_w = weights["w13"].shape
    pooled = "pooler" in weights
    return Dims(
        hidden=weights["qkv_gate"].shape[1], hq=config["num_q_heads"], hkv=config["num_kv_heads"],
        head_dim=config["head_dim"], n_experts=weights["router"].shape[0], local_experts=el,
        top_k=config["top_k"], moe_width=2 * half_w, inter=two_i // 2, pooled=pooled,
        shared_inter=(weights["shared_w13"].shape[0] // 2 if "shared_w13" in weights else 0))


# ---------------------------------------------------------------- small pieces
def rms(x, eps=RMS_EPS):
    """reference.py:189-191."""
    x = x.float()
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def quant_fp8(x, scale):
    """reference.py:181-182 (torch's e4m3fn cast: round-to-nearest-even, no saturation)."""
    return (x.float() / scale).to(FP8)


def dequant_fp8(x, scale):
    return x.float() * scale


def rope_interleaved(x, pos, theta, head_dim):
    """reference.py:329-336: pairs (2i, 2i+1) rotate by pos * theta^(-2i/head_dim)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    ang = pos.float()[:, None] * inv_freq
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    even, odd = x[..., 0::2], x[..., 1::2]
    return torch.stack([even * cos - odd * sin, even * sin + odd * cos], -1).flatten(-2)


def residual_coefficients(gate):
    """reference.py:339-344."""
    w = gate.float() / RESIDUAL_TEMPERATURE
    beta = torch.sigmoid(w)
    alpha = torch.sqrt(torch.clamp(torch.sigmoid(-w) * (1.0 + beta), min=RESIDUAL_GATE_EPS))
    return alpha, beta


_E2M1_MIDS = (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0)       # nvfp4.py:27


def nvfp4_quantize_rows(x):
    """The reference's NVFP4 quantiser (muse_prefill_layer/nvfp4.py:59-88) applied to every row with
    that row's own tensor scale: scale_r = amax_r / (6 * 448), block scale = e4m3(amax_block / 6 /
    scale_r), element codes = nearest grid value of x / (block scale * scale_r).  Returns (values on
    the e2m1 grid fp32 [rows, k], block scales fp32 [rows, k/16], row scales fp32 [rows]).  Exact
    mid-points between two grid values go to the lower magnitude here (torch.bucketize,
    nvfp4.py:52-53) and to the even code in the hardware conversion; real inputs do not hit them."""
    xf = x.float()
    rows, k = xf.shape
    amax = xf.abs().amax(dim=-1)
    rs = torch.where(amax > 0, amax / (6.0 * 448.0), torch.ones_like(amax))
    blocks = xf.view(rows, k // NVFP4_BLOCK, NVFP4_BLOCK)
    sf = (blocks.abs().amax(dim=-1) / 6.0 / rs[:, None]).clamp(max=448.0).to(torch.float8_e4m3fn).float()
    scale = (sf * rs[:, None]).unsqueeze(-1)
    q = torch.where(scale > 0, blocks / scale, torch.zeros_like(blocks))
    mids = torch.tensor(_E2M1_MIDS, dtype=torch.float32)
    grid = torch.tensor(_E2M1, dtype=torch.float32)
    mag = grid[torch.bucketize(q.abs().clamp(max=6.0), mids)]
    return (torch.sign(q) * mag).view(rows, k), sf, rs


def nvfp4_dequantize(packed, sf, gs):
    """muse_prefill_layer/nvfp4.py:40-47,90-97 in torch (see oracle/nvfp4_ref.py for numpy)."""
    p = packed.view(torch.uint8)
    codes = torch.stack((p & 0xF, (p >> 4) & 0xF), dim=-1).flatten(-2)
    grid = torch.tensor(_E2M1, dtype=torch.float32)
    mag = grid[(codes & 7).long()]
    vals = torch.where((codes & 8) != 0, -mag, mag)
    k = vals.shape[-1]
    blocks = vals.view(*vals.shape[:-1], k // NVFP4_BLOCK, NVFP4_BLOCK)
    scale = sf.float() * torch.as_tensor(gs, dtype=torch.float32)
    return (blocks * scale.unsqueeze(-1)).view_as(vals)


def request_lengths(data) -> list[int]:
    """New tokens per request. The reference has one q_len for all (reference.py:289);
    here cu_seqlens_q may be ragged."""
    cu = data["cu_seqlens_q"].tolist()
    return [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]


def token_positions(data) -> torch.Tensor:
    """Position of every new token, request-major (reference.py:363)."""
    seq = data["seq_lens"].tolist()
    return torch.cat([s + torch.arange(n) for s, n in zip(seq, request_lengths(data))]).long()


def new_slots(data) -> torch.Tensor:
    """Flat cache row of every new token, request-major [T] (reference.py:347-353)."""
    size = data["config"]["page_size"]
    out = []
    for b, (s, n) in enumerate(zip(data["seq_lens"].tolist(), request_lengths(data))):
        pos = s + torch.arange(n)
        page = data["page_table"][b].long()[pos // size]
        out.append(page * size + pos % size)
    return torch.cat(out)


# ---------------------------------------------------------------- attention
def attend(q, k_new, v_new, data, d: Dims):
    """Causal attention of the new tokens over the cached prefix plus the block itself
    (reference.py:376-408).  q fp32 [T, HQ, D] already scaled; k_new/v_new FP8 [T, HKV, D].
    Returns fp32 [T, HQ, D]."""
    cfg = data["config"]
    window, size = cfg["window"], cfg["page_size"]
    k_flat = data["k_cache"].view(-1, d.hkv, d.head_dim)
    v_flat = data["v_cache"].view(-1, d.hkv, d.head_dim)
    group = d.hq // d.hkv
    out = torch.empty((q.shape[0], d.hq, d.head_dim))
    at = 0
    for b, length in enumerate(request_lengths(data)):
        seq = int(data["seq_lens"][b])
        first = max(0, seq - window + 1) if window else 0
        past = torch.arange(first, seq)
        rows = data["page_table"][b].long()[past // size] * size + past % size
        sl = slice(at, at + length)
        keys = torch.cat([dequant_fp8(k_flat[rows], data["k_scale"]), dequant_fp8(k_new[sl], data["k_scale"])])
        vals = torch.cat([dequant_fp8(v_flat[rows], data["v_scale"]), dequant_fp8(v_new[sl], data["v_scale"])])
        steps = torch.arange(length)
        key_pos = torch.cat([past, seq + steps])
        keys_h = keys.repeat_interleave(group, dim=1).transpose(0, 1)   # [HQ, S, D]
        vals_h = vals.repeat_interleave(group, dim=1).transpose(0, 1)
        for c in range(0, length, QUERY_CHUNK):
            j = slice(c, min(c + QUERY_CHUNK, length))
            query_pos = seq + steps[j]
            visible = key_pos[None, :] <= query_pos[:, None]
            if window:
                visible &= key_pos[None, :] > query_pos[:, None] - window
            qq = q[sl][j].transpose(0, 1)   # [HQ, n, D]
            att = torch.einsum("hnd,hsd->hns", qq, keys_h) * cfg["sm_scale"]
            att = att.masked_fill(~visible[None], float("-inf")).softmax(-1)
            out[at + c: at + c + att.shape[1]] = torch.einsum("hns,hsd->hnd", att, vals_h).transpose(0, 1)
        at += length
    return out


def attention_block(data, x, weights, d: Dims, query_dtype=torch.bfloat16):
    """reference.py:356-410: QKV(+gate) projection, per-head RMS norm of q and k, interleaved
    RoPE when rope_theta != 0, query rounding, FP8 cache entries, attention, per-head RMS norm of
    the output times sigmoid(gate).  Returns (o_in fp32 [T, HQ*D], k_new, v_new FP8 [T, HKV, D])."""
    cfg = data["config"]
    qkv = x @ weights["qkv_gate"].float().T
    q, k, v, gate = qkv.split([d.q_size, d.kv_size, d.kv_size, d.q_size], dim=-1)
    pos = token_positions(data)
    q = rms(q.reshape(-1, d.hq, d.head_dim))
    k = rms(k.reshape(-1, d.hkv, d.head_dim))
    if cfg["rope_theta"]:
        q = rope_interleaved(q, pos, cfg["rope_theta"], d.head_dim)
        k = rope_interleaved(k, pos, cfg["rope_theta"], d.head_dim)
    if query_dtype == torch.bfloat16:
        q = (q * cfg["qk_scale_factor"]).to(torch.bfloat16).float()
    else:
        q = q.to(query_dtype).float() * cfg["qk_scale_factor"]
    k_new = quant_fp8(k, data["k_scale"])
    v_new = quant_fp8(v.reshape(-1, d.hkv, d.head_dim), data["v_scale"])
    out = attend(q, k_new, v_new, data, d)
    out = rms(out).reshape(-1, d.q_size) * torch.sigmoid(gate)
    return out, k_new, v_new


# ---------------------------------------------------------------- router and experts
def route(h, weights):
    """reference.py:419-424: fp64 logits, sigmoid, + bias (bias only chooses)."""
    logits = h.double() @ weights["router"].double().T
    scores = torch.sigmoid(logits * ROUTER_MULTIPLIER).float()
    return scores, scores + weights["router_bias"].float()


def topk_ids(biased, k):
    """The k largest biased scores per token, lowest index first among exact ties (the
    reference takes torch.topk at reference.py:564; its shipped kernel breaks ties the same
    way, submission.py:873)."""
    order = torch.sort(biased, dim=-1, descending=True, stable=True).indices
    return order[:, :k].to(torch.int32)


def route_weights(scores, ids):
    """reference.py:462-463."""
    picked = scores.gather(1, ids.long())
    return picked / (picked.sum(-1, keepdim=True) + ROUTE_EPS)


def post_expert_norm(y, w):
    """reference.py:427-430: scale by (1 + w), then RMS norm with eps 1e-8."""
    y = y.float() * (1.0 + w.float())
    return y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + POST_NORM_EPS)


def experts(x, local_ids, topk_weights, weights, d: Dims):
    """reference.py:433-444: per local expert, gate/up GEMM on dequantised NVFP4 weights,
    SiLU(gate) * up, down GEMM, post-expert norm, weighted sum per token."""
    out = torch.zeros((x.shape[0], d.moe_width), dtype=torch.float32)
    for e in torch.unique(local_ids).tolist():
        if not 0 <= e < d.local_experts:
            continue
        tok, slot = (local_ids == e).nonzero(as_tuple=True)
        w13 = nvfp4_dequantize(weights["w13"][e], weights["w13_sf"][e], weights["w13_gs"][e])
        h = x[tok] @ w13.T
        inter = torch.nn.functional.silu(h[:, :d.inter]) * h[:, d.inter:]
        w2 = nvfp4_dequantize(weights["w2"][e], weights["w2_sf"][e], weights["w2_gs"][e])
        y = inter @ w2.T
        out.index_add_(0, tok, post_expert_norm(y, weights["post_expert_norm"]) * topk_weights[tok, slot, None])
    return out


def shared_expert(x, weights, d: Dims):
    """Dense gated MLP on BF16 weights: silu(x Wg^T) * (x Wu^T) then Wd^T; gate rows first in
    shared_w13 like the routed banks.  No counterpart in the reference."""
    h = x @ weights["shared_w13"].float().T
    inter = torch.nn.functional.silu(h[:, :d.shared_inter]) * h[:, d.shared_inter:]
    return inter @ weights["shared_w2"].float().T


# ---------------------------------------------------------------- the two halves and the layer
def ref_front(data, weights, query_dtype=torch.bfloat16):
    """reference.py:447-457."""
    d = dims_of(weights, data["config"])
    o, k_new, v_new = attention_block(data, data["attn_input"].float(), weights, d, query_dtype)
    a = o @ weights["o"].float().T
    alpha1, beta1 = residual_coefficients(weights["attn_residual_gate"])
    stream1 = alpha1 * data["stream"].float() + beta1 * rms(a, POST_NORM_EPS)
    h = rms(stream1) * (1.0 + weights["pre_ffn_norm"].float())
    scores, biased = route(h, weights)
    return {"stream1": stream1, "h": h, "scores": scores, "biased": biased, "k_new": k_new, "v_new": v_new,
            "local_start": int(data["local_start"]), "dims": d}


def moe_block(h, scores, ids, local_start, weights, d: Dims):
    """The FFN branch before its boundary (reference.py:462-472).  Returns fp32 [T, hidden]."""
    tw = route_weights(scores, ids)
    if d.pooled:
        p = h @ weights["pooler"].float().T
        p = rms(p) * (1.0 + weights["pre_expert_norm"].float())
    else:
        p = h
    local = (ids.long() - local_start) % d.n_experts
    moe = experts(p, local, tw, weights, d)
    if d.shared_inter:
        moe = moe + shared_expert(p, weights, d)
    if d.pooled:
        if len(moe) <= SLICED_MAX_TOKENS:
            # decode / verify blocks: this GPU forms only its hidden/8 columns (reference.py:56-58,468-470)
            cols = d.hidden // 8
            f = torch.zeros((len(moe), d.hidden), dtype=moe.dtype)
            f[:, :cols] = moe @ weights["unpooler"][:cols].float().T
            return f
        return moe @ weights["unpooler"].float().T
    return moe


def ref_back(front, weights, ids):
    """reference.py:460-477."""
    d = front["dims"]
    f = moe_block(front["h"], front["scores"], ids, front["local_start"], weights, d)
    f = f * (1.0 + weights["post_ffn_norm"].float())
    alpha2, beta2 = residual_coefficients(weights["ffn_residual_gate"])
    stream2 = alpha2 * front["stream1"] + beta2 * rms(f, POST_NORM_EPS)
    hidden = rms(stream2) * (1.0 + weights["next_pre_attn_norm"].float())
    return hidden.to(torch.bfloat16), stream2


def ref_kernel(data, weights, topk=None, query_dtype=torch.bfloat16):
    """reference.py:559-566.  Returns (hidden bf16 [T,H], stream fp32 [T,H], ids int32 [T,K],
    k_new, v_new FP8 [T,HKV,D])."""
    front = ref_front(data, weights, query_dtype)
    ids = topk_ids(front["biased"], front["dims"].top_k) if topk is None else topk
    hidden, stream = ref_back(front, weights, ids)
    return hidden, stream, ids, front["k_new"], front["v_new"]


# ---------------------------------------------------------------- checks (reference.py:609-672, checks.py)
def relative_l2(a, b) -> float:
    return float((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12))


def error_report(out, ref) -> dict:
    """The three error figures stated for the layer output: whole-tensor relative L2, mean
    absolute error, and the largest absolute error divided by the reference's RMS."""
    o, r = out.float(), ref.float()
    diff = (o - r).abs()
    return {"rel_l2": relative_l2(o, r), "mean_abs": float(diff.mean()),
            "max_over_rms": float(diff.max() / r.pow(2).mean().sqrt().clamp(min=1e-12))}


def compare_rows(out, ref, tol, row_factor=5.0, row_floor=0.1):
    """checks.py:31-55: whole-tensor relative L2 <= tol and each row <= row_factor * tol, a row
    being measured against max(its norm, row_floor * mean row norm)."""
    o, r = out.float(), ref.float()
    if not torch.isfinite(o).all():
        return False, "NaN or Inf"
    diff = o - r
    err = float(diff.norm() / r.norm().clamp(min=1e-12))
    rows_ref = r.reshape(-1, r.shape[-1]).norm(dim=-1)
    floor = (row_floor * rows_ref.mean()).clamp(min=1e-12)
    row_err = diff.reshape(-1, r.shape[-1]).norm(dim=-1) / torch.maximum(rows_ref, floor)
    worst = float(row_err.max())
    ok = err <= tol and worst <= row_factor * tol
    return ok, f"rel-L2 {err:.3e} (worst row {worst:.3e}) vs {tol:g}"


def check_routing(ids, biased, d: Dims, local_start=0, route_tol=5e-2, keep_tol=(0.03, 0.04), keep_tokens=256,
                  local_slack=(0.08, 4), distinct_slack=(0.15, 2)):
    """reference.py:609-637, None when acceptable."""
    k = d.top_k
    if ids.min() < 0 or ids.max() >= d.n_experts:
        return "expert id out of range"
    ranked = ids.long().sort(-1).values
    if (ranked[:, 1:] == ranked[:, :-1]).any():
        return "a token routed to the same expert twice"
    best = biased.topk(k, dim=-1)
    gap = best.values[:, -1:] - biased.gather(1, ids.long())
    if gap.max() > route_tol:
        return f"a pick is {float(gap.max()):.2e} below the k-th best"
    if d.n_experts > k:
        nxt = biased.topk(k + 1, dim=-1).values[:, -1:]
        tol = keep_tol[0] if len(ids) <= keep_tokens else keep_tol[1]
        kept = (best.indices[:, :, None] == ids.long()[:, None, :]).any(-1)
        local = (best.indices - local_start) % d.n_experts < d.local_experts
        if (local & ~kept & (best.values - nxt > tol)).any():
            return "dropped a clear local pick"

    def load(x):
        loc = x[(x - local_start) % d.n_experts < d.local_experts]
        return int(loc.numel()), int(torch.unique(loc).numel())
    routes, distinct = load(ids.long())
    ref_routes, ref_distinct = load(best.indices)
    if routes < ref_routes * (1 - local_slack[0]) - local_slack[1]:
        return f"{routes} local routes vs {ref_routes}"
    if distinct < ref_distinct * (1 - distinct_slack[0]) - distinct_slack[1]:
        return f"{distinct} local experts vs {ref_distinct}"
    return None


def check_layer(data, weights, hidden, stream, ids, k_rows, v_rows, rel_l2_tol=0.15, factor=2.5, floor=0.03,
                cache_tol=8e-2):
    """reference.py:640-672: routing check, then the residual update and the next attention
    input against the fp32 reference run with the SAME expert ids, with bounds derived from the
    reference's own FP8-query error; new cache rows within cache_tol (dequantised)."""
    front = ref_front(data, weights)
    d = front["dims"]
    err = check_routing(ids, front["biased"], d, front["local_start"])
    if err:
        return False, f"routing: {err}", {}
    ref_hidden, ref_stream = ref_back(front, weights, ids)
    a1, _ = residual_coefficients(weights["attn_residual_gate"])
    a2, _ = residual_coefficients(weights["ffn_residual_gate"])
    carried = a1 * a2 * data["stream"].float()
    q8_hidden, q8_stream = ref_back(ref_front(data, weights, FP8), weights, ids)
    bound = lambda e: min(rel_l2_tol, max(floor, factor * e))  # noqa: E731
    tol = bound(relative_l2(q8_stream - carried, ref_stream - carried))
    htol = bound(relative_l2(q8_hidden, ref_hidden))
    report = {"update_vs_fp32": error_report(stream - carried, ref_stream - carried),
              "hidden_vs_fp32": error_report(hidden, ref_hidden),
              "update_vs_fp8q": error_report(stream - carried, q8_stream - carried),
              "hidden_vs_fp8q": error_report(hidden, q8_hidden),
              "update_bound": tol, "hidden_bound": htol}
    ok, msg = compare_rows(stream - carried, ref_stream - carried, tol)
    if not ok:
        return False, f"residual update: {msg}", report
    ok, hmsg = compare_rows(hidden, ref_hidden, htol)
    if not ok:
        return False, f"next attention input: {hmsg}", report
    for name, got, want, scale in (("key", k_rows, front["k_new"], data["k_scale"]),
                                   ("value", v_rows, front["v_new"], data["v_scale"])):
        ok, kmsg = compare_rows(dequant_fp8(got, scale), dequant_fp8(want, scale), cache_tol)
        if not ok:
            return False, f"new {name} cache rows: {kmsg}", report
    return True, f"update {msg}; attention input {hmsg}", report
