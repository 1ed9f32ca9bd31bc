"""Drop-in entry points of the reference's prefill layer: `prepare(weights)` and
`kernel_fn(data, state)` (muse_prefill_layer/submission.py:1013,1073; contract in TASK.md:27 and
baseline.py:66-122).

`prepare` runs once: it re-tiles the NVFP4 expert banks losslessly, splits the fp32 router into a
BF16 hi + lo pair, precomputes the residual coefficients and (1 + w) norm vectors in fp32, and
allocates grow-only scratch.  `kernel_fn` is a straight-line sequence of launches from libmsl.so on
the current stream: no host synchronisation, no data-dependent allocation or branching, so it can
be captured in a CUDA graph and replayed on fresh inputs of the same shape.

All sizes come from the weight shapes and `data["config"]`, so the same code serves the
reference's native shard and the benchmark configurations.  Beyond the reference's contract:
`cu_seqlens_q` may be ragged; without "pooler"/"unpooler" weights the experts read the FFN input
directly; "shared_w13"/"shared_w2" add a dense BF16 shared expert.
"""
from __future__ import annotations

import os

import torch

from . import ops
from ._lib import OUT_BF16, OUT_F32, OUT_SWIGLU_BF16, ERR_CAPACITY, ERR_DEVICE_TIMEOUT, MslError

ROUTER_MULTIPLIER = 0.1767766952966369      # reference.py:51
RMS_EPS, POST_NORM_EPS = 1e-5, 1e-8         # reference.py:38-39


def _coeffs(gate):
    """Residual coefficients (reference.py:339-344), fp32."""
    w = gate.float() / 0.3
    beta = torch.sigmoid(w)
    alpha = torch.sqrt(torch.clamp(torch.sigmoid(-w) * (1.0 + beta), min=1e-3))
    return alpha.contiguous(), beta.contiguous()


def prepare(weights: dict, experts_nvfp4: bool = None) -> dict:
    """One-time preparation of a layer's weights.  `experts_nvfp4` opts in to running the routed experts
    with NVFP4 activations on the block-scaled tensor-core path (default: the environment variable
    MSL_EXPERTS_NVFP4=1, read here once, else off): about twice the expert rate, at the cost of 4-bit
    activations, which the reference's contract does not allow (TASK.md:89: BF16 activations), so the
    default stays W4A16."""
    dev = weights["qkv_gate"].device
    if dev.type != "cuda":
        raise MslError("prepare() needs CUDA tensors: this implementation has no CPU path")
    if experts_nvfp4 is None:
        experts_nvfp4 = os.environ.get("MSL_EXPERTS_NVFP4", "0") == "1"
    st = {"device": dev, "experts_nvfp4": bool(experts_nvfp4)}
    st["qkv_gate"] = weights["qkv_gate"].contiguous()
    st["o"] = weights["o"].contiguous()
    router = weights["router"].float()
    hi = router.to(torch.bfloat16)
    lo = (router - hi.float()).to(torch.bfloat16)
    st["router_hilo"] = torch.cat([hi, lo], dim=1).contiguous()       # [E, 2H]: hi | lo per row
    st["router_bias"] = weights["router_bias"].float().contiguous()
    st["n_experts"] = router.shape[0]
    st["a1"], st["b1"] = _coeffs(weights["attn_residual_gate"])
    st["a2"], st["b2"] = _coeffs(weights["ffn_residual_gate"])
    for dst, src in (("w_pre_ffn", "pre_ffn_norm"), ("w_post_exp", "post_expert_norm"),
                     ("w_post_ffn", "post_ffn_norm"), ("w_next", "next_pre_attn_norm")):
        st[dst] = (1.0 + weights[src].float()).contiguous()
    st["pooled"] = "pooler" in weights
    if st["pooled"]:
        st["pooler"] = weights["pooler"].contiguous()
        st["unpooler"] = weights["unpooler"].contiguous()
        st["w_pre_exp"] = (1.0 + weights["pre_expert_norm"].float()).contiguous()
    el, two_i, half_w = weights["w13"].shape
    st["n_local"], st["inter"], st["moe_width"] = el, two_i // 2, 2 * half_w
    if st["experts_nvfp4"]:
        if st["moe_width"] % 256 or st["inter"] % 256:
            raise MslError("experts_nvfp4 needs an expert width and intermediate size that are multiples of 256")
        # the 4-bit codes are consumed as the reference stores them; only the block scales are re-tiled
        st["w13_codes"] = weights["w13"].view(torch.uint8).contiguous()
        st["w2_codes"] = weights["w2"].view(torch.uint8).contiguous()
        st["w13_sf_t"] = ops.nvfp4_bs_sf_repack(weights["w13_sf"], True)
        st["w2_sf_t"] = ops.nvfp4_bs_sf_repack(weights["w2_sf"], False)
    else:
        st["w13_q"], st["w13_s"], st["w13_rows"] = ops.nvfp4_repack(weights["w13"], weights["w13_sf"], interleave=True)
        st["w2_q"], st["w2_s"], st["w2_rows"] = ops.nvfp4_repack(weights["w2"], weights["w2_sf"], interleave=False)
    st["w13_gs"] = weights["w13_gs"].float().contiguous()
    st["w2_gs"] = weights["w2_gs"].float().contiguous()
    st["shared"] = "shared_w13" in weights
    if st["shared"]:
        if st["pooled"]:
            raise MslError("a shared expert together with pooler/unpooler is not supported")
        st["shared_w13"] = ops.interleave_gate_up(weights["shared_w13"])
        st["shared_w2"] = weights["shared_w2"].contiguous()
    st["counts"] = torch.zeros(el, dtype=torch.int32, device=dev)     # zero between launches (the kernel re-zeroes)
    st["sync"] = torch.zeros(2, dtype=torch.int32, device=dev)        # grid-barrier words of the routing kernel
    st["offsets"] = torch.zeros(el + 1, dtype=torch.int32, device=dev)
    st["status"] = torch.zeros(1, dtype=torch.int32, device=dev)
    st["inv_freq"] = {}
    st["cap"] = 0
    st["side"] = torch.cuda.Stream(dev)
    torch.cuda.synchronize(dev)
    return st


def _scratch(st, tokens, top_k):
    """Slab buffers for `tokens * top_k` routes; grow-only, old buffers stay alive because graphs
    captured earlier still point into them."""
    rows = tokens * top_k
    if rows > st["cap"]:
        st.setdefault("retired", []).extend(st[k] for k in ("slab_x", "slab_i") if k in st)
        dev = st["device"]
        st["slab_x"] = torch.empty((rows, st["moe_width"]), dtype=torch.bfloat16, device=dev)   # x, later y
        st["slab_i"] = torch.empty((rows, st["inter"]), dtype=torch.bfloat16, device=dev)
        st["cap"] = rows
    return st["slab_x"][:rows], st["slab_i"][:rows]


def _inv_freq(st, theta, head_dim):
    key = (float(theta), head_dim)
    if key not in st["inv_freq"]:
        st["inv_freq"][key] = (1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32,
                                                             device=st["device"]) / head_dim))).contiguous()
    return st["inv_freq"][key]


def _mark(st, name):
    """Stage boundary for per-kernel timing: when st["marks"] is a list, record a CUDA event on the
    current stream after the launches of stage `name` (one event per stage; no synchronisation)."""
    marks = st.get("marks")
    if marks is not None:
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        marks.append((name, ev))


def stage_times_ms(marks):
    """[(stage, milliseconds)] from the events of one `kernel_fn` call (after a synchronise)."""
    return [(marks[i][0], marks[i - 1][1].elapsed_time(marks[i][1])) for i in range(1, len(marks))]


def attention_stage(data, st, after_store=None):
    """QKV+gate projection, QK-norm/RoPE/FP8/cache store, attention with the fused per-head norm
    and gate.  Returns bf16 [T, hq*head_dim].  `after_store()` runs between the cache store and the
    attention (the K/V hand-off of a sequence prefilled in chunks on several ranks)."""
    cfg = data["config"]
    hq, hkv, d = cfg["num_q_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    status = st["status"]
    _mark(st, "begin")
    qkv = ops.gemm(data["attn_input"], st["qkv_gate"], status=status)
    _mark(st, "gemm_qkv")
    inv_freq = _inv_freq(st, cfg["rope_theta"], d) if cfg["rope_theta"] else None
    q8 = ops.qk_rope_store(qkv, data["positions"], data["cache_loc"], inv_freq, data["k_scale"], data["v_scale"],
                           data["k_cache"], data["v_cache"], hq, hkv, d, status=status)
    _mark(st, "qk_rope_store")
    if after_store is not None:
        after_store()
        _mark(st, "kv_handoff")
    gate = qkv[:, (hq + 2 * hkv) * d:]
    out = ops.attention(q8, data["k_cache"], data["v_cache"], data["page_table"], data["seq_lens"],
                         data["cu_seqlens_q"], data["k_scale"], data["v_scale"],
                         cfg["sm_scale"] * cfg["qk_scale_factor"], cfg["batch"], cfg["q_len"], hq, hkv, d,
                         cfg["page_size"], cfg["window"], gate=gate, status=status)
    _mark(st, "attention")
    return out


def _router_logits(h, st):
    """Router logits as a BF16 hi + lo product with fp32 output (TASK.md:88 allows the split)."""
    hidden = h.shape[1]
    logits = ops.gemm(h, st["router_hilo"], out_mode=OUT_F32, k=hidden, segs=2, a_seg_stride=0, b_seg_stride=hidden,
                      status=st["status"])
    _mark(st, "gemm_router")
    return logits


def _shared_expert(h, st):
    s_inter = ops.gemm(h, st["shared_w13"], out_mode=OUT_SWIGLU_BF16, status=st["status"])
    shared = ops.gemm(s_inter, st["shared_w2"], status=st["status"])
    _mark(st, "shared_expert")
    return shared


def moe_stage(h, data, st, boundary_stream=None):
    """Router, dispatch, routed experts (+ shared expert), weighted combine, unpooler.
    h: bf16 [T, H], the FFN input.  Returns (FFN branch bf16 [T, H], expert ids i32 [T, K]).
    With `boundary_stream` (the fp32 residual stream entering the FFN boundary; layers without an
    unpooler only) the weighted combine and the FFN boundary run as one kernel and the first result
    is (stream_out fp32, hidden bf16) instead.

    The router product runs on a side stream next to the dense GEMM that does not depend on it
    (shared expert, or pooler), as the reference forks its router (submission.py:1105-1117); fork and
    join are stream waits, so the call stays capturable.  Top-k, slot assignment and dispatch are one
    kernel.  With per-stage timing marks enabled everything runs on one stream."""
    cfg = data["config"]
    top_k, status = cfg["top_k"], st["status"]
    tokens = h.shape[0]
    slab_x, slab_i = _scratch(st, tokens, top_k)
    overlap = st.get("marks") is None
    main = torch.cuda.current_stream()
    side = st["side"] if overlap else main

    def route_dispatch(x, norm_w, logits):
        out = ops.route_dispatch(logits, st["router_bias"], ROUTER_MULTIPLIER, data["local_start"], st["n_experts"],
                                 top_k, st["n_local"], x, norm_w, slab_x, st["offsets"], st["counts"], st["sync"],
                                 status)
        _mark(st, "route_dispatch")
        return out

    if overlap:
        side.wait_stream(main)
    with torch.cuda.stream(side):
        logits = _router_logits(h, st)
        if not st["pooled"]:
            ids, tw, rowmap = route_dispatch(h, None, logits)
    shared = None
    if st["pooled"]:
        p = ops.gemm(h, st["pooler"], status=status)
        _mark(st, "gemm_pooler")
    elif st["shared"]:
        shared = _shared_expert(h, st)
    if overlap:
        main.wait_stream(side)
        logits.record_stream(main)             # allocated on the side stream, read (or freed) on the main one
    if st["pooled"]:
        ids, tw, rowmap = route_dispatch(p, st["w_pre_exp"], logits)
    elif overlap:
        for t in (ids, tw, rowmap):
            t.record_stream(main)
    expert_gemms(slab_x, slab_i, st["offsets"], st)
    if boundary_stream is not None and not st["pooled"]:
        out = ops.combine_boundary(slab_x, rowmap, tw, st["w_post_exp"], shared, st["w_post_ffn"], boundary_stream,
                                   st["a2"], st["b2"], st["w_next"], POST_NORM_EPS, RMS_EPS, status)
        _mark(st, "combine_boundary_ffn")
        return out, ids
    moe = ops.combine(slab_x, rowmap, tw, st["w_post_exp"], addend=shared, status=status)
    _mark(st, "combine")
    if st["pooled"]:
        moe = unpool(moe, st)
        _mark(st, "gemm_unpooler")
    return moe, ids


def _lib_row_tiles(rows, groups):
    from . import _lib
    return _lib.lib().msl_nvfp4_bs_row_tiles(rows, groups)


def expert_gemms(slab_x, slab_i, offsets, st):
    """Gate/up projection with fused SiLU * up (slab_x -> slab_i), then the down projection (slab_i ->
    slab_x, in place of the inputs).  Default: NVFP4 weights x BF16 activations.  Opt-in
    (st["experts_nvfp4"]): each slab is first quantised to NVFP4 (4-bit codes, a UE4M3 scale per 16
    elements, an fp32 scale per row) and both products run on the block-scaled MMA."""
    status = st["status"]
    if st["experts_nvfp4"]:
        def quantised(key, slab):
            # buffers sized for the scratch capacity, grow-only like the slabs they mirror
            rows, k = slab.shape
            bufs = st.get(key)
            cap = max(st.get("cap", 0), rows)          # expert parallel: the slab is the caller's, not st's
            if bufs is None or bufs[0].shape[0] < cap or bufs[3] != offsets.numel():
                st.setdefault("retired", []).append(bufs)
                dev = st["device"]
                tiles = int(_lib_row_tiles(cap, offsets.numel() - 1))
                bufs = (torch.empty((cap, k // 2), dtype=torch.uint8, device=dev),
                        torch.zeros((tiles, k // 256, 4, 512), dtype=torch.uint8, device=dev),
                        torch.ones(cap, dtype=torch.float32, device=dev), offsets.numel())
                st[key] = bufs
            return ops.nvfp4_bs_quantize(slab, offsets, out=(bufs[0][:rows], bufs[1], bufs[2][:rows]))

        xq = quantised("quant_x", slab_x)
        _mark(st, "quantize_x")
        ops.grouped_gemm_nvfp4_bs(xq, st["w13_codes"], st["w13_sf_t"], st["w13_gs"], offsets, slab_i, st["inter"], True,
                                  status)
        _mark(st, "experts_gate_up")
        iq = quantised("quant_i", slab_i)
        _mark(st, "quantize_inter")
        ops.grouped_gemm_nvfp4_bs(iq, st["w2_codes"], st["w2_sf_t"], st["w2_gs"], offsets, slab_x, st["moe_width"],
                                  False, status)
        _mark(st, "experts_down")
        return
    ops.grouped_gemm_nvfp4(slab_x, st["w13_q"], st["w13_s"], st["w13_gs"], offsets, slab_i, st["inter"], True, status)
    _mark(st, "experts_gate_up")
    ops.grouped_gemm_nvfp4(slab_i, st["w2_q"], st["w2_s"], st["w2_gs"], offsets, slab_x, st["moe_width"], False,
                           status)
    _mark(st, "experts_down")


SLICED_MAX_TOKENS = 8          # reference.py:58


def unpool(moe, st):
    """MoE width back to the hidden size.  Up to 8 tokens (decode steps, verify blocks) this GPU forms
    only its first hidden/8 columns and leaves the rest zero, as the reference does
    (reference.py:56-58,468-470: the all-gather it stands for is the identity there)."""
    tokens = moe.shape[0]
    if tokens > SLICED_MAX_TOKENS:
        return ops.gemm(moe, st["unpooler"], status=st["status"])
    hidden = st["unpooler"].shape[0]
    cols = hidden // 8
    f = torch.zeros((tokens, hidden), dtype=torch.bfloat16, device=moe.device)
    ops.gemm(moe, st["unpooler"][:cols], out=f[:, :cols], status=st["status"])
    return f


def kernel_fn(data: dict, st: dict):
    """(hidden bf16 [T, H], stream fp32 [T, H], expert ids int32 [T, K]); writes the new K/V rows
    into data["k_cache"] / data["v_cache"] in place."""
    o_in = attention_stage(data, st)
    a = ops.gemm(o_in, st["o"], status=st["status"])
    _mark(st, "gemm_o")
    s1, h = ops.boundary(a, None, data["stream"], st["a1"], st["b1"], st["w_pre_ffn"], POST_NORM_EPS, RMS_EPS)
    _mark(st, "boundary_attn")
    if not st["pooled"]:                       # combine and FFN boundary as one kernel
        (s2, hidden), ids = moe_stage(h, data, st, boundary_stream=s1)
        return hidden, s2, ids
    f, ids = moe_stage(h, data, st)
    s2, hidden = ops.boundary(f, st["w_post_ffn"], s1, st["a2"], st["b2"], st["w_next"], POST_NORM_EPS, RMS_EPS)
    _mark(st, "boundary_ffn")
    return hidden, s2, ids


def check_status(st: dict) -> None:
    """Read the device status word (synchronises; call outside any timed region) and raise if a
    kernel reported a timed-out wait or an overflowing buffer."""
    code = int(st["status"].item())
    if code:
        st["status"].zero_()
        what = {ERR_DEVICE_TIMEOUT: "a device-side wait ran out of time",
                ERR_CAPACITY: "a cache row or slab row was out of range"}.get(code, "unknown device error")
        raise MslError(f"device status {code}: {what}")
