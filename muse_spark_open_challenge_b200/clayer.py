"""The layer through the library's own C host (`msl_layer_prepare`, `msl_layer_prefill`) instead of the
Python launch sequence of `layer.py`: the binding a non-Python server would write, kept here so that the
C path is exercised by the same tests.  Same entry points as `layer`: `prepare(weights, config)` and
`kernel_fn(data, state)` (submission.py:1013, 1073); torch only provides the memory and the streams.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import MslError, check

_p, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float


def _struct(name, fields):
    return type(name, (C.Structure,), {"_fields_": fields})


# field order as in include/msl.h
Config = _struct("MslLayerConfig", [(n, _i) for n in (
    "tokens", "batch", "max_q_len", "hidden", "hq", "hkv", "head_dim", "n_experts", "n_local", "top_k", "moe_width",
    "inter", "pooled", "shared_inter", "page_size", "max_pages", "window")] + [("cache_rows", _i64),
                                                                                ("softmax_scale", _f), ("rope_theta", _f)])
RAW_FIELDS = ("qkv_gate", "o", "attn_residual_gate", "ffn_residual_gate", "pre_ffn_norm", "post_expert_norm",
              "post_ffn_norm", "next_pre_attn_norm", "pre_expert_norm", "pooler", "unpooler", "shared_w13", "shared_w2",
              "router", "router_bias", "w13", "w13_sf", "w2", "w2_sf", "w13_gs", "w2_gs")
RawWeights = _struct("MslLayerRawWeights", [(n, _p) for n in RAW_FIELDS])
PREPARED_FIELDS = ("qkv_gate", "o", "router_hilo", "pooler", "unpooler", "shared_w13", "shared_w2", "router_bias", "a1",
                   "b1", "a2", "b2", "w_pre_ffn", "w_post_exp", "w_post_ffn", "w_next", "w_pre_exp", "inv_freq", "w13_q",
                   "w13_s", "w2_q", "w2_s", "w13_gs", "w2_gs")
Weights = _struct("MslLayerWeights", [(n, _p) for n in PREPARED_FIELDS] + [("w13_rows", _i), ("w2_rows", _i)])
Inputs = _struct("MslLayerInputs", [(n, _p) for n in (
    "stream", "attn_input", "k_cache", "v_cache", "positions", "cache_loc", "seq_lens", "cu_seqlens_q", "page_table",
    "k_scale", "v_scale", "local_start")])
Outputs = _struct("MslLayerOutputs", [(n, _p) for n in ("hidden", "stream", "ids")])
Streams = _struct("MslLayerStreams", [(n, _p) for n in ("main", "side", "fork_event", "join_event")])


def make_config(weights: dict, cfg: dict, page_table: torch.Tensor, cache_rows: int) -> Config:
    """The C configuration of one call from the weight shapes and the call's `config` dict."""
    el, two_i, half_w = weights["w13"].shape
    c = Config()
    c.tokens, c.batch, c.max_q_len = cfg["tokens"], cfg["batch"], cfg["q_len"]
    c.hidden, c.hq, c.hkv, c.head_dim = weights["qkv_gate"].shape[1], cfg["num_q_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    c.n_experts, c.n_local, c.top_k = weights["router"].shape[0], el, cfg["top_k"]
    c.moe_width, c.inter = 2 * half_w, two_i // 2
    c.pooled = int("pooler" in weights)
    c.shared_inter = weights["shared_w13"].shape[0] // 2 if "shared_w13" in weights else 0
    c.page_size, c.max_pages, c.window = cfg["page_size"], page_table.shape[1], cfg["window"]
    c.cache_rows = cache_rows
    c.softmax_scale = cfg["sm_scale"] * cfg["qk_scale_factor"]
    c.rope_theta = float(cfg["rope_theta"] or 0.0)
    return c


def prepare(weights: dict, config: Config) -> dict:
    """`msl_layer_prepare` into one torch-owned buffer.  The raw weights stay referenced by the state."""
    dev = weights["qkv_gate"].device
    if dev.type != "cuda":
        raise MslError("prepare() needs CUDA tensors: this implementation has no CPU path")
    lib = _lib.lib()
    size = lib.msl_layer_prepared_bytes(C.byref(config))
    if size < 0:
        raise MslError("the layer configuration was rejected")
    keep = {k: v.contiguous() for k, v in weights.items()}
    raw = RawWeights()
    for name in RAW_FIELDS:
        setattr(raw, name, keep[name].data_ptr() if name in keep else None)
    buf = torch.empty(size, dtype=torch.uint8, device=dev)
    prepared = Weights()
    check(lib.msl_layer_prepare(C.byref(config), C.byref(raw), buf.data_ptr(), size, C.byref(prepared),
                                torch.cuda.current_stream().cuda_stream), "msl_layer_prepare")
    torch.cuda.synchronize(dev)
    return {"device": dev, "raw": keep, "buffer": buf, "weights": prepared, "side": torch.cuda.Stream(dev),
            "fork": torch.cuda.Event(), "join": torch.cuda.Event(), "workspace": None,
            "status": torch.zeros(1, dtype=torch.int32, device=dev)}


def kernel_fn(data: dict, st: dict, config: Config, fork: bool = True):
    """(hidden bf16 [T, H], stream fp32 [T, H], expert ids int32 [T, K]) through `msl_layer_prefill`."""
    lib = _lib.lib()
    dev = st["device"]
    need = lib.msl_layer_workspace_bytes(C.byref(config))
    if need < 0:
        raise MslError("the layer configuration was rejected")
    if st["workspace"] is None or st["workspace"].numel() < need:
        st["workspace"] = torch.empty(need, dtype=torch.uint8, device=dev)      # grow-only, like layer.py's slabs
    t = config.tokens
    hidden = torch.empty((t, config.hidden), dtype=torch.bfloat16, device=dev)
    stream = torch.empty((t, config.hidden), dtype=torch.float32, device=dev)
    ids = torch.empty((t, config.top_k), dtype=torch.int32, device=dev)
    ins = Inputs()
    for name in ("stream", "attn_input", "k_cache", "v_cache", "positions", "cache_loc", "seq_lens", "cu_seqlens_q",
                 "page_table", "k_scale", "v_scale", "local_start"):
        setattr(ins, name, data[name].data_ptr())
    outs = Outputs(hidden.data_ptr(), stream.data_ptr(), ids.data_ptr())
    main = torch.cuda.current_stream()
    if fork:
        # the events must exist as CUDA events before the library records them
        st["fork"].record(main)
        st["join"].record(st["side"])
        streams = Streams(main.cuda_stream, st["side"].cuda_stream, st["fork"].cuda_event, st["join"].cuda_event)
    else:
        streams = Streams(main.cuda_stream, None, None, None)
    check(lib.msl_layer_prefill(C.byref(config), C.byref(st["weights"]), C.byref(ins), C.byref(outs),
                                st["workspace"].data_ptr(), st["workspace"].numel(), C.byref(streams),
                                st["status"].data_ptr()), "msl_layer_prefill")
    return hidden, stream, ids
