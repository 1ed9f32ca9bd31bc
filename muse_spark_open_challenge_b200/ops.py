"""Thin torch-tensor wrappers over the C ABI (include/msl.h): one function per kernel.

torch supplies device memory and the current stream only; all arithmetic happens in libmsl.so.
Every wrapper validates dtypes/contiguity, launches on `torch.cuda.current_stream()` and raises
`MslError` on a non-zero status.  Nothing here synchronises.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import OUT_BF16, OUT_F32, OUT_SWIGLU_BF16, MslError, check

FP8 = torch.float8_e4m3fn
TILE_N = 256      # weight rows per tile of a re-tiled NVFP4 bank (kGN in csrc/grouped_nvfp4.cu)


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _need(t, dtype, name):
    if t.dtype != dtype or not t.is_cuda:
        raise MslError(f"{name}: expected a CUDA tensor of {dtype}, got {t.dtype} on {t.device}")


def _rows(t, name):
    """Row pitch (elements) of a 2-D tensor whose last dim is contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise MslError(f"{name}: expected a 2-D tensor with a contiguous last dim")
    return t.stride(0)


def gemm(a, w, out_mode=OUT_BF16, out=None, k=None, segs=1, a_seg_stride=0, b_seg_stride=0, alpha=1.0, status=None,
         splits=None):
    """out[m, n] = alpha * sum_s a[:, s*a_seg_stride : +k] @ w[:, s*b_seg_stride : +k].T (bf16 in,
    fp32 accumulate).  OUT_SWIGLU_BF16 expects w rows interleaved in 128-gate / 128-up blocks.
    Products with few output tiles and a long K run split over K (`splits`; None lets the library
    choose from the sizes)."""
    _need(a, torch.bfloat16, "a"), _need(w, torch.bfloat16, "w")
    m, n = a.shape[0], w.shape[0]
    k = a.shape[1] if k is None else k
    n_out = n // 2 if out_mode == OUT_SWIGLU_BF16 else n
    if out is None:
        out = torch.empty((m, n_out), dtype=torch.float32 if out_mode == OUT_F32 else torch.bfloat16, device=a.device)
    lib = _lib.lib()
    if splits is None:
        splits = int(lib.msl_gemm_splitk_plan(m, n, k, segs, out_mode)) if m > 0 else 1
    args = (a.data_ptr(), _rows(a, "a"), w.data_ptr(), _rows(w, "w"), out.data_ptr(), _rows(out, "out"), m, n, k, segs,
            a_seg_stride, b_seg_stride, out_mode, float(alpha))
    if splits > 1:
        work = torch.empty(splits * m * n, dtype=torch.float32, device=a.device)
        check(lib.msl_gemm_bf16_splitk(*args, splits, work.data_ptr(), _ptr(status), _stream()), "msl_gemm_bf16_splitk")
    else:
        check(lib.msl_gemm_bf16(*args, _ptr(status), _stream()), "msl_gemm_bf16")
    return out


def qk_rope_store(qkv, positions, cache_loc, inv_freq, k_scale, v_scale, k_cache, v_cache, hq, hkv, head_dim,
                  status=None):
    """Returns q8 [T, hq, head_dim] (E4M3) and writes the new K/V rows into the paged caches."""
    _need(qkv, torch.bfloat16, "qkv"), _need(positions, torch.int64, "positions")
    _need(cache_loc, torch.int64, "cache_loc"), _need(k_cache, FP8, "k_cache"), _need(v_cache, FP8, "v_cache")
    t = qkv.shape[0]
    q8 = torch.empty((t, hq, head_dim), dtype=FP8, device=qkv.device)
    cache_rows = k_cache.numel() // (hkv * head_dim)
    check(_lib.lib().msl_qk_rope_store(qkv.data_ptr(), _rows(qkv, "qkv"), positions.data_ptr(), cache_loc.data_ptr(),
                                       _ptr(inv_freq), k_scale.data_ptr(), v_scale.data_ptr(), q8.data_ptr(),
                                       k_cache.data_ptr(), v_cache.data_ptr(), t, hq, hkv, head_dim, cache_rows,
                                       _ptr(status), _stream()), "msl_qk_rope_store")
    return q8


def attention(q8, k_cache, v_cache, page_table, seq_lens, cu_seqlens_q, k_scale, v_scale, softmax_scale, batch,
              max_q_len, hq, hkv, head_dim, page_size, window, gate=None, out=None, status=None, kv_splits=None):
    """bf16 [T, hq*head_dim]; with `gate` (a bf16 2-D view with the same columns) the per-head RMS
    norm and sigmoid gate are applied in the epilogue.  When the query blocks are too few to fill the
    GPU (short blocks over long cached contexts) the keys are cut into `kv_splits` slices that run as
    separate CTAs and are merged afterwards; None lets the library choose from the sizes."""
    _need(q8, FP8, "q8"), _need(page_table, torch.int32, "page_table"), _need(seq_lens, torch.int32, "seq_lens")
    _need(cu_seqlens_q, torch.int32, "cu_seqlens_q")
    t = q8.shape[0]
    if out is None:
        out = torch.empty((t, hq * head_dim), dtype=torch.bfloat16, device=q8.device)
    cache_rows = k_cache.numel() // (hkv * head_dim)
    lib = _lib.lib()
    if kv_splits is None:
        kv_splits = int(lib.msl_attention_split_plan(batch, max_q_len, hq, hkv, page_table.shape[1], page_size, window))
    args = (q8.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_table.data_ptr(), page_table.shape[1],
            seq_lens.data_ptr(), cu_seqlens_q.data_ptr(), k_scale.data_ptr(), v_scale.data_ptr(), float(softmax_scale),
            batch, max_q_len, t, hq, hkv, head_dim, page_size, window, cache_rows, out.data_ptr(), _rows(out, "out"),
            _ptr(gate), 0 if gate is None else _rows(gate, "gate"))
    if kv_splits > 1:
        work = torch.empty(int(lib.msl_attention_split_workspace(kv_splits, t, hq, head_dim)) // 4, dtype=torch.float32,
                           device=q8.device)
        check(lib.msl_attention_fp8_split(*args, kv_splits, work.data_ptr(), _ptr(status), _stream()),
              "msl_attention_fp8_split")
    else:
        check(lib.msl_attention_fp8(*args, _ptr(status), _stream()), "msl_attention_fp8")
    return out


def boundary(branch, branch_scale, stream_in, alpha, beta, norm_w, eps_branch=1e-8, eps_out=1e-5):
    """(stream_out fp32 [T, H], hidden bf16 [T, H])."""
    _need(branch, torch.bfloat16, "branch"), _need(stream_in, torch.float32, "stream_in")
    t, h = stream_in.shape
    s_out = torch.empty_like(stream_in)
    hid = torch.empty((t, h), dtype=torch.bfloat16, device=branch.device)
    check(_lib.lib().msl_boundary(branch.data_ptr(), _rows(branch, "branch"), _ptr(branch_scale), stream_in.data_ptr(),
                                  alpha.data_ptr(), beta.data_ptr(), norm_w.data_ptr(), s_out.data_ptr(),
                                  hid.data_ptr(), h, t, h, float(eps_branch), float(eps_out), _stream()),
          "msl_boundary")
    return s_out, hid


def route_topk(logits, bias, multiplier, local_start, n_experts, top_k, n_local, counts, hilo=False):
    """(ids i32 [T,K], weights f32 [T,K], local_ids i32 [T,K], slots i32 [T,K]); `counts` (i32
    [n_local], zeroed by the caller) receives the per-expert route counts."""
    _need(logits, torch.float32, "logits"), _need(bias, torch.float32, "bias"), _need(counts, torch.int32, "counts")
    _need(local_start, torch.int32, "local_start")
    t, dev = logits.shape[0], logits.device
    ids = torch.empty((t, top_k), dtype=torch.int32, device=dev)
    weights = torch.empty((t, top_k), dtype=torch.float32, device=dev)
    local_ids = torch.empty((t, top_k), dtype=torch.int32, device=dev)
    slots = torch.empty((t, top_k), dtype=torch.int32, device=dev)
    check(_lib.lib().msl_route_topk(logits.data_ptr(), _rows(logits, "logits"), int(hilo), bias.data_ptr(),
                                    float(multiplier), local_start.data_ptr(), t, n_experts, top_k, n_local,
                                    ids.data_ptr(), weights.data_ptr(), local_ids.data_ptr(), slots.data_ptr(),
                                    counts.data_ptr(), _stream()), "msl_route_topk")
    return ids, weights, local_ids, slots


def dispatch(x, norm_w, local_ids, slots, counts, slab, offsets, status=None):
    """Fills `slab` [rows, width] and `offsets` [n_local + 1]; returns rowmap i32 [T, K]."""
    _need(x, torch.bfloat16, "x"), _need(slab, torch.bfloat16, "slab"), _need(offsets, torch.int32, "offsets")
    t, top_k = local_ids.shape
    rowmap = torch.empty((t, top_k), dtype=torch.int32, device=x.device)
    check(_lib.lib().msl_dispatch(x.data_ptr(), _rows(x, "x"), _ptr(norm_w), local_ids.data_ptr(), slots.data_ptr(),
                                  counts.data_ptr(), t, counts.numel(), top_k, slab.shape[1], slab.data_ptr(),
                                  slab.shape[0], rowmap.data_ptr(), offsets.data_ptr(), _ptr(status), _stream()),
          "msl_dispatch")
    return rowmap


def route_dispatch(logits, bias, multiplier, local_start, n_experts, top_k, n_local, x, norm_w, slab, offsets, counts,
                   sync, status=None, hilo=False):
    """`route_topk` and `dispatch` as one launch.  Returns (ids, weights, rowmap); fills `slab` and
    `offsets`.  `counts` i32 [n_local] and `sync` i32 [2] must be zero on entry and are zero again when
    the kernel ends (the counts of the call are the differences of `offsets`)."""
    _need(logits, torch.float32, "logits"), _need(bias, torch.float32, "bias"), _need(counts, torch.int32, "counts")
    _need(local_start, torch.int32, "local_start"), _need(x, torch.bfloat16, "x"), _need(slab, torch.bfloat16, "slab")
    _need(offsets, torch.int32, "offsets"), _need(sync, torch.int32, "sync")
    t, dev = logits.shape[0], logits.device
    ids = torch.empty((t, top_k), dtype=torch.int32, device=dev)
    weights = torch.empty((t, top_k), dtype=torch.float32, device=dev)
    scratch = torch.empty((2, t, top_k), dtype=torch.int32, device=dev)          # local ids, slots
    rowmap = torch.empty((t, top_k), dtype=torch.int32, device=dev)
    check(_lib.lib().msl_route_dispatch(logits.data_ptr(), _rows(logits, "logits"), int(hilo), bias.data_ptr(),
                                        float(multiplier), local_start.data_ptr(), x.data_ptr(), _rows(x, "x"),
                                        _ptr(norm_w), t, n_experts, top_k, n_local, slab.shape[1], ids.data_ptr(),
                                        weights.data_ptr(), scratch[0].data_ptr(), scratch[1].data_ptr(),
                                        counts.data_ptr(), sync.data_ptr(), slab.data_ptr(), slab.shape[0],
                                        rowmap.data_ptr(), offsets.data_ptr(), _ptr(status), _stream()),
          "msl_route_dispatch")
    return ids, weights, rowmap


def combine(y, rowmap, weights, post_w, addend=None, out=None, status=None):
    """bf16 [T, width] = sum_j w_j * rms(y[rowmap_j] * post_w, 1e-8) (+ addend)."""
    _need(y, torch.bfloat16, "y"), _need(rowmap, torch.int32, "rowmap"), _need(weights, torch.float32, "weights")
    t, top_k = rowmap.shape
    width = y.shape[1]
    if out is None:
        out = torch.empty((t, width), dtype=torch.bfloat16, device=y.device)
    check(_lib.lib().msl_combine(y.data_ptr(), rowmap.data_ptr(), weights.data_ptr(), post_w.data_ptr(), _ptr(addend),
                                 0 if addend is None else _rows(addend, "addend"), out.data_ptr(), _rows(out, "out"),
                                 t, top_k, width, _ptr(status), _stream()), "msl_combine")
    return out


def combine_boundary(y, rowmap, weights, post_w, addend, branch_scale, stream_in, alpha, beta, norm_w,
                     eps_branch=1e-8, eps_out=1e-5, status=None):
    """`combine` followed by `boundary` in one kernel (the combined row never leaves the registers).
    Returns (stream_out fp32 [T, H], hidden bf16 [T, H]); y's width must be the hidden size."""
    _need(y, torch.bfloat16, "y"), _need(rowmap, torch.int32, "rowmap"), _need(weights, torch.float32, "weights")
    _need(stream_in, torch.float32, "stream_in")
    t, top_k = rowmap.shape
    width = y.shape[1]
    if stream_in.shape != (t, width) or not stream_in.is_contiguous():
        raise MslError("combine_boundary: stream_in must be a contiguous [tokens, width] tensor")
    s_out = torch.empty_like(stream_in)
    hid = torch.empty((t, width), dtype=torch.bfloat16, device=y.device)
    check(_lib.lib().msl_combine_boundary(y.data_ptr(), rowmap.data_ptr(), weights.data_ptr(), post_w.data_ptr(),
                                          _ptr(addend), 0 if addend is None else _rows(addend, "addend"), t, top_k,
                                          width, _ptr(branch_scale), stream_in.data_ptr(), alpha.data_ptr(),
                                          beta.data_ptr(), norm_w.data_ptr(), s_out.data_ptr(), hid.data_ptr(), width,
                                          float(eps_branch), float(eps_out), _ptr(status), _stream()),
          "msl_combine_boundary")
    return s_out, hid


def ep_plan(counts_all, rank, cap, dest_base, group_offsets, status):
    """Row bases in the owners' slabs and this rank's (source, expert) group ranges from the
    all-gathered route counts i32 [world, E]."""
    _need(counts_all, torch.int32, "counts_all")
    world, e = counts_all.shape
    check(_lib.lib().msl_ep_plan(counts_all.data_ptr(), world, e // world, rank, cap, dest_base.data_ptr(),
                                 group_offsets.data_ptr(), _ptr(status), _stream()), "msl_ep_plan")


def peer_barrier(flag_bases, rank, world, status, timeout_ms=20000):
    """Barrier over the ranks on the current stream (flag_bases: device array of flag-word pointers)."""
    check(_lib.lib().msl_peer_barrier(int(flag_bases), rank, world, timeout_ms, _ptr(status), _stream()),
          "msl_peer_barrier")


def dispatch_peer(x, norm_w, ids, slots, dest_base, peer_bases, local_experts, cap, rowmap=None):
    """Token rows written straight into the owning ranks' slabs (peer_bases: device array of slab
    pointers, one per rank)."""
    _need(x, torch.bfloat16, "x"), _need(ids, torch.int32, "ids"), _need(slots, torch.int32, "slots")
    t, top_k = ids.shape
    if rowmap is None:
        rowmap = torch.empty((t, top_k), dtype=torch.int32, device=x.device)
    check(_lib.lib().msl_dispatch_peer(x.data_ptr(), _rows(x, "x"), _ptr(norm_w), ids.data_ptr(), slots.data_ptr(),
                                       dest_base.data_ptr(), int(peer_bases), local_experts, cap, t, top_k,
                                       x.shape[1], rowmap.data_ptr(), _stream()),
          "msl_dispatch_peer")
    return rowmap


def combine_peer(peer_bases, cap, width, rowmap, weights, post_w, addend=None, out=None):
    """`combine` with the expert outputs read from the owning ranks' slabs."""
    _need(rowmap, torch.int32, "rowmap"), _need(weights, torch.float32, "weights")
    t, top_k = rowmap.shape
    if out is None:
        out = torch.empty((t, width), dtype=torch.bfloat16, device=rowmap.device)
    check(_lib.lib().msl_combine_peer(int(peer_bases), cap, rowmap.data_ptr(), weights.data_ptr(), post_w.data_ptr(),
                                      _ptr(addend), 0 if addend is None else _rows(addend, "addend"), out.data_ptr(),
                                      _rows(out, "out"), t, top_k, width, _stream()), "msl_combine_peer")
    return out


def kv_rows_copy(src, dst, n, src_idx=None, dst_idx=None, status=None):
    """dst[dst_idx[i] or i] = src[src_idx[i] or i] for i < n; src and dst are 2-D byte-addressable
    row tensors with the same row size (a multiple of 16 bytes), indices int64."""
    row_bytes = src.shape[-1] * src.element_size()
    if dst.shape[-1] * dst.element_size() != row_bytes or not src.is_contiguous() or not dst.is_contiguous():
        raise MslError("kv_rows_copy: contiguous row tensors with equal row sizes are required")
    for idx in (src_idx, dst_idx):
        if idx is not None:
            _need(idx, torch.int64, "index")
    check(_lib.lib().msl_kv_rows_copy(src.data_ptr(), _ptr(src_idx), src.shape[0], dst.data_ptr(), _ptr(dst_idx),
                                      dst.shape[0], n, row_bytes, _ptr(status), _stream()), "msl_kv_rows_copy")


def nvfp4_repack(codes, scales, interleave):
    """Re-tile an NVFP4 bank (codes u8 [E, rows, k/2], scales e4m3 [E, rows, k/16]) for the grouped
    GEMM.  Returns (tiled codes u8, tiled scales u8, padded rows)."""
    e, rows, half_k = codes.shape
    k = 2 * half_k
    n_pad = int(_lib.lib().msl_nvfp4_padded_rows(rows, int(interleave)))
    codes = codes.contiguous().view(torch.uint8)
    scales = scales.contiguous().view(torch.uint8)
    out_q = torch.empty((e, n_pad // TILE_N, k // 64, TILE_N, 32), dtype=torch.uint8, device=codes.device)
    out_s = torch.empty((e, n_pad // TILE_N, k // 64, TILE_N, 4), dtype=torch.uint8, device=codes.device)
    check(_lib.lib().msl_nvfp4_repack(codes.data_ptr(), scales.data_ptr(), out_q.data_ptr(), out_s.data_ptr(), e, rows,
                                      k, int(interleave), _stream()), "msl_nvfp4_repack")
    return out_q, out_s, n_pad


def grouped_gemm_nvfp4(x, codes_t, scales_t, global_scales, offsets, out, n_out, swiglu, status=None):
    """out[r] = gs[e] * x[r] @ dq(W_e).T over each row group's slab range (fused SiLU*up when swiglu).
    `offsets` has one more entry than there are row groups; group g uses weight bank g % E."""
    _need(x, torch.bfloat16, "x"), _need(out, torch.bfloat16, "out"), _need(offsets, torch.int32, "offsets")
    _need(global_scales, torch.float32, "global_scales")
    e, n_tiles, k_blocks = codes_t.shape[:3]
    if not x.is_contiguous():
        raise MslError("x must be contiguous")
    check(_lib.lib().msl_grouped_gemm_nvfp4(x.data_ptr(), x.shape[0], codes_t.data_ptr(), scales_t.data_ptr(),
                                            global_scales.data_ptr(), offsets.data_ptr(), out.data_ptr(),
                                            _rows(out, "out"), offsets.numel() - 1, e, n_tiles * TILE_N, k_blocks * 64,
                                            n_out, int(swiglu),
                                            _ptr(status), _stream()), "msl_grouped_gemm_nvfp4")
    return out


# ---- opt-in expert mode: NVFP4 activations on the block-scaled tensor-core path
def nvfp4_bs_sf_repack(scales, swiglu):
    """Re-tile a bank's e4m3 block scales [E, rows, k/16] for `grouped_gemm_nvfp4_bs` (load time)."""
    e, rows, k16 = scales.shape
    k = 16 * k16
    tiles = int(_lib.lib().msl_nvfp4_bs_tiles(rows, int(swiglu)))
    out = torch.empty((e, tiles, k // 256, 4, 2, 512), dtype=torch.uint8, device=scales.device)
    check(_lib.lib().msl_nvfp4_bs_sf_repack(scales.contiguous().view(torch.uint8).data_ptr(), out.data_ptr(), e, rows,
                                            k, int(swiglu), _stream()), "msl_nvfp4_bs_sf_repack")
    return out


def nvfp4_bs_quantize(x, offsets, out=None):
    """Rows [0, offsets[-1]) of x (bf16 [rows, k]) -> (codes u8 [rows, k/2], block scales in the GEMM's
    tile layout, row scales fp32 [rows]).  `out` reuses a previous result's buffers."""
    _need(x, torch.bfloat16, "x"), _need(offsets, torch.int32, "offsets")
    rows, k = x.shape
    groups = offsets.numel() - 1
    if out is None:
        row_tiles = int(_lib.lib().msl_nvfp4_bs_row_tiles(rows, groups))
        out = (torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device),
               torch.zeros((row_tiles, k // 256, 4, 512), dtype=torch.uint8, device=x.device),
               torch.ones(rows, dtype=torch.float32, device=x.device))
    codes, scales, row_scales = out
    check(_lib.lib().msl_nvfp4_bs_quantize(x.data_ptr(), _rows(x, "x"), rows, k, offsets.data_ptr(), groups,
                                           codes.data_ptr(), scales.data_ptr(), row_scales.data_ptr(), _stream()),
          "msl_nvfp4_bs_quantize")
    return out


def grouped_gemm_nvfp4_bs(xq, w_codes, w_scales_tiled, global_scales, offsets, out, n_out, swiglu, status=None):
    """`grouped_gemm_nvfp4` with 4-bit activations: xq = (codes, block scales, row scales) from
    `nvfp4_bs_quantize`; w_codes u8 [E, rows, k/2] as the reference stores them."""
    codes, scales, row_scales = xq
    _need(out, torch.bfloat16, "out"), _need(offsets, torch.int32, "offsets")
    e, rows, half_k = w_codes.shape
    if not w_codes.is_contiguous():
        raise MslError("w_codes must be contiguous")
    check(_lib.lib().msl_grouped_gemm_nvfp4_bs(codes.data_ptr(), scales.data_ptr(), row_scales.data_ptr(),
                                               codes.shape[0], w_codes.data_ptr(), w_scales_tiled.data_ptr(),
                                               global_scales.data_ptr(), offsets.data_ptr(), out.data_ptr(),
                                               _rows(out, "out"), offsets.numel() - 1, e, rows, 2 * half_k, n_out,
                                               int(swiglu), _ptr(status), _stream()), "msl_grouped_gemm_nvfp4_bs")
    return out


def interleave_gate_up(w13: torch.Tensor) -> torch.Tensor:
    """Reorder a [2*I, K] gate-then-up matrix into blocks of 128 gate rows followed by their 128
    up rows, the row order OUT_SWIGLU_BF16 expects.  I must be a multiple of 128."""
    two_i, k = w13.shape
    inter = two_i // 2
    if inter % 128:
        raise MslError("the SwiGLU epilogue needs an intermediate size that is a multiple of 128")
    g = w13[:inter].view(inter // 128, 128, k)
    u = w13[inter:].view(inter // 128, 128, k)
    return torch.stack([g, u], dim=1).reshape(two_i, k).contiguous()
