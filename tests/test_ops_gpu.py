"""Op-level parity on the GPU: every C-ABI kernel against the CPU oracle (or a plain fp32 torch
restatement of the same formula) on the same seeded inputs.  Integer outputs (expert ids, slots,
cache rows) must be identical; floating-point outputs carry the tolerance stated at each check."""
import math

import pytest
import torch

from conftest import GOLDEN_CASES, load_golden_case, to_device
from oracle import layer_ref as L

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn


@pytest.fixture(scope="module")
def ops():
    from muse_spark_open_challenge_b200 import ops as _ops
    return _ops


def rel_l2(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp(min=1e-12))


# ------------------------------------------------------------------------------ dense GEMM
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 512), (300, 1280, 512), (1, 256, 128), (777, 128, 256),
                                   (130, 16, 512), (4096, 4096, 1024), (2500, 10240, 512),
                                   (753, 8192, 1024)])      # 96 tiles of 256 rows, the last row tile ragged
def test_gemm_bf16_matches_fp32_matmul(ops, m, n, k):
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n)
    a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") / math.sqrt(k)).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = a.float() @ w.float().T
    out = ops.gemm(a, w, status=status)
    assert int(status.item()) == 0
    # bf16 output: each value within one bf16 rounding (2^-8 relative) of the fp32 product
    assert torch.allclose(out.float(), ref, rtol=2 ** -7, atol=2e-3)
    assert rel_l2(out, ref) < 3e-3
    out32 = ops.gemm(a, w, out_mode=ops.OUT_F32, status=status)
    assert torch.allclose(out32, ref, rtol=1e-4, atol=1e-4)
    assert int(status.item()) == 0


@pytest.mark.parametrize("m,n,k,segs,splits", [(753, 2304, 8192, 1, 2), (8, 2304, 4096, 1, 16), (100, 256, 2048, 2, 7),
                                               (24, 64, 1024, 1, 16), (300, 1280, 1024, 1, 3),
                                               (753, 2304, 8192, 1, 5), (753, 4096, 8192, 1, 3)])   # 256-row tiles
def test_gemm_split_k(ops, m, n, k, segs, splits):
    """K cut into slices on separate CTAs, summed in a fixed order: same bound as the one-pass product,
    repeatable bit for bit, for bf16 and fp32 outputs and for the two-segment (router) form."""
    g = torch.Generator(device="cuda").manual_seed(m + n + splits)
    a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, segs * k), generator=g, device="cuda") / math.sqrt(segs * k)).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = sum(a.float() @ w[:, s * k:(s + 1) * k].float().T for s in range(segs))
    kw = dict(k=k, segs=segs, a_seg_stride=0, b_seg_stride=k, status=status)
    out32 = ops.gemm(a, w, out_mode=ops.OUT_F32, splits=splits, **kw)
    again = ops.gemm(a, w, out_mode=ops.OUT_F32, splits=splits, **kw)
    one = ops.gemm(a, w, out_mode=ops.OUT_F32, splits=1, **kw)
    out16 = ops.gemm(a, w, splits=splits, alpha=0.5, **kw)
    assert int(status.item()) == 0
    assert torch.equal(out32, again)
    assert torch.allclose(out32, ref, rtol=1e-4, atol=1e-4) and torch.allclose(out32, one, rtol=1e-4, atol=1e-4)
    assert torch.allclose(out16.float(), 0.5 * ref, rtol=2 ** -7, atol=2e-3)


def test_gemm_split_k_plan(ops):
    from muse_spark_open_challenge_b200 import _lib
    plan = _lib.lib().msl_gemm_splitk_plan
    assert plan(16384, 10240, 4096, 1, 0) == 1                    # prefill-sized: tiles fill the GPU
    assert plan(753, 256, 8192, 2, 1) > 1                         # the router of a 753-token chunk
    assert plan(8, 2304, 8192, 1, 0) > 1                          # a decode step's QKV product
    assert plan(753, 256, 8192, 2, 2) == 1                        # no split-K with the SwiGLU epilogue


def test_gemm_two_segment_router_product(ops):
    """fp32 router as BF16 hi + lo: logits within 2e-5 of the fp64 product."""
    t, h, e = 500, 512, 16
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn((t, h), generator=g, device="cuda").to(torch.bfloat16)
    r = 0.045 * torch.randn((e, h), generator=g, device="cuda")
    hi = r.to(torch.bfloat16)
    lo = (r - hi.float()).to(torch.bfloat16)
    w = torch.cat([hi, lo], 1).contiguous()
    out = ops.gemm(x, w, out_mode=ops.OUT_F32, k=h, segs=2, a_seg_stride=0, b_seg_stride=h)
    ref = (x.double() @ r.double().T).float()
    assert torch.allclose(out, ref, atol=2e-5, rtol=1e-5)


def test_gemm_swiglu_epilogue(ops):
    m, inter, k = 300, 256, 512
    g = torch.Generator(device="cuda").manual_seed(9)
    a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w13 = (torch.randn((2 * inter, k), generator=g, device="cuda") / math.sqrt(k)).to(torch.bfloat16)
    out = ops.gemm(a, ops.interleave_gate_up(w13), out_mode=ops.OUT_SWIGLU_BF16)
    hh = a.float() @ w13.float().T
    ref = torch.nn.functional.silu(hh[:, :inter]) * hh[:, inter:]
    assert out.shape == (m, inter)
    assert rel_l2(out, ref) < 4e-3


# ------------------------------------------------------------------------------ QK norm / RoPE / cache store
@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_qk_rope_store_matches_reference_vectors(ops, name):
    """Given the same bf16 QKV rows, the FP8 bytes must equal the oracle's up to rounding ties
    caused by last-ulp differences in rsqrt / sincos: at most 1 E4M3 step, on < 0.5 % of values.
    Cache slots are exact (every new row lands where the reference puts it, nothing else moves)."""
    g, w = load_golden_case(name)
    data = to_device(g["data"], "cuda")
    cfg = data["config"]
    d = L.dims_of(w, cfg)
    qkv = (g["data"]["attn_input"].float() @ w["qkv_gate"].float().T).to(torch.bfloat16)
    q, k, v, _ = qkv.float().split([d.q_size, d.kv_size, d.kv_size, d.q_size], dim=-1)
    pos = L.token_positions(g["data"])
    qn, kn = L.rms(q.reshape(-1, d.hq, d.head_dim)), L.rms(k.reshape(-1, d.hkv, d.head_dim))
    if cfg["rope_theta"]:
        qn = L.rope_interleaved(qn, pos, cfg["rope_theta"], d.head_dim)
        kn = L.rope_interleaved(kn, pos, cfg["rope_theta"], d.head_dim)
    want_q = qn.to(FP8)
    want_k = L.quant_fp8(kn, g["data"]["k_scale"])
    want_v = L.quant_fp8(v.reshape(-1, d.hkv, d.head_dim), g["data"]["v_scale"])
    inv_freq = None
    if cfg["rope_theta"]:
        inv_freq = (1.0 / (cfg["rope_theta"] ** (torch.arange(0, d.head_dim, 2).float() / d.head_dim))).cuda()
    before_k = data["k_cache"].clone()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    q8 = ops.qk_rope_store(qkv.cuda(), data["positions"], data["cache_loc"], inv_freq, data["k_scale"],
                           data["v_scale"], data["k_cache"], data["v_cache"], d.hq, d.hkv, d.head_dim, status=status)
    assert int(status.item()) == 0
    slots = g["ref"]["slots"].cuda()
    got_k = data["k_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
    got_v = data["v_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
    for got, want in ((q8.cpu(), want_q), (got_k, want_k), (got_v, want_v)):
        gb, wb = got.view(torch.uint8), want.view(torch.uint8)
        differ = gb != wb
        assert differ.float().mean() < 5e-3
        # adjacent E4M3 codes of the same sign differ by exactly 1 in their byte
        assert ((gb.int() - wb.int()).abs()[differ] <= 1).all()
    # rows other than the new slots are untouched
    mask = torch.ones(before_k.view(-1, d.hkv, d.head_dim).shape[0], dtype=torch.bool, device="cuda")
    mask[slots] = False
    assert torch.equal(data["k_cache"].view(-1, d.hkv, d.head_dim)[mask].view(torch.uint8),
                       before_k.view(-1, d.hkv, d.head_dim)[mask].view(torch.uint8))


# ------------------------------------------------------------------------------ boundary
@pytest.mark.parametrize("t,h,scaled", [(37, 512, False), (64, 4096, True), (5, 8192, True), (3, 256, False)])
def test_boundary_matches_formula(ops, t, h, scaled):
    g = torch.Generator(device="cuda").manual_seed(h + t)
    branch = torch.randn((t, h), generator=g, device="cuda").to(torch.bfloat16)
    s_in = torch.randn((t, h), generator=g, device="cuda")
    gate = (0.3 * torch.randn((h,), generator=g, device="cuda")).to(torch.bfloat16)
    alpha, beta = L.residual_coefficients(gate)
    norm_w = 1.0 + 0.1 * torch.randn((h,), generator=g, device="cuda")
    bscale = (1.0 + 0.1 * torch.randn((h,), generator=g, device="cuda")) if scaled else None
    s_out, hid = ops.boundary(branch, bscale, s_in, alpha.contiguous(), beta.contiguous(), norm_w)
    b = branch.float() * (bscale if scaled else 1.0)
    ref_s = alpha * s_in + beta * L.rms(b, 1e-8)
    ref_h = L.rms(ref_s) * norm_w
    assert torch.allclose(s_out, ref_s, rtol=1e-5, atol=1e-5)       # fp32 arithmetic, different sum order
    assert torch.allclose(hid.float(), ref_h, rtol=2 ** -7, atol=1e-5)   # one bf16 rounding


# ------------------------------------------------------------------------------ routing
@pytest.mark.parametrize("t,e,k,n_local,start", [(256, 16, 4, 16, 0), (1000, 128, 8, 128, 0), (777, 256, 8, 32, 96),
                                                 (33, 256, 8, 32, 240), (4096, 128, 8, 128, 0)])
def test_route_topk_ids_exact_and_slots_unique(ops, t, e, k, n_local, start):
    g = torch.Generator(device="cuda").manual_seed(e + t)
    logits = 3.0 * torch.randn((t, e), generator=g, device="cuda")
    logits[0, :] = 0.25                  # exact ties everywhere: lowest indices must win
    bias = 0.1 * torch.randn((e,), generator=g, device="cuda")
    bias[1::2] = bias[0::2]              # more ties between neighbours on row 0
    counts = torch.zeros(n_local, dtype=torch.int32, device="cuda")
    ls = torch.tensor([start], dtype=torch.int32, device="cuda")
    ids, w, local_ids, slots = ops.route_topk(logits, bias, 0.1767766952966369, ls, e, k, n_local, counts)
    scores = torch.sigmoid(logits.double().cpu() * 0.1767766952966369).float()
    biased = scores + bias.cpu()
    want = L.topk_ids(biased, k)
    assert torch.equal(ids.cpu(), want)                        # bit-exact expert ids, order included
    want_w = L.route_weights(scores, want)
    assert torch.allclose(w.cpu(), want_w, rtol=1e-5, atol=1e-7)
    want_local = (want.long() - start) % e
    want_local = torch.where(want_local < n_local, want_local, torch.full_like(want_local, -1)).int()
    assert torch.equal(local_ids.cpu(), want_local)
    assert torch.equal(counts.cpu(), torch.bincount(want_local[want_local >= 0].long(), minlength=n_local).int())
    # every local route has a unique slot in [0, count) of its expert
    sl, li = slots.cpu(), local_ids.cpu()
    assert (sl[li < 0] == -1).all()
    for ex in range(n_local):
        s = sl[li == ex].sort().values
        assert torch.equal(s, torch.arange(len(s), dtype=torch.int32))


def test_route_topk_hilo_halves_are_added(ops):
    t, e, k = 100, 16, 4
    g = torch.Generator(device="cuda").manual_seed(3)
    hi = torch.randn((t, e), generator=g, device="cuda")
    lo = 1e-3 * torch.randn((t, e), generator=g, device="cuda")
    bias = torch.zeros(e, device="cuda")
    ls = torch.zeros(1, dtype=torch.int32, device="cuda")
    c1 = torch.zeros(e, dtype=torch.int32, device="cuda")
    c2 = torch.zeros(e, dtype=torch.int32, device="cuda")
    ids_a, w_a, _, _ = ops.route_topk(torch.cat([hi, lo], 1).contiguous(), bias, 1.0, ls, e, k, e, c1, hilo=True)
    ids_b, w_b, _, _ = ops.route_topk((hi + lo).contiguous(), bias, 1.0, ls, e, k, e, c2)
    assert torch.equal(ids_a, ids_b) and torch.equal(w_a, w_b)


# ------------------------------------------------------------------------------ dispatch + combine
@pytest.mark.parametrize("t,width,e,k,normed", [(200, 256, 16, 4, True), (513, 4096, 128, 8, False),
                                                (64, 512, 32, 8, True)])
def test_dispatch_then_combine_round_trip(ops, t, width, e, k, normed):
    g = torch.Generator(device="cuda").manual_seed(t)
    x = torch.randn((t, width), generator=g, device="cuda").to(torch.bfloat16)
    logits = torch.randn((t, 2 * e), generator=g, device="cuda")   # twice as many experts as are local
    bias = torch.zeros(2 * e, device="cuda")
    counts = torch.zeros(e, dtype=torch.int32, device="cuda")
    ls = torch.tensor([e // 2], dtype=torch.int32, device="cuda")
    ids, w, local_ids, slots = ops.route_topk(logits, bias, 1.0, ls, 2 * e, k, e, counts)
    slab = torch.full((t * k, width), float("nan"), dtype=torch.bfloat16, device="cuda")
    offsets = torch.zeros(e + 1, dtype=torch.int32, device="cuda")
    norm_w = (1.0 + 0.1 * torch.randn((width,), generator=g, device="cuda")) if normed else None
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rowmap = ops.dispatch(x, norm_w, local_ids, slots, counts, slab, offsets, status)
    assert int(status.item()) == 0
    assert torch.equal(offsets[1:].cpu(), torch.cumsum(counts.cpu(), 0).int()) and int(offsets[0]) == 0
    want_rows = (L.rms(x) * norm_w).to(torch.bfloat16) if normed else x
    rm, li = rowmap.cpu(), local_ids.cpu()
    assert ((rm >= 0) == (li >= 0)).all()
    live = rm >= 0
    assert len(torch.unique(rm[live])) == int(live.sum()) == int(counts.sum())   # a permutation of the live rows
    tok = torch.arange(t)[:, None].expand(t, k)[live]
    got = slab[rm[live].cuda().long()]
    if normed:
        assert torch.allclose(got.float(), want_rows[tok.cuda()].float(), rtol=2 ** -7, atol=1e-6)
    else:
        assert torch.equal(got.view(torch.int16), want_rows[tok.cuda()].view(torch.int16))   # a pure copy
    ex_of_row = torch.bucketize(rm[live], offsets[1:].cpu(), right=True)
    assert torch.equal(ex_of_row.int(), li[live])                    # each row lies in its expert's range
    # combine over the dispatched rows themselves (y = slab)
    post_w = 1.0 + 0.1 * torch.randn((width,), generator=g, device="cuda")
    add = torch.randn((t, width), generator=g, device="cuda").to(torch.bfloat16)
    out = ops.combine(slab, rowmap, w, post_w, addend=add, status=status)
    yy = L.post_expert_norm(want_rows.float(), post_w - 1.0)          # (1 + w) form of the oracle
    weight_sum = (w * (rowmap >= 0)).sum(-1, keepdim=True)
    ref = yy * weight_sum + add.float()
    assert torch.allclose(out.float(), ref, rtol=2 ** -6, atol=2e-2)
    assert rel_l2(out, ref) < 5e-3
    assert int(status.item()) == 0


@pytest.mark.parametrize("t,width,e,k,n_local,start,normed", [(200, 256, 16, 4, 16, 0, True),
                                                              (4100, 4096, 128, 8, 128, 0, False),
                                                              (777, 512, 256, 8, 32, 96, True),
                                                              (5, 512, 16, 4, 8, 12, False)])
def test_fused_route_dispatch_matches_the_two_kernels(ops, t, width, e, k, n_local, start, normed):
    """msl_route_dispatch (one cooperative launch) against msl_route_topk + msl_dispatch: ids and weights
    bit-exact, the same per-expert offsets, every route's slab row holds the same bytes and lies in its
    expert's range; the kernel leaves its counters and barrier words at zero, so a second call on other
    inputs (no memset in between) is right as well."""
    g = torch.Generator(device="cuda").manual_seed(t + e)
    ls = torch.tensor([start], dtype=torch.int32, device="cuda")
    counts1 = torch.zeros(n_local, dtype=torch.int32, device="cuda")
    sync = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for rep_i in range(2):
        logits = 2.0 * torch.randn((t, e), generator=g, device="cuda")
        bias = 0.1 * torch.randn((e,), generator=g, device="cuda")
        x = torch.randn((t, width), generator=g, device="cuda").to(torch.bfloat16)
        norm_w = (1.0 + 0.1 * torch.randn((width,), generator=g, device="cuda")) if normed else None
        counts0 = torch.zeros(n_local, dtype=torch.int32, device="cuda")
        ids0, w0, local_ids, slots = ops.route_topk(logits, bias, 0.5, ls, e, k, n_local, counts0)
        slab0 = torch.zeros((t * k, width), dtype=torch.bfloat16, device="cuda")
        off0 = torch.zeros(n_local + 1, dtype=torch.int32, device="cuda")
        rowmap0 = ops.dispatch(x, norm_w, local_ids, slots, counts0, slab0, off0, status)
        slab1 = torch.zeros_like(slab0)
        off1 = torch.zeros_like(off0)
        ids1, w1, rowmap1 = ops.route_dispatch(logits, bias, 0.5, ls, e, k, n_local, x, norm_w, slab1, off1, counts1,
                                               sync, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(ids0, ids1) and torch.equal(w0, w1)
        assert torch.equal(off0, off1)
        assert int(counts1.abs().sum()) == 0 and int(sync.abs().sum()) == 0       # left clean for the next call
        live = rowmap0 >= 0
        assert torch.equal(live, rowmap1 >= 0)
        assert torch.equal(slab0[rowmap0[live].long()].view(torch.int16), slab1[rowmap1[live].long()].view(torch.int16))
        rows = rowmap1[live].long()
        assert len(torch.unique(rows)) == rows.numel() == int(off1[-1])
        assert torch.equal(torch.bucketize(rows, off1[1:].long(), right=True).int(), local_ids[live])


@pytest.mark.parametrize("t,width,k", [(300, 4096, 8), (64, 512, 4), (33, 8192, 8)])
def test_fused_combine_boundary_matches_combine_then_boundary(ops, t, width, k):
    """One kernel against the two it replaces: bit-identical up to width 4096 (the same per-thread sums
    in the same order, the combined row rounded to bf16 in between as the unfused path stores it)."""
    g = torch.Generator(device="cuda").manual_seed(width + t)
    rows = t * k
    y = torch.randn((rows, width), generator=g, device="cuda").to(torch.bfloat16)
    rowmap = torch.randperm(rows, generator=g, device="cuda").int().view(t, k)
    rowmap[::5, 1] = -1                                               # routes without a row
    rowmap[3] = -1                                                    # a token with no local route at all
    w = torch.rand((t, k), generator=g, device="cuda")
    vec = lambda: 1.0 + 0.1 * torch.randn((width,), generator=g, device="cuda")   # noqa: E731
    post_w, branch_scale, norm_w = vec(), vec(), vec()
    alpha, beta = torch.rand((width,), generator=g, device="cuda"), torch.rand((width,), generator=g, device="cuda")
    add = torch.randn((t, width), generator=g, device="cuda").to(torch.bfloat16)
    s_in = torch.randn((t, width), generator=g, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    moe = ops.combine(y, rowmap, w, post_w, addend=add, status=status)
    s_want, h_want = ops.boundary(moe, branch_scale, s_in, alpha, beta, norm_w)
    s_got, h_got = ops.combine_boundary(y, rowmap, w, post_w, add, branch_scale, s_in, alpha, beta, norm_w,
                                        status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    if width <= 4096:
        assert torch.equal(s_got, s_want) and torch.equal(h_got.view(torch.int16), h_want.view(torch.int16))
    else:
        assert torch.allclose(s_got, s_want, rtol=1e-5, atol=1e-5) and rel_l2(h_got, h_want) < 2e-3


# ------------------------------------------------------------------------------ grouped NVFP4 GEMM
def _bank(e, rows, k, g, wide=False):
    codes = torch.randint(0, 256, (e, rows, k // 2), dtype=torch.uint8, generator=g, device="cuda")
    if wide:
        u = torch.rand((e, rows, k // 16), generator=g, device="cuda")
        sf = torch.exp2(-9 + u * 17.8).to(FP8)
    else:
        sf = torch.exp2(7 + 0.4 * torch.randn((e, rows, k // 16), generator=g, device="cuda")).clamp(8, 448).to(FP8)
    gs = (torch.exp(torch.randn((e,), generator=g, device="cuda")) / (300.0 * math.sqrt(k))).float()
    return codes, sf, gs


def test_grouped_dequant_is_exact_for_every_code_and_scale(ops):
    """One-hot activations read single weights back: out[r, n] = code value * block scale, exactly
    representable in bf16, for all 16 codes and every finite E4M3 scale byte (subnormals, zero and
    negative scales included)."""
    e, rows, k = 1, 256, 64
    codes = torch.zeros((e, rows, k // 2), dtype=torch.uint8)
    sf = torch.zeros((e, rows, k // 16), dtype=torch.uint8)
    for n in range(rows):
        for i in range(k // 2):
            lo, hi = (2 * i + n) % 16, (2 * i + 1 + 3 * n) % 16
            codes[0, n, i] = lo | (hi << 4)
        for b in range(k // 16):
            s = (n + 64 * b) % 256
            sf[0, n, b] = s if (s & 0x7F) != 0x7F else 0x38
    codes, sf = codes.cuda(), sf.cuda().view(FP8)
    gs = torch.ones(1, device="cuda")
    cq, cs, n_pad = ops.nvfp4_repack(codes, sf, interleave=False)
    x = torch.eye(k, dtype=torch.bfloat16, device="cuda")
    offsets = torch.tensor([0, k], dtype=torch.int32, device="cuda")
    out = torch.zeros((k, rows), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.grouped_gemm_nvfp4(x, cq, cs, gs, offsets, out, rows, False, status)
    assert int(status.item()) == 0
    want = L.nvfp4_dequantize(codes.cpu()[0], sf.cpu()[0], 1.0).T      # [k, rows]
    assert torch.equal(out.float().cpu(), want)


@pytest.mark.parametrize("counts,n,k,swiglu", [
    ([0, 1, 7, 128, 129, 300, 0, 5], 512, 256, True),
    ([0, 1, 7, 128, 129, 300, 0, 5], 256, 256, False),
    ([255, 256, 257, 0, 0, 16, 17, 15], 128, 128, False),
    ([2000, 800, 0, 3], 3072, 1024, True),
    ([255, 256, 257, 0, 511, 513, 1, 900], 512, 256, True),
    ([255, 256, 257, 0, 511, 513, 1, 900], 1024, 512, False),
])
@pytest.mark.parametrize("variant", ["narrow", "wide"])
def test_grouped_gemm_matches_dequantised_matmul(ops, counts, n, k, swiglu, variant):
    """rel-L2 per expert against x.float() @ dequantize(w).T (the check of the reference's
    tools/prefill/moe_kernel/test_moe_fp4.py:124-145; its kernels score about 1.7e-3)."""
    g = torch.Generator(device="cuda").manual_seed(n + k)
    e = len(counts)
    codes, sf, gs = _bank(e, n, k, g, wide=(k == 128))
    cq, cs, n_pad = ops.nvfp4_repack(codes, sf, interleave=swiglu)
    total = sum(counts)
    x = torch.randn((total + 5, k), generator=g, device="cuda").to(torch.bfloat16)   # 5 spare slab rows
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    n_out = n // 2 if swiglu else n
    out = torch.full((total + 5, n_out), 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    old = ops._lib.set_option("grouped_wide", variant == "wide")     # 128-row or (when the groups fill them) 256-row tiles
    try:
        ops.grouped_gemm_nvfp4(x, cq, cs, gs, offsets, out, n_out, swiglu, status)
    finally:
        ops._lib.set_option("grouped_wide", old)
    assert int(status.item()) == 0
    at = 0
    for ex, c in enumerate(counts):
        if c == 0:
            continue
        w = L.nvfp4_dequantize(codes[ex].cpu(), sf[ex].cpu(), gs[ex].cpu()).cuda()
        ref = x[at:at + c].float() @ w.T
        if swiglu:
            ref = torch.nn.functional.silu(ref[:, :n // 2]) * ref[:, n // 2:]
        assert rel_l2(out[at:at + c], ref) < 4e-3, f"expert {ex}"
        at += c
    assert (out[total:] == 7.0).all()              # rows outside every expert's range are never written


@pytest.mark.parametrize("variant", ["narrow", "wide"])
def test_grouped_gemm_never_stores_past_the_slab(ops, variant):
    """Offsets that run past the slab (what an expert-parallel plan could hand over when the routing
    needs more rows than the buffers hold) must not make the kernel store beyond it: the output
    buffer is longer than the slab it is declared with, and the rows behind the declared end stay as
    they were."""
    g = torch.Generator(device="cuda").manual_seed(3)
    n, k, e = 512, 256, 4
    codes, sf, gs = _bank(e, n, k, g)
    cq, cs, _ = ops.nvfp4_repack(codes, sf, interleave=False)
    slab_rows, guard = 1024, 512
    x_all = torch.randn((slab_rows + guard, k), generator=g, device="cuda").to(torch.bfloat16)
    out_all = torch.full((slab_rows + guard, n), 7.0, dtype=torch.bfloat16, device="cuda")
    # the groups claim 1400 rows of a 1024-row slab
    offsets = torch.tensor([0, 500, 900, 1300, 1400], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    old = ops._lib.set_option("grouped_wide", variant == "wide")
    try:
        ops.grouped_gemm_nvfp4(x_all[:slab_rows], cq, cs, gs, offsets, out_all[:slab_rows], n, False, status)
    finally:
        ops._lib.set_option("grouped_wide", old)
    torch.cuda.synchronize()
    assert (out_all[slab_rows:] == 7.0).all()
    w0 = L.nvfp4_dequantize(codes[0].cpu(), sf[0].cpu(), gs[0].cpu()).cuda()
    assert rel_l2(out_all[:500], x_all[:500].float() @ w0.T) < 4e-3           # the rows inside are still right


# ------------------------------------------------------------------------------ attention
def _attention_case(ops, shape, lens, ctxs, page, kv_scale, window, seed, zero_q=False, kv_splits=1):
    from muse_spark_open_challenge_b200 import synth
    import dataclasses
    shape = dataclasses.replace(shape, window=window)
    data = synth.make_input(shape, lens, ctxs, seed=seed, page=page, kv_scale=kv_scale)
    cfg = data["config"]
    d = L.Dims(shape.hidden, shape.hq, shape.hkv, shape.head_dim, 1, 1, 1, 1, 1, False, 0)
    t = cfg["tokens"]
    g = torch.Generator().manual_seed(seed + 1)
    q = torch.randn((t, shape.hq, shape.head_dim), generator=g)
    q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True))
    if zero_q:
        q = torch.zeros_like(q)
    q8 = q.to(FP8)
    k_new = (torch.randn((t, shape.hkv, shape.head_dim), generator=g) / kv_scale).to(FP8)
    v_new = (torch.randn((t, shape.hkv, shape.head_dim), generator=g) / kv_scale).to(FP8)
    ref = L.attend(q8.float() * cfg["qk_scale_factor"], k_new, v_new, data, d)          # fp32 [T, HQ, D]
    dev = to_device(data, "cuda")
    slots = L.new_slots(data).cuda()
    dev["k_cache"].view(-1, shape.hkv, shape.head_dim)[slots] = k_new.cuda()
    dev["v_cache"].view(-1, shape.hkv, shape.head_dim)[slots] = v_new.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.attention(q8.cuda(), dev["k_cache"], dev["v_cache"], dev["page_table"], dev["seq_lens"],
                        dev["cu_seqlens_q"], dev["k_scale"], dev["v_scale"], cfg["sm_scale"] * cfg["qk_scale_factor"],
                        cfg["batch"], cfg["q_len"], shape.hq, shape.hkv, shape.head_dim, page, window, status=status,
                        kv_splits=kv_splits)
    assert int(status.item()) == 0
    return out.float().cpu().view(t, shape.hq, shape.head_dim), ref


ATTN_CASES = [
    # (shape name, new lens, cached lens, page, kv_scale, window)
    ("MID", [256], [0], 64, 1.0, 0),
    ("MID", [100, 300, 33], [0, 77, 500], 64, 1 / 64, 0),
    ("MID", [200, 200], [300, 10], 16, 0.5, 128),
    ("MID", [130], [1000], 1, 1.0, 0),
    ("TINY", [256], [0], 64, 1.0, 0),
    ("TINY", [80, 80], [100, 100], 64, 1 / 64, 96),
    ("NATIVE", [300], [700], 1, 1.0, 0),
    ("NATIVE", [150, 97], [2500, 2400], 1, 1.0, 2048),
]


@pytest.mark.parametrize("case", ATTN_CASES)
def test_attention_matches_oracle(ops, case):
    """FP8 P (E4M3, 3 mantissa bits) bounds the accuracy: rel-L2 <= 3e-2 against the fp32 softmax
    over the same FP8 Q/K/V."""
    from muse_spark_open_challenge_b200 import synth
    name, lens, ctxs, page, kv_scale, window = case
    out, ref = _attention_case(ops, getattr(synth, name), lens, ctxs, page, kv_scale, window, seed=len(lens) + page)
    assert torch.isfinite(out).all()
    assert rel_l2(out, ref) < 3e-2


SPLIT_CASES = [
    # (shape name, new lens, cached lens, page, kv_scale, window, key slices)
    ("MID", [40], [3000], 64, 1 / 64, 0, 4),
    ("MID", [1, 1, 1], [2000, 5, 700], 64, 1.0, 0, 3),            # decode: some slices are empty
    ("MID", [100, 300, 33], [0, 77, 500], 16, 0.5, 0, 2),         # the gather path, ragged requests
    ("NATIVE", [97], [5000], 64, 1.0, 0, 7),
    ("NATIVE", [8, 8], [2500, 2400], 1, 1.0, 2048, 5),            # sliding window, verify blocks
    ("TINY", [80, 80], [100, 100], 64, 1 / 64, 96, 16),           # more slices than key tiles
]


@pytest.mark.parametrize("case", SPLIT_CASES)
def test_split_kv_attention_matches_oracle(ops, case):
    """The key range cut into slices that are merged afterwards: same bound as the single pass."""
    from muse_spark_open_challenge_b200 import synth
    name, lens, ctxs, page, kv_scale, window, splits = case
    out, ref = _attention_case(ops, getattr(synth, name), lens, ctxs, page, kv_scale, window, seed=splits + page,
                               kv_splits=splits)
    one, _ = _attention_case(ops, getattr(synth, name), lens, ctxs, page, kv_scale, window, seed=splits + page)
    assert torch.isfinite(out).all()
    assert rel_l2(out, ref) < 3e-2
    assert rel_l2(out, one) < 3e-2


def test_split_plan_slices_only_short_blocks_over_long_contexts(ops):
    from muse_spark_open_challenge_b200 import _lib
    plan = _lib.lib().msl_attention_split_plan
    assert plan(4, 4096, 32, 8, 64, 64, 0) == 1                   # mid prefill: thousands of CTAs already
    assert plan(1, 753, 16, 2, 1262, 64, 0) > 1                   # one short chunk after 80000 cached tokens
    assert plan(1, 1, 16, 2, 2, 64, 0) == 1                       # nothing to slice
    assert _lib.lib().msl_attention_split_workspace(3, 10, 16, 64) == 3 * 10 * 16 * 66 * 4


def test_attention_uniform_weights_average_the_values(ops):
    """Zero queries make every visible key weigh the same: the output is the running mean of the
    values, which isolates the P V product (orientation of V) from the Q K^T product."""
    from muse_spark_open_challenge_b200 import synth
    out, ref = _attention_case(ops, synth.MID, [200], [56], 64, 1.0, 0, seed=11, zero_q=True)
    assert rel_l2(out, ref) < 2e-2


def test_attention_fused_norm_and_gate(ops):
    from muse_spark_open_challenge_b200 import synth
    shape = synth.MID
    data = synth.make_input(shape, [150, 90], [40, 0], seed=2, page=64, kv_scale=1.0)
    cfg = data["config"]
    t = cfg["tokens"]
    g = torch.Generator().manual_seed(8)
    q8 = torch.randn((t, shape.hq, shape.head_dim), generator=g).to(FP8)
    gate = torch.randn((t, shape.q_size + 64), generator=g).to(torch.bfloat16)[:, 64:]    # a strided view
    dev = to_device(data, "cuda")
    plain = ops.attention(q8.cuda(), dev["k_cache"], dev["v_cache"], dev["page_table"], dev["seq_lens"],
                          dev["cu_seqlens_q"], dev["k_scale"], dev["v_scale"], 0.5, cfg["batch"], cfg["q_len"],
                          shape.hq, shape.hkv, shape.head_dim, 64, 0)
    gate_dev = gate.cuda()
    fused = ops.attention(q8.cuda(), dev["k_cache"], dev["v_cache"], dev["page_table"], dev["seq_lens"],
                          dev["cu_seqlens_q"], dev["k_scale"], dev["v_scale"], 0.5, cfg["batch"], cfg["q_len"],
                          shape.hq, shape.hkv, shape.head_dim, 64, 0, gate=gate_dev)
    ref = (L.rms(plain.float().view(t, shape.hq, shape.head_dim)).reshape(t, -1) * torch.sigmoid(gate_dev.float()))
    # the fused epilogue normalises the fp32 accumulator, the check normalises its bf16 rounding
    assert rel_l2(fused, ref) < 6e-3


# ------------------------------------------------------------------------------ multi-GPU plumbing on one GPU
def test_kv_rows_copy_gathers_scatters_and_reports_bad_rows(ops):
    g = torch.Generator(device="cuda").manual_seed(3)
    cache = torch.randint(0, 256, (500, 256), dtype=torch.uint8, generator=g, device="cuda")
    idx = torch.randperm(500, generator=g, device="cuda")[:123]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    packed = torch.zeros((200, 256), dtype=torch.uint8, device="cuda")
    ops.kv_rows_copy(cache, packed, 123, src_idx=idx, status=status)               # gather
    assert torch.equal(packed[:123], cache[idx]) and not packed[123:].any()
    other = torch.zeros_like(cache)
    where = torch.randperm(500, generator=g, device="cuda")[:123]
    ops.kv_rows_copy(packed, other, 123, dst_idx=where, status=status)             # scatter
    assert torch.equal(other[where], cache[idx]) and int(status.item()) == 0
    bad = where.clone()
    bad[5] = 500                                                                    # past the last row: skipped, reported
    before = other.clone()
    ops.kv_rows_copy(packed, other, 123, dst_idx=bad, status=status)
    assert int(status.item()) == ops._lib.ERR_CAPACITY
    assert torch.equal(other, before)


@pytest.mark.parametrize("world,local", [(4, 3), (8, 16), (2, 64)])
def test_ep_plan_places_every_rank_and_reports_overflow(ops, world, local):
    g = torch.Generator().manual_seed(1)
    counts = torch.randint(0, 50, (world, world * local), generator=g, dtype=torch.int32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    seen = {}
    for rank in range(world):
        dest = torch.zeros(world * local, dtype=torch.int32, device="cuda")
        offs = torch.zeros(world * local + 1, dtype=torch.int32, device="cuda")
        ops.ep_plan(counts.cuda(), rank, 10 ** 6, dest, offs, status)
        seen[rank] = (dest.cpu(), offs.cpu())
    assert int(status.item()) == 0
    for owner in range(world):
        # the owner's slab: groups ordered (source rank, local expert); sources write where the owner reads
        want, at = [], 0
        for src in range(world):
            for le in range(local):
                want.append(at)
                assert int(seen[src][0][owner * local + le]) == at, (owner, src, le)
                at += int(counts[src, owner * local + le])
        assert seen[owner][1].tolist() == want + [at]
    # a slab smaller than the rows routed to rank 0 is reported, and the row ranges stop at its end
    small = torch.zeros(world * local + 1, dtype=torch.int32, device="cuda")
    ops.ep_plan(counts.cuda(), 0, 8, torch.zeros(world * local, dtype=torch.int32, device="cuda"), small, status)
    assert int(status.item()) == ops._lib.ERR_CAPACITY
    small = small.cpu()
    assert int(small.max()) == 8 and int(small[-1]) == 8 and bool((small.diff() >= 0).all())
    assert small.tolist() == [min(v, 8) for v in seen[0][1].tolist()]


def test_peer_barrier_gives_up_when_a_rank_never_arrives(ops):
    """Two ranks' flag words on ONE GPU, only rank 0 runs: its wait for rank 1 runs out after the
    limit (50 ms here), the kernel sets the status word and returns, and the context stays usable.
    A second barrier with both ranks' kernels run one after the other cannot be tested on one GPU
    (kernels that wait on one another must not share a GPU), so rank 1's arrival is written by hand."""
    flags = torch.zeros((2, 3), dtype=torch.int32, device="cuda")          # [rank][world + 1]
    bases = torch.tensor([flags[0].data_ptr(), flags[1].data_ptr()], dtype=torch.int64, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.peer_barrier(bases.data_ptr(), 0, 2, status, timeout_ms=50)
    torch.cuda.synchronize()
    assert int(status.item()) == ops._lib.ERR_DEVICE_TIMEOUT
    assert flags[1, 0].item() == 1 and flags[0, 0].item() == 1             # rank 0 announced barrier 1 to both
    status.zero_()
    flags[0, 1] = 2                                                         # "rank 1" has already reached barrier 2
    ops.peer_barrier(bases.data_ptr(), 0, 2, status, timeout_ms=50)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and flags[0, 2].item() == 2
