"""The opt-in expert mode with NVFP4 activations on the block-scaled tensor-core path
(tcgen05.mma kind::mxf4nvf4): the quantiser against the oracle's restatement of the reference's
quantiser, the grouped GEMM against an fp32 product of the SAME quantised operands (the kernel's
arithmetic, free of quantisation noise), its error against the W4A16 result it approximates
(reported, with loose bounds), and the whole layer in this mode."""
import dataclasses
import math

import pytest
import torch

from conftest import to_device
from oracle import layer_ref as L

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn
GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


@pytest.fixture(scope="module")
def ops():
    from muse_spark_open_challenge_b200 import ops as o
    return o


def _decode(codes, k):
    """u8 [rows, k/2] -> e2m1 values fp32 [rows, k] (element 2i in the low nibble)."""
    c = torch.stack((codes & 0xF, codes >> 4), dim=-1).flatten(-2).long().cpu()
    v = GRID[c & 7]
    return torch.where((c & 8) != 0, -v, v)


def _scales_of(sf_tiled, offsets, rows, k):
    """The quantiser's tiled scale bytes back as fp32 [rows, k/16]."""
    offs = offsets.cpu().tolist()
    sf = sf_tiled.cpu()
    out = torch.zeros((rows, k // 16))
    tile0 = 0
    for g in range(len(offs) - 1):
        n = offs[g + 1] - offs[g]
        for i in range(n):
            tile, rt = tile0 + i // 128, i % 128
            for b in range(k // 16):
                step = b // 4
                byte = sf[tile, step // 4, step % 4, (rt % 32) * 16 + (rt // 32) * 4 + b % 4]
                out[offs[g] + i, b] = float(torch.tensor([int(byte)], dtype=torch.uint8).view(FP8).float())
        tile0 += (n + 127) // 128
    return out


def test_quantiser_matches_the_reference_rule(ops):
    g = torch.Generator(device="cuda").manual_seed(1)
    counts = [5, 0, 130, 64, 257]
    rows, k = sum(counts) + 3, 512                                   # three slab rows beyond the last group
    x = (torch.randn((rows, k), generator=g, device="cuda") * torch.exp(torch.randn((rows, 1), generator=g, device="cuda"))
         ).to(torch.bfloat16)
    x[7] = 0                                                         # an all-zero row
    x[9, 16:32] = 0                                                  # an all-zero block
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    codes, sf_t, rs = ops.nvfp4_bs_quantize(x, offsets)
    torch.cuda.synchronize()
    used = sum(counts)
    want_v, want_sf, want_rs = L.nvfp4_quantize_rows(x[:used].cpu())
    assert torch.equal(rs[:used].cpu(), want_rs)                     # fp32 row scales: the same expression
    got_sf = _scales_of(sf_t, offsets, used, k)
    assert torch.equal(got_sf, want_sf)                              # block scale bytes bit-exact
    got_v = _decode(codes[:used], k)
    differs = got_v != want_v
    # The only admissible differences sit at a mid-point between two grid values (to within the last
    # bit of x / scale, which the kernel forms as x * (1 / scale)): the hardware conversion rounds an exact
    # tie to the even code (0.75 -> 1, 1.75 -> 2, 3.5 -> 4), the reference's bucketize to the lower magnitude
    # (nvfp4.py:52-53).  With bf16 inputs and a block scale set by the block's own largest element such
    # ties do occur (about one element in a thousand); the two results are then neighbours on the grid.
    scale = (want_sf * want_rs[:, None]).repeat_interleave(16, dim=1)
    q = (x[:used].float().cpu() / scale)[differs].abs()
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    nearest = mids[(q[:, None] - mids[None, :]).abs().argmin(dim=1)]
    assert bool(((q - nearest).abs() <= 4e-7 * nearest).all())
    assert float((got_v - want_v).abs().max()) <= 2.0 and float(differs.float().mean()) < 5e-3
    both = torch.stack((got_v[differs].abs(), want_v[differs].abs()), dim=1).sort(dim=1).values
    idx = torch.bucketize(both, GRID)
    assert bool((idx[:, 1] - idx[:, 0] == 1).all())                  # neighbours on the grid


@pytest.mark.parametrize("counts,n,k,swiglu", [
    ([0, 1, 7, 128, 129, 300, 0, 5], 512, 256, True),
    ([0, 1, 7, 128, 129, 300, 0, 5], 256, 512, False),
    ([255, 256, 257, 0, 511, 513, 1, 900], 1024, 1024, False),
    ([2000, 800, 0, 3], 3072, 1024, True),
    ([40, 9], 4096, 1536, False),
])
def test_block_scaled_gemm_matches_product_of_the_quantised_operands(ops, counts, n, k, swiglu):
    from muse_spark_open_challenge_b200 import synth
    g = torch.Generator(device="cuda").manual_seed(n + k)
    e = len(counts)
    w_codes = torch.randint(0, 256, (e, n, k // 2), dtype=torch.uint8, generator=g, device="cuda")
    w_sf = torch.exp2(7 + 0.4 * torch.randn((e, n, k // 16), generator=g, device="cuda")).clamp(8, 448).to(FP8)
    gs = (torch.exp(torch.randn((e,), generator=g, device="cuda")) / (300.0 * math.sqrt(k))).float()
    total = sum(counts)
    x = torch.randn((total + 5, k), generator=g, device="cuda").to(torch.bfloat16)
    offsets = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    xq = ops.nvfp4_bs_quantize(x, offsets)
    w_sf_t = ops.nvfp4_bs_sf_repack(w_sf, swiglu)
    n_out = n // 2 if swiglu else n
    out = torch.full((total + 5, n_out), 7.0, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.grouped_gemm_nvfp4_bs(xq, w_codes, w_sf_t, gs, offsets, out, n_out, swiglu, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    # what the kernel multiplies: the quantised activations, dequantised on the CPU
    xv = _decode(xq[0][:total], k).view(total, k // 16, 16)
    xs = _scales_of(xq[1], offsets, total, k) * xq[2][:total].cpu()[:, None]
    x_dq = (xv * xs[:, :, None]).view(total, k)
    at, worst_q, worst_w4a16 = 0, 0.0, 0.0
    for ex, c in enumerate(counts):
        if c == 0:
            continue
        w = L.nvfp4_dequantize(w_codes[ex].cpu(), w_sf[ex].cpu(), gs[ex].cpu())
        ref_q = x_dq[at:at + c] @ w.T
        ref_full = x[at:at + c].float().cpu() @ w.T
        if swiglu:
            ref_q = torch.nn.functional.silu(ref_q[:, :n // 2]) * ref_q[:, n // 2:]
            ref_full = torch.nn.functional.silu(ref_full[:, :n // 2]) * ref_full[:, n // 2:]
        got = out[at:at + c].float().cpu()
        worst_q = max(worst_q, L.relative_l2(got, ref_q))
        worst_w4a16 = max(worst_w4a16, L.relative_l2(got, ref_full))
        at += c
    print(f"rel-L2 vs the product of the quantised operands {worst_q:.2e}; vs the BF16-activation product {worst_w4a16:.2e}")
    assert worst_q < 4e-3, "the kernel does not compute the product of its own operands"
    assert worst_w4a16 < 0.2
    assert (out[total:] == 7.0).all()              # rows outside every group's range are never written


def test_layer_with_nvfp4_activations_reports_its_error():
    """The whole layer with the experts in this mode against the fp32 oracle: the routing is unchanged
    (bit-exact ids), the residual update carries the extra quantisation error, which is reported."""
    from muse_spark_open_challenge_b200 import layer, synth
    shape = dataclasses.replace(synth.MID, hidden=1024, hq=8, hkv=2, n_experts=16, local_experts=16, moe_width=1024,
                                inter=512, shared_inter=512)
    weights = synth.make_weights(shape, seed=5)
    data = synth.make_input(shape, [150, 77], [30, 0], seed=20, page=64, kv_scale=0.5)
    dev_w = to_device(weights, "cuda")
    base = layer.prepare(dev_w)
    fp4 = layer.prepare(dev_w, experts_nvfp4=True)
    h0, s0, i0 = layer.kernel_fn(to_device(data, "cuda"), base)
    h1, s1, i1 = layer.kernel_fn(to_device(data, "cuda"), fp4)
    h2, s2, i2 = layer.kernel_fn(to_device(data, "cuda"), fp4)
    torch.cuda.synchronize()
    layer.check_status(base), layer.check_status(fp4)
    assert torch.equal(i0, i1) and torch.equal(h1, h2) and torch.equal(s1, s2)
    front = L.ref_front(data, weights)
    ref_hidden, ref_stream = L.ref_back(front, weights, i1.cpu())
    a1, _ = L.residual_coefficients(weights["attn_residual_gate"])
    a2, _ = L.residual_coefficients(weights["ffn_residual_gate"])
    carried = a1 * a2 * data["stream"].float()
    for name, s, h in (("W4A16", s0, h0), ("NVFP4 activations", s1, h1)):
        upd = L.error_report(s.cpu() - carried, ref_stream - carried)
        hid = L.error_report(h.cpu(), ref_hidden)
        print(name, "update", upd, "hidden", hid)
    upd = L.error_report(s1.cpu() - carried, ref_stream - carried)
    assert upd["rel_l2"] < 0.25 and torch.isfinite(h1.float()).all()
