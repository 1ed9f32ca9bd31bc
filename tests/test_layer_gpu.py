"""The whole layer through the reference's entry points (`prepare` / `kernel_fn`) on the GPU,
judged the way the reference judges a submission (routing check, residual update and next
attention input within the FP8-query-derived bounds, new cache rows within 8 %), first on the
reference-made golden vectors, then on seeded synthetic shapes against the CPU oracle."""
import dataclasses

import pytest
import torch

from conftest import GOLDEN_CASES, load_golden_case, to_device
from oracle import layer_ref as L

pytestmark = pytest.mark.gpu


def _run(data_cpu, weights_cpu):
    from muse_spark_open_challenge_b200 import layer
    w = to_device(weights_cpu, "cuda")
    st = layer.prepare({k: v.clone() for k, v in w.items()})
    data = to_device(data_cpu, "cuda")
    hidden, stream, ids = layer.kernel_fn(data, st)
    torch.cuda.synchronize()
    layer.check_status(st)
    d = L.dims_of(weights_cpu, data_cpu["config"])
    slots = L.new_slots(data_cpu).cuda()
    k_rows = data["k_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
    v_rows = data["v_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
    return hidden.cpu(), stream.cpu(), ids.cpu(), k_rows, v_rows, st, data


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_layer_on_reference_vectors(name):
    g, weights = load_golden_case(name)
    hidden, stream, ids, k_rows, v_rows, _, _ = _run(g["data"], weights)
    t = g["data"]["config"]["tokens"]
    assert hidden.dtype == torch.bfloat16 and stream.dtype == torch.float32 and ids.dtype == torch.int32
    assert hidden.shape == g["ref"]["hidden"].shape and ids.shape == g["ref"]["ids"].shape
    ok, msg, rep = L.check_layer(g["data"], weights, hidden, stream, ids, k_rows, v_rows)
    print(name, msg, rep)
    assert ok, msg
    # Stated tolerance for the BF16 layer output against the reference run with FP8 queries and the
    # same expert ids: relative L2 <= 2e-2.
    q8_hidden, _ = L.ref_back(L.ref_front(g["data"], weights, torch.float8_e4m3fn), weights, ids)
    assert L.relative_l2(hidden, q8_hidden) <= 2e-2
    # new K/V rows: the projection feeding them is rounded to bf16 here and kept in fp32 by the
    # reference, so a few per cent of the E4M3 values land on the neighbouring code (never further)
    for got, want in ((k_rows, g["ref"]["k_new"]), (v_rows, g["ref"]["v_new"])):
        gb, wb = got.reshape(t, -1).view(torch.uint8), want.reshape(t, -1).view(torch.uint8)
        assert (gb != wb).float().mean() < 5e-2
        assert L.relative_l2(got.reshape(t, -1).float(), want.reshape(t, -1).float()) < 2.5e-2   # reference bound: 8e-2
    # expert ids: equal to the reference's wherever its k-th and (k+1)-th scores are not a near tie
    biased = g["ref"]["biased"]
    k = ids.shape[1]
    top = biased.topk(k + 1, dim=-1).values
    clear = (top[:, k - 1] - top[:, k]) > 1e-2
    same = (ids.sort(-1).values == g["ref"]["ids"].sort(-1).values).all(-1)
    assert same[clear].all()


def test_layer_is_repeatable_and_graph_capturable():
    """Same inputs twice give identical outputs (no stale scratch or counters), and a CUDA-graph
    replay on fresh inputs of the same shape matches the eager call."""
    from muse_spark_open_challenge_b200 import layer
    g, weights = load_golden_case("case_tiny_full")
    g2, _ = load_golden_case("case_tiny_full")
    w = to_device(weights, "cuda")
    st = layer.prepare(w)
    d1, d2 = to_device(g["data"], "cuda"), to_device(g2["data"], "cuda")
    h1, s1, i1 = layer.kernel_fn(d1, st)
    h2, s2, i2 = layer.kernel_fn(d2, st)
    torch.cuda.synchronize()
    assert torch.equal(h1, h2) and torch.equal(s1, s2) and torch.equal(i1, i2)
    static = to_device(g["data"], "cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer.kernel_fn(static, st)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = layer.kernel_fn(static, st)
    static["stream"].copy_(d1["stream"] * 1.5)
    static["attn_input"].copy_(L.rms(static["stream"]).to(torch.bfloat16))
    graph.replay()
    torch.cuda.synchronize()
    fresh = to_device(g["data"], "cuda")
    fresh["stream"] = static["stream"].clone()
    fresh["attn_input"] = static["attn_input"].clone()
    h3, s3, i3 = layer.kernel_fn(fresh, st)
    torch.cuda.synchronize()
    layer.check_status(st)
    assert torch.equal(out[0], h3) and torch.equal(out[1], s3) and torch.equal(out[2], i3)


SYNTH_CASES = [
    # (shape, new lens, cached lens, page, kv_scale, local_start)
    # the reference's own shard sizes (hidden 8192, 16q/2kv x 64, 32 of 256 experts x 4096, pooler and
    # unpooler) on the contest's first must-pass shape: sliding window + RoPE, page size 1
    ("NATIVE_SLIDING", [300], [0], 1, 1.0, 96),
    ("MID_SMALL", [300, 211], [0, 130], 64, 1 / 64, 0),
    ("EP_SMALL", [257], [64], 64, 1.0, 32),
    ("TINY", [5, 64, 1, 130], [0, 3, 700, 64], 16, 0.25, 0),
    # decode steps (one new token per request) and verify blocks (eight)
    ("MID_DECODE", [1, 1, 1, 1, 1, 1], [200, 37, 64, 5, 130, 1000], 64, 1 / 64, 0),
    ("MID_VERIFY", [8, 8, 8], [0, 300, 63], 64, 1 / 64, 0),
    ("NATIVE_DECODE", [1, 1, 1], [2500, 77, 300], 64, 1.0, 224),
]


@pytest.mark.parametrize("case", SYNTH_CASES)
def test_layer_on_synthetic_shapes(case):
    """Shapes the reference cannot express (no pooler, shared expert, ragged requests) against the
    CPU oracle that was pinned to the reference on the shapes it can."""
    from muse_spark_open_challenge_b200 import synth
    name, lens, ctxs, page, kv_scale, local_start = case
    shapes = {
        "TINY": synth.TINY,
        "NATIVE_SLIDING": dataclasses.replace(synth.NATIVE, window=2048, rope_theta=5e5),
        # the mid-prefill architecture at reduced width: no pooler, shared expert, head_dim 128
        "MID_SMALL": dataclasses.replace(synth.MID, hidden=1024, hq=8, hkv=2, n_experts=32, local_experts=32,
                                         moe_width=1024, inter=384, shared_inter=512),
        "EP_SMALL": dataclasses.replace(synth.MID, hidden=1024, hq=8, hkv=2, n_experts=64, local_experts=16,
                                        moe_width=1024, inter=256, shared_inter=0),
    }
    shapes["MID_DECODE"] = shapes["MID_VERIFY"] = shapes["MID_SMALL"]
    shapes["NATIVE_DECODE"] = shapes["NATIVE_SLIDING"]
    shape = shapes[name]
    weights = synth.make_weights(shape, seed=7)
    data = synth.make_input(shape, lens, ctxs, seed=8, page=page, kv_scale=kv_scale, local_start=local_start)
    hidden, stream, ids, k_rows, v_rows, _, _ = _run(data, weights)
    ok, msg, rep = L.check_layer(data, weights, hidden, stream, ids, k_rows, v_rows)
    print(name, msg, rep)
    assert ok, msg
    # Stated tolerance at these widths for the BF16 layer output against the reference run with FP8
    # queries and the same expert ids: relative L2 <= 3e-2 (measured 1.5e-2 ... 2.7e-2; the reference-made
    # tiny cases above hold 2e-2), mean absolute error <= 2.5e-2 on outputs of unit scale.
    assert rep["hidden_vs_fp8q"]["rel_l2"] <= 3e-2 and rep["hidden_vs_fp8q"]["mean_abs"] <= 2.5e-2
