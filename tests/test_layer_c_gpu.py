"""The whole layer through the library's C host (msl_layer_prepare / msl_layer_prefill) against the
Python host of the same kernels: the prepared weights agree (bit for bit where the arithmetic is integer
or a copy, to fp32 rounding where a sigmoid or a power is evaluated), and with the SAME prepared weights
the C call gives layer.kernel_fn's outputs bit for bit, with and without the side-stream fork."""
import pytest
import torch

from conftest import GOLDEN_CASES, load_golden_case, to_device
from oracle import layer_ref as L

pytestmark = pytest.mark.gpu


def _setup(weights_cpu, data_cpu):
    from muse_spark_open_challenge_b200 import clayer, layer
    weights = to_device(weights_cpu, "cuda")
    data = to_device(data_cpu, "cuda")
    d = L.dims_of(weights_cpu, data_cpu["config"])
    cache_rows = data["k_cache"].numel() // (d.hkv * d.head_dim)
    cfg = clayer.make_config(weights, data_cpu["config"], data["page_table"], cache_rows)
    return clayer, layer, weights, data, cfg


def _ptr_view(st, ptr, dtype, shape):
    """A tensor over a piece of the prepared buffer, found by its device address."""
    n = 1
    for s in shape:
        n *= s
    at = ptr - st["buffer"].data_ptr()
    size = n * torch.empty((), dtype=dtype).element_size()
    assert 0 <= at and at + size <= st["buffer"].numel()
    return st["buffer"][at:at + size].view(dtype).view(shape)


@pytest.mark.parametrize("name", ["case_tiny_full", "case_tiny_sliding", "case_tiny_decode", "case_d128_ep"])
def test_c_host_matches_python_host_on_reference_vectors(name):
    g, weights_cpu = load_golden_case(name)
    clayer, layer, weights, data, cfg = _setup(weights_cpu, g["data"])
    st_py = layer.prepare(weights)
    st_c = clayer.prepare(weights, cfg)
    w = st_c["weights"]
    h, e = cfg.hidden, cfg.n_experts
    # prepared weights: copies and integer work bit for bit ...
    assert torch.equal(_ptr_view(st_c, w.router_hilo, torch.bfloat16, (e, 2 * h)).view(torch.int16),
                       st_py["router_hilo"].view(torch.int16))
    assert torch.equal(_ptr_view(st_c, w.w13_q, torch.uint8, tuple(st_py["w13_q"].shape)), st_py["w13_q"])
    assert torch.equal(_ptr_view(st_c, w.w2_s, torch.uint8, tuple(st_py["w2_s"].shape)), st_py["w2_s"])
    assert torch.equal(_ptr_view(st_c, w.w_pre_ffn, torch.float32, (h,)), st_py["w_pre_ffn"])
    # ... sigmoid / sqrt / pow to fp32 rounding
    for field, key in (("a1", "a1"), ("b1", "b1"), ("a2", "a2"), ("b2", "b2")):
        assert torch.allclose(_ptr_view(st_c, getattr(w, field), torch.float32, (h,)), st_py[key], rtol=2e-6, atol=1e-7), field
    # the C call on the Python host's prepared weights: the same kernels in the same order
    for name_c, key in (("a1", "a1"), ("b1", "b1"), ("a2", "a2"), ("b2", "b2"), ("w_pre_ffn", "w_pre_ffn"),
                        ("w_post_exp", "w_post_exp"), ("w_post_ffn", "w_post_ffn"), ("w_next", "w_next")):
        setattr(w, name_c, st_py[key].data_ptr())
    if cfg.pooled:
        w.w_pre_exp = st_py["w_pre_exp"].data_ptr()
    if cfg.rope_theta:
        w.inv_freq = layer._inv_freq(st_py, g["data"]["config"]["rope_theta"], cfg.head_dim).data_ptr()
    want = layer.kernel_fn(to_device(g["data"], "cuda"), st_py)
    for fork in (True, False):
        fresh = to_device(g["data"], "cuda")
        got = clayer.kernel_fn(fresh, st_c, cfg, fork=fork)
        torch.cuda.synchronize()
        assert int(st_c["status"].item()) == 0
        assert torch.equal(got[2], want[2]), f"{name}: expert ids differ (fork={fork})"
        assert torch.equal(got[1], want[1]) and torch.equal(got[0], want[0]), f"{name}: outputs differ (fork={fork})"
    layer.check_status(st_py)


def test_c_host_with_its_own_prepared_weights_passes_the_oracle():
    """Mid-width synthetic layer (no pooler, shared expert, ragged requests) prepared AND run by the C host."""
    import dataclasses
    from muse_spark_open_challenge_b200 import synth
    shape = dataclasses.replace(synth.MID, hidden=1024, hq=8, hkv=2, n_experts=16, local_experts=16, moe_width=1024,
                                inter=256, shared_inter=512)
    weights_cpu = synth.make_weights(shape, seed=5)
    data_cpu = synth.make_input(shape, [150, 77], [30, 0], seed=20, page=64, kv_scale=0.5)
    clayer, layer, weights, data, cfg = _setup(weights_cpu, data_cpu)
    st = clayer.prepare(weights, cfg)
    hidden, stream, ids = clayer.kernel_fn(data, st, cfg)
    again = clayer.kernel_fn(data, st, cfg)                          # the workspace is reused as it is
    torch.cuda.synchronize()
    assert int(st["status"].item()) == 0
    assert all(torch.equal(a, b) for a, b in zip(again, (hidden, stream, ids)))
    d = L.dims_of(weights_cpu, data_cpu["config"])
    slots = L.new_slots(data_cpu).cuda()
    k_rows = data["k_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
    v_rows = data["v_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
    ok, msg, _ = L.check_layer(data_cpu, weights_cpu, hidden.cpu(), stream.cpu(), ids.cpu(), k_rows, v_rows)
    assert ok, msg
