"""The CPU oracle against the golden vectors made by the unmodified reference
(tests/golden/make_golden.py): ids, cache rows and slots identical; fp32 tensors to rounding."""
import numpy as np
import pytest
import torch

from conftest import GOLDEN, GOLDEN_CASES, load_golden_case, load_golden_weights
from oracle import layer_ref as L
from oracle import nvfp4_ref


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_layer_oracle_matches_reference_vectors(name):
    g, weights = load_golden_case(name)
    data, ref = g["data"], g["ref"]
    hidden, stream, ids, k_new, v_new = L.ref_kernel(data, weights)
    t = data["config"]["tokens"]
    assert torch.equal(ids, ref["ids"])
    assert torch.equal(k_new.reshape(t, -1).view(torch.uint8), ref["k_new"].reshape(t, -1).view(torch.uint8))
    assert torch.equal(v_new.reshape(t, -1).view(torch.uint8), ref["v_new"].reshape(t, -1).view(torch.uint8))
    assert torch.equal(L.new_slots(data), ref["slots"])
    assert L.relative_l2(stream, ref["stream"]) < 2e-6
    assert L.relative_l2(hidden, ref["hidden"]) < 2e-3     # bf16: a flipped rounding is 4e-3 of one value
    front = L.ref_front(data, weights)
    assert L.relative_l2(front["stream1"], ref["stream1"]) < 2e-6
    assert L.relative_l2(front["h"], ref["h"]) < 2e-6
    assert torch.allclose(front["biased"], ref["biased"], atol=2e-6)
    q8h, q8s = L.ref_back(L.ref_front(data, weights, torch.float8_e4m3fn), weights, ref["ids"])
    assert L.relative_l2(q8s, ref["q8_stream"]) < 2e-6


@pytest.mark.parametrize("name", GOLDEN_CASES[:2])
def test_check_layer_accepts_reference_and_rejects_noise(name):
    g, weights = load_golden_case(name)
    data, ref = g["data"], g["ref"]
    t = data["config"]["tokens"]
    d = L.dims_of(weights, data["config"])
    k = ref["k_new"].reshape(t, d.hkv, d.head_dim)
    v = ref["v_new"].reshape(t, d.hkv, d.head_dim)
    ok, msg, rep = L.check_layer(data, weights, ref["hidden"], ref["stream"], ref["ids"], k, v)
    assert ok, msg
    noisy = ref["stream"] + 0.3 * torch.randn(ref["stream"].shape, generator=torch.Generator().manual_seed(0))
    ok, msg, _ = L.check_layer(data, weights, ref["hidden"], noisy, ref["ids"], k, v)
    assert not ok
    bad_ids = ref["ids"].clone()
    bad_ids[:, 1] = bad_ids[:, 0]
    ok, msg, _ = L.check_layer(data, weights, ref["hidden"], ref["stream"], bad_ids, k, v)
    assert not ok and "routing" in msg


@pytest.mark.parametrize("shape", ["tiny", "d128"])
def test_nvfp4_codec_known_answers(shape):
    w = load_golden_weights(shape)
    ka = torch.load(f"{GOLDEN}/{shape}_dequant.pt")
    for bank, e, key in (("w13", 0, "w13_rows"), ("w2", -1, "w2_rows")):
        packed = w[bank][e, :8].numpy()
        sf = w[bank + "_sf"][e, :8].view(torch.uint8).numpy()
        gs = float(w[bank + "_gs"][e])
        got = nvfp4_ref.dequantize(packed, sf, gs)
        assert np.array_equal(got, ka[key].numpy())
        got_t = L.nvfp4_dequantize(w[bank][e, :8], w[bank + "_sf"][e, :8], w[bank + "_gs"][e])
        assert torch.equal(got_t, ka[key])


def test_e4m3_decode_matches_torch():
    b = torch.arange(256, dtype=torch.uint8)
    want = b.view(torch.float8_e4m3fn).float().numpy()
    got = nvfp4_ref.e4m3_to_f32(b.numpy())
    assert np.array_equal(np.isnan(got), np.isnan(want))
    m = ~np.isnan(want)
    assert np.array_equal(got[m], want[m])


def test_ragged_requests_equal_separate_uniform_calls():
    """Per-request lengths (absent from the reference) must reduce to the uniform case: a ragged
    batch gives each request the output it gets when run alone."""
    from muse_spark_open_challenge_b200 import synth
    shape = synth.TINY
    w = synth.make_weights(shape, seed=3)
    lens, ctxs = [37, 64, 5], [10, 0, 130]
    data = synth.make_input(shape, lens, ctxs, seed=4, page=16, kv_scale=0.25)
    o_all, k_all, v_all = L.attention_block(data, data["attn_input"].float(), w, L.dims_of(w, data["config"]))
    at = 0
    for b, n in enumerate(lens):
        one = dict(data)
        one["cu_seqlens_q"] = torch.tensor([0, n], dtype=torch.int32)
        one["seq_lens"] = data["seq_lens"][b:b + 1]
        one["page_table"] = data["page_table"][b:b + 1]
        o1, k1, v1 = L.attention_block(one, data["attn_input"][at:at + n].float(), w, L.dims_of(w, data["config"]))
        assert torch.allclose(o1, o_all[at:at + n], atol=1e-6)
        assert torch.equal(k1.view(torch.uint8), k_all[at:at + n].view(torch.uint8))
        at += n
