"""No-GPU checks of the drop-in boundary: the library builds, loads and exports exactly the entry
points include/msl.h declares; argument errors are rejected on the host before any launch; the
pure-host parts of `prepare` (router split, gate/up interleave, synthetic generators) behave."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT


@pytest.fixture(scope="module")
def lib():
    from muse_spark_open_challenge_b200 import build, _lib
    build.build()
    return _lib.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "msl.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(msl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    from muse_spark_open_challenge_b200 import _lib
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/msl.h but not exported"
    assert sorted(_lib.SIGNATURES) == names          # the ctypes table binds exactly the header
    assert lib.msl_abi_version() == _lib.ABI_VERSION == 2
    assert lib.msl_status_string(0) == b"ok" and b"argument" in lib.msl_status_string(-1)


def test_argument_errors_are_rejected_before_any_launch(lib):
    null = ctypes.c_void_p(0)
    assert lib.msl_gemm_bf16(null, 8, null, 8, null, 8, 1, 1, 8, 1, 0, 0, 0, 1.0, null, null) == -1
    fake = ctypes.c_void_p(1 << 20)
    assert lib.msl_gemm_bf16(fake, 7, fake, 8, fake, 8, 1, 8, 8, 1, 0, 0, 0, 1.0, null, null) == -2   # pitch
    assert lib.msl_gemm_bf16(fake, 8, fake, 8, fake, 8, 0, 8, 8, 1, 0, 0, 0, 1.0, null, null) == 0    # m = 0
    assert lib.msl_boundary(fake, 8, null, fake, fake, fake, fake, fake, fake, 8, 0, 8, 1e-8, 1e-5, null) == 0
    assert lib.msl_boundary(fake, 8, null, fake, fake, fake, fake, fake, fake, 8, 1, 12, 1e-8, 1e-5, null) == -2
    assert lib.msl_route_topk(fake, 8, 0, fake, 1.0, fake, 1, 4, 8, 4, fake, fake, fake, fake, fake, null) == -1
    # the allocation-free routing entry checks everything before it touches its array or enqueues work
    rds = lambda **kw: lib.msl_route_dispatch_static(   # noqa: E731
        kw.get("logits", fake), 8, 0, fake, 1.0, fake, kw.get("x", fake), kw.get("ldx", 8), null, kw.get("tokens", 4),
        kw.get("n_experts", 16), kw.get("top_k", 4), kw.get("n_local", 8), kw.get("width", 8), fake, fake,
        kw.get("slab", fake), 64, fake, fake, null, null)
    assert rds(n_local=0) == -1 and rds(n_local=-3) == -1 and rds(n_local=17) == -1
    assert rds(logits=null) == -1 and rds(x=null) == -1 and rds(slab=null) == -1
    assert rds(top_k=17, n_experts=64) == -1                      # accepted by the routing, not by the dispatch
    assert rds(n_experts=1024, n_local=8) == -7                   # more experts than the routing kernel supports
    assert rds(width=12) == -2 and rds(ldx=4) == -2 and rds(x=ctypes.c_void_p((1 << 20) + 8)) == -2
    assert rds(tokens=0) == 0
    assert lib.msl_route_dispatch(fake, 8, 0, fake, 1.0, fake, fake, 8, null, 4, 16, 4, 8, 8, fake, fake, fake, fake,
                                  fake, null, fake, 64, fake, fake, null, null) == -1      # no barrier words
    assert lib.msl_combine_boundary(fake, fake, fake, fake, null, 0, 4, 4, 64, null, null, fake, fake, fake, fake, fake,
                                    64, 1e-8, 1e-5, null, null) == -1                      # no residual stream
    # options: a value outside {0, 1} or an unknown option is refused; a set value reads back
    assert lib.msl_set_option(99, 1) == -1 and lib.msl_set_option(0, 2) == -1
    old = lib.msl_get_option(1)
    assert lib.msl_set_option(1, 0) == 0 and lib.msl_get_option(1) == 0
    assert lib.msl_set_option(1, old) == 0 and lib.msl_get_option(1) == old
    assert lib.msl_nvfp4_padded_rows(3072, 1) == 3072 and lib.msl_nvfp4_padded_rows(512, 1) == 512
    assert lib.msl_nvfp4_padded_rows(128, 0) == 256 and lib.msl_nvfp4_padded_rows(200, 1) == 256


def test_split_kv_plan_counts_waves(lib):
    """The slice count of split-KV attention comes from sizes alone (148 SMs assumed without a GPU): one CTA
    runs per SM at a time, so the plan takes the count whose waves x key tiles per slice is smallest, and
    leaves calls that already fill two waves unsliced (their bits must not depend on the batch)."""
    plan = lib.msl_attention_split_plan
    # 753 new tokens after 80000 cached, 16 q / 2 kv heads, one-token pages: 48 query blocks
    assert plan(1, 753, 16, 2, 80753, 1, 0) == 3           # 144 CTAs: one wave of 211 tiles (7 slices: 3 waves of 91)
    assert plan(4, 753, 16, 2, 80753, 1, 0) == 3           # 576 CTAs: 3.9 waves of 211 (2 slices: 2.6 waves of 316)
    # whole prefills are never sliced, alone or in a batch
    assert plan(1, 4096, 32, 8, 64, 64, 0) == 1 and plan(4, 4096, 32, 8, 64, 64, 0) == 1
    # a decode step over 4096 cached tokens: as many slices as leave eight key tiles each
    assert plan(1, 1, 32, 8, 64, 64, 0) == 4
    # short contexts and bad arguments: no slicing
    assert plan(1, 1, 32, 8, 8, 64, 0) == 1 and plan(0, 1, 32, 8, 64, 64, 0) == 1 and plan(1, 1, 32, 5, 64, 64, 0) == 1


def test_split_k_plan_follows_the_cost_model(lib):
    """The K slices of a dense product come from sizes alone (148 SMs assumed without a GPU): rounds of work
    items x K steps per item, plus the reduction pass, for 128- and 256-row tiles; slicing must save 5 %."""
    plan = lib.msl_gemm_splitk_plan
    # the 753-token products of the native shard: QKV and pooler as K slices of 256-row tiles
    assert plan(753, 2304, 8192, 1, 0) == 5 and plan(753, 4096, 8192, 1, 0) == 3
    # unpooler and output projection: 96 tiles of 256 rows in one round, nothing to gain from slices
    assert plan(753, 8192, 4096, 1, 0) == 1 and plan(753, 8192, 1024, 1, 0) == 1
    # six tiles with 256 K steps (the two-segment router): the most slices allowed
    assert plan(753, 256, 8192, 2, 1) == 16
    # prefill-sized products fill the GPU; the fused SiLU output cannot be sliced; short K is not sliced
    assert plan(16384, 10240, 4096, 1, 0) == 1 and plan(3012, 4096, 8192, 1, 0) == 1
    assert plan(753, 256, 8192, 2, 2) == 1 and plan(8, 2304, 512, 1, 0) == 1
    # with slicing switched off every product runs in one pass
    old = lib.msl_get_option(0)
    try:
        assert lib.msl_set_option(0, 0) == 0 and plan(753, 2304, 8192, 1, 0) == 1
    finally:
        lib.msl_set_option(0, old)


def test_missing_library_fails_loudly(tmp_path):
    from muse_spark_open_challenge_b200 import _lib
    with pytest.raises(_lib.MslError):
        _lib.load(str(tmp_path / "nope.so"))


def test_prepare_refuses_cpu_tensors():
    from muse_spark_open_challenge_b200 import layer, synth
    from muse_spark_open_challenge_b200._lib import MslError
    w = synth.make_weights(synth.TINY, seed=0)
    with pytest.raises(MslError):
        layer.prepare(w)


def test_interleave_gate_up_layout():
    from muse_spark_open_challenge_b200 import ops
    inter, k = 384, 8
    w = torch.arange(2 * inter, dtype=torch.float32)[:, None].expand(2 * inter, k).contiguous()
    out = ops.interleave_gate_up(w)
    for tile in range(inter // 128):
        blk = out[tile * 256:(tile + 1) * 256, 0]
        assert torch.equal(blk[:128], torch.arange(tile * 128, tile * 128 + 128).float())
        assert torch.equal(blk[128:], inter + torch.arange(tile * 128, tile * 128 + 128).float())


def test_router_hi_lo_split_recovers_fp32_to_2e_minus_17():
    r = 0.045 * torch.randn((64, 512), generator=torch.Generator().manual_seed(0))
    hi = r.to(torch.bfloat16)
    lo = (r - hi.float()).to(torch.bfloat16)
    err = (hi.float() + lo.float() - r).abs().max() / r.abs().max()
    assert err < 2 ** -16


def test_synthetic_generators_follow_the_reference_schema():
    from muse_spark_open_challenge_b200 import synth
    from oracle import layer_ref as L
    shape = synth.TINY
    w = synth.make_weights(shape, seed=1)
    data = synth.make_input(shape, [7, 64, 3], [0, 100, 5], seed=2, page=16, kv_scale=0.5)
    assert data["stream"].dtype == torch.float32 and data["attn_input"].dtype == torch.bfloat16
    assert data["k_cache"].dtype == torch.float8_e4m3fn and data["k_cache"].shape[1:] == (16, shape.hkv, shape.head_dim)
    assert data["cu_seqlens_q"].tolist() == [0, 7, 71, 74] and data["positions"].dtype == torch.int64
    assert torch.equal(data["cache_loc"], L.new_slots(data))       # the two slot derivations agree
    assert len(set(data["cache_loc"].tolist())) == 74
    d = L.dims_of(w, data["config"])
    assert (d.hidden, d.moe_width, d.inter, d.pooled) == (512, 256, 256, True)
    # a ragged batch runs through the oracle end to end
    hidden, stream, ids, k_new, v_new = L.ref_kernel(data, w)
    assert hidden.shape == (74, 512) and ids.shape == (74, 4) and torch.isfinite(stream).all()


def test_zipf_targets_and_router_skew():
    from muse_spark_open_challenge_b200 import synth
    t = synth.zipf_targets(128, 16384 * 8, s=1.1, cap=3000, n_empty=2)
    assert abs(float(t.sum()) - 16384 * 8) < 1 and float(t.max()) <= 3000 and int((t == 0).sum()) == 2
    shape = synth.TINY
    w = synth.make_weights(shape, seed=3)
    h = torch.randn((2048, shape.hidden), generator=torch.Generator().manual_seed(4))
    targets = synth.zipf_targets(shape.n_experts, 2048 * shape.top_k, cap=2048, n_empty=1)
    synth.skew_router(w, h, targets, shape.top_k, sample=2048)
    scores = torch.sigmoid((h @ w["router"].T) * synth.ROUTER_MULTIPLIER) + w["router_bias"]
    counts = torch.bincount(scores.topk(shape.top_k, dim=-1).indices.flatten(), minlength=shape.n_experts)
    assert int((counts == 0).sum()) >= 1 and counts.max() > 4 * counts[counts > 0].min()
