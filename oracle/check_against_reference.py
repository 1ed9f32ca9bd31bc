"""TEST INFRASTRUCTURE ONLY: pin oracle/layer_ref.py to the unmodified reference.

Runs the reference's own `generate_weights` / `generate_input` / `ref_kernel` /
`check_implementation` and the restatement on the same seeded CPU tensors and requires:
expert ids and new FP8 cache rows identical, stream and hidden equal to fp32 rounding
(the reference switches to a fused SDPA call for blocks of >= 256 queries, the restatement
always uses the explicit softmax, so the last bits may differ).

    MUSE_REFERENCE_DIR=<checkout> python oracle/check_against_reference.py
"""
from __future__ import annotations

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import layer_ref as L  # noqa: E402
from oracle.reference_bridge import load_reference, set_shape  # noqa: E402

SHAPES = {
    "tiny": dict(hidden=512, hq=8, hkv=2, head_dim=64, n_experts=16, local_experts=16, top_k=4, d_expert=256,
                 window=96, rope_theta=1e6),
    "d128": dict(hidden=1024, hq=8, hkv=2, head_dim=128, n_experts=32, local_experts=8, top_k=8, d_expert=512,
                 window=64, rope_theta=5e5),
}
CASES = [
    ("tiny", dict(batch=1, ctx=0, layer="full", q_len=256, page=64, seed=0)),
    ("tiny", dict(batch=2, ctx=100, layer="sliding", q_len=80, page=64, seed=1, kv_scale=1 / 64)),
    ("tiny", dict(batch=3, ctx=150, layer="full", q_len=40, page=1, seed=2, dist="outliers")),
    ("tiny", dict(batch=2, ctx=300, layer="sliding", q_len=300, page=16, seed=3, spread="agentic", dist="soft")),
    ("d128", dict(batch=2, ctx=70, layer="full", q_len=90, page=64, seed=4, local_start=8)),
    ("d128", dict(batch=1, ctx=200, layer="sliding", q_len=130, page=1, seed=5, local_start=24, kv_scale=0.5)),
    # decode steps and verify blocks; up to 8 tokens take the sliced unpooler (reference.py:468-470)
    ("tiny", dict(batch=4, ctx=200, layer="full", q_len=1, page=64, seed=6)),
    ("tiny", dict(batch=1, ctx=150, layer="sliding", q_len=8, page=16, seed=7, kv_scale=1 / 64)),
    ("tiny", dict(batch=3, ctx=120, layer="sliding", q_len=8, page=64, seed=8)),
    ("d128", dict(batch=9, ctx=90, layer="full", q_len=1, page=64, seed=9, local_start=16)),
]


def main(ref_dir=None):
    R = load_reference(ref_dir)
    worst = 0.0
    for shape_name, case in CASES:
        set_shape(R, **SHAPES[shape_name])
        weights = R.generate_weights(R.WEIGHTS_SEED, device="cpu")
        data = R.generate_input(**case, device="cpu")
        hid_r, str_r, ids_r, k_r, v_r = R.ref_kernel(data, weights)
        hid_o, str_o, ids_o, k_o, v_o = L.ref_kernel(data, weights)
        t = data["config"]["tokens"]
        assert torch.equal(ids_r, ids_o), f"{shape_name} {case}: expert ids differ"
        assert torch.equal(k_r.reshape(t, -1).view(torch.uint8), k_o.reshape(t, -1).view(torch.uint8)), "k rows"
        assert torch.equal(v_r.reshape(t, -1).view(torch.uint8), v_o.reshape(t, -1).view(torch.uint8)), "v rows"
        assert torch.equal(R.new_slots(data).reshape(-1), L.new_slots(data)), "cache slots"
        e_s, e_h = L.relative_l2(str_o, str_r), L.relative_l2(hid_o, hid_r)
        worst = max(worst, e_s, e_h)
        assert e_s < 2e-6 and e_h < 2e-3, (e_s, e_h)     # hidden is bf16: one flipped rounding = 4e-3 of one value
        # The restatement's acceptance check agrees with the reference's on the reference's own output.
        slots = L.new_slots(data)
        kf = data["k_cache"].view(-1, R.HKV, R.HEAD_DIM)
        vf = data["v_cache"].view(-1, R.HKV, R.HEAD_DIM)
        kf[slots] = k_r.reshape(t, R.HKV, R.HEAD_DIM)      # what a layer implementation writes in place
        vf[slots] = v_r.reshape(t, R.HKV, R.HEAD_DIM)
        raw = R.collect(data, (hid_r, str_r, ids_r))
        ok_r, msg_r = R.check_implementation(data, raw, weights)
        ok_o, msg_o, _ = L.check_layer(data, weights, hid_r, str_r, ids_r, kf[slots], vf[slots])
        assert ok_r and ok_o, (msg_r, msg_o)
        # and both reject a perturbed output alike
        bad = str_r + 0.5 * str_r.abs().mean() * torch.randn(str_r.shape, generator=torch.Generator().manual_seed(1))
        ok_rb, _ = R.check_implementation(data, R.collect(data, (hid_r, bad, ids_r)), weights)
        ok_ob, _, _ = L.check_layer(data, weights, hid_r, bad, ids_r, kf[slots], vf[slots])
        assert not ok_rb and not ok_ob
        print(f"ok {shape_name} {case}  stream {e_s:.1e} hidden {e_h:.1e}  ref-check={ok_r}")
    print(f"restatement pinned to the reference on {len(CASES)} cases; worst rel-L2 {worst:.2e}")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else None)
