"""Produce the golden vectors in this directory by running the UNMODIFIED reference
(nvbkdw/muse-spark-open-challenge, muse_prefill_layer/reference.py) on CPU.

    MUSE_REFERENCE_DIR=<checkout> python tests/golden/make_golden.py

Each `<shape>_weights.pt` holds `reference.generate_weights(5353)` at that shape; each
`case_*.pt` holds one `reference.generate_input(...)` dict plus what the reference computes
from it: `ref_kernel` outputs (hidden, stream, expert ids, new FP8 cache rows), the
intermediate tensors of `ref_front` (stream1, h, scores, biased), the attention block's
output, the same outputs with FP8 queries, and the new-token cache slots.  FP8 tensors are
stored as their bytes (uint8).  The tests replay these files without the reference.
"""
from __future__ import annotations

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.reference_bridge import load_reference, set_shape  # noqa: E402

SHAPES = {
    # BASELINE config 0: hidden 512, 8q/2kv x 64, 16 experts top-4, expert width/intermediate 256
    "tiny": dict(hidden=512, hq=8, hkv=2, head_dim=64, n_experts=16, local_experts=16, top_k=4, d_expert=256,
                 window=96, rope_theta=1e6),
    # head_dim 128 with an expert-parallel slice (8 of 16 experts local)
    "d128": dict(hidden=256, hq=4, hkv=1, head_dim=128, n_experts=16, local_experts=8, top_k=4, d_expert=128,
                 window=64, rope_theta=5e5),
}
CASES = {
    "case_tiny_full": ("tiny", dict(batch=1, ctx=0, layer="full", q_len=256, page=64, seed=0)),
    "case_tiny_sliding": ("tiny", dict(batch=2, ctx=100, layer="sliding", q_len=80, page=64, seed=1,
                                       kv_scale=1 / 64)),
    "case_tiny_page1": ("tiny", dict(batch=3, ctx=150, layer="full", q_len=40, page=1, seed=2, dist="outliers")),
    "case_d128_ep": ("d128", dict(batch=2, ctx=70, layer="sliding", q_len=90, page=64, seed=4, local_start=8,
                                  kv_scale=0.5)),
    # a decode step (4 tokens: the sliced unpooler) and a verify block (3 x 8 tokens)
    "case_tiny_decode": ("tiny", dict(batch=4, ctx=200, layer="full", q_len=1, page=64, seed=6)),
    "case_tiny_verify": ("tiny", dict(batch=3, ctx=120, layer="sliding", q_len=8, page=64, seed=8, kv_scale=1 / 64)),
}


def _plain(t):
    return t.view(torch.uint8) if isinstance(t, torch.Tensor) and t.dtype == torch.float8_e4m3fn else t


def main(ref_dir=None):
    R = load_reference(ref_dir)
    import nvfp4 as N   # the reference's codec module, beside reference.py
    done = set()
    for name, (shape_name, case) in CASES.items():
        if os.path.exists(os.path.join(HERE, f"{name}.pt")) and "--all" not in sys.argv:
            continue                           # existing fixtures are kept byte for byte; --all rewrites them
        set_shape(R, **SHAPES[shape_name])
        weights = R.generate_weights(R.WEIGHTS_SEED, device="cpu")
        if shape_name not in done and not os.path.exists(os.path.join(HERE, f"{shape_name}_weights.pt")):
            torch.save({k: _plain(v) for k, v in weights.items()}, os.path.join(HERE, f"{shape_name}_weights.pt"))
            # codec known-answer: the reference's own dequantisation of expert 0's first rows
            torch.save({"w13_rows": N.dequantize(weights["w13"][0, :8], weights["w13_sf"][0, :8], weights["w13_gs"][0]),
                        "w2_rows": N.dequantize(weights["w2"][-1, :8], weights["w2_sf"][-1, :8], weights["w2_gs"][-1])},
                       os.path.join(HERE, f"{shape_name}_dequant.pt"))
            done.add(shape_name)
        data = R.generate_input(**case, device="cpu")
        front = R.ref_front(data, weights)
        hidden, stream, ids, k_new, v_new = R.ref_kernel(data, weights)
        o_in, _, _ = R._attention(data, data["attn_input"].float(), weights)
        q8_hidden, q8_stream = R.ref_back(R.ref_front(data, weights, torch.float8_e4m3fn), weights, ids)
        out = {
            "shape": SHAPES[shape_name], "case": case,
            "data": {k: _plain(v) for k, v in data.items()},
            "ref": {"hidden": hidden, "stream": stream, "ids": ids, "k_new": _plain(k_new), "v_new": _plain(v_new),
                    "stream1": front["stream1"], "h": front["h"], "scores": front["scores"],
                    "biased": front["biased"], "attn_out": o_in, "slots": R.new_slots(data).reshape(-1),
                    "q8_hidden": q8_hidden, "q8_stream": q8_stream},
        }
        torch.save(out, os.path.join(HERE, f"{name}.pt"))
        print("wrote", name, {k: tuple(v.shape) for k, v in out["ref"].items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else None)
