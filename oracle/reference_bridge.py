"""TEST INFRASTRUCTURE ONLY: import the unmodified reference (a checkout of
nvbkdw/muse-spark-open-challenge) and run it at sizes other than its hard-coded shard.

The reference reads its sizes from module globals at call time (muse_prefill_layer/
reference.py:29-58), so re-assigning them before a call makes its own code compute another
shape.  Used only to pin the restatement in oracle/layer_ref.py and to produce the golden
vectors under tests/golden/; the checkout directory is given by the MUSE_REFERENCE_DIR
environment variable or a command-line argument and is never needed at test or bench time.
"""
from __future__ import annotations

import importlib
import os
import sys


def load_reference(ref_dir: str | None = None):
    ref_dir = ref_dir or os.environ.get("MUSE_REFERENCE_DIR")
    if not ref_dir or not os.path.isdir(os.path.join(ref_dir, "muse_prefill_layer")):
        raise FileNotFoundError("set MUSE_REFERENCE_DIR to a checkout of the reference repository")
    path = os.path.join(ref_dir, "muse_prefill_layer")
    if path not in sys.path:
        sys.path.insert(0, path)
    return importlib.import_module("reference")


def set_shape(R, *, hidden, hq, hkv, head_dim, n_experts, local_experts, top_k, d_expert, window=None,
              rope_theta=None):
    """Re-assign the reference's size globals (pooled structure only: its D_EXPERT is both the
    MoE width and the experts' intermediate size)."""
    R.HIDDEN, R.HEAD_DIM, R.HQ, R.HKV = hidden, head_dim, hq, hkv
    R.Q_SIZE, R.KV_SIZE = hq * head_dim, hkv * head_dim
    R.QKV_SIZE = 2 * R.Q_SIZE + 2 * R.KV_SIZE
    R.SM_SCALE = head_dim ** -0.5
    R.D_EXPERT, R.N_EXPERTS, R.LOCAL_EXPERTS, R.TOP_K = d_expert, n_experts, local_experts, top_k
    R.UNPOOL_SLICE = hidden // 8
    if window is not None:
        R.SLIDING_WINDOW = window
    if rope_theta is not None:
        R.ROPE_THETA = rope_theta
    R._stream_basis.cache_clear()
    return R
