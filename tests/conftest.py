"""Shared test plumbing: the `gpu` marker, golden-vector loading, repo root on sys.path."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")
FP8 = torch.float8_e4m3fn
_FP8_KEYS = {"k_cache", "v_cache", "k_new", "v_new", "w13_sf", "w2_sf"}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _restore(d):
    return {k: (v.view(FP8) if k in _FP8_KEYS and isinstance(v, torch.Tensor) else v) for k, v in d.items()}


def load_golden_weights(shape_name):
    return _restore(torch.load(os.path.join(GOLDEN, f"{shape_name}_weights.pt")))


def load_golden_case(name):
    g = torch.load(os.path.join(GOLDEN, f"{name}.pt"))
    g["data"] = _restore(g["data"])
    g["ref"] = _restore(g["ref"])
    shape_name = "tiny" if "tiny" in name else "d128"
    return g, load_golden_weights(shape_name)


GOLDEN_CASES = ["case_tiny_full", "case_tiny_sliding", "case_tiny_page1", "case_d128_ep", "case_tiny_decode",
                "case_tiny_verify"]


def to_device(obj, device):
    if isinstance(obj, torch.Tensor):
        return obj.to(device)
    if isinstance(obj, dict):
        return {k: to_device(v, device) for k, v in obj.items()}
    return obj
