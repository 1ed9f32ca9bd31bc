"""Several decoder layers back to back (layer i's hidden state and residual stream feed layer i + 1,
reference.py:559-566): every layer is judged by the oracle's layer check on exactly the inputs the
layer before produced; two micro-batches interleaved on two streams give the bits each gives alone;
the whole stack replays as one CUDA graph."""
import dataclasses

import pytest
import torch

from conftest import to_device
from oracle import layer_ref as L

pytestmark = pytest.mark.gpu
N_LAYERS = 3


def _stack(seed0=5):
    from muse_spark_open_challenge_b200 import synth
    shape = dataclasses.replace(synth.MID, hidden=1024, hq=8, hkv=2, n_experts=16, local_experts=16, moe_width=1024,
                                inter=256, shared_inter=512)
    return shape, [synth.make_weights(shape, seed=seed0 + i) for i in range(N_LAYERS)]


def _step(shape, lens, ctxs, seed):
    """A step's inputs: one synthetic layer input per layer supplies that layer's own caches."""
    from muse_spark_open_challenge_b200 import synth
    per_layer = [synth.make_input(shape, lens, ctxs, seed=seed + 100 * i, page=64, kv_scale=0.5) for i in range(N_LAYERS)]
    step = dict(per_layer[0])
    step["k_caches"] = [d["k_cache"] for d in per_layer]
    step["v_caches"] = [d["v_cache"] for d in per_layer]
    del step["k_cache"], step["v_cache"]
    return step


def _to_dev(step):
    out = to_device({k: v for k, v in step.items() if k not in ("k_caches", "v_caches")}, "cuda")
    out["k_caches"] = [t.cuda() for t in step["k_caches"]]
    out["v_caches"] = [t.cuda() for t in step["v_caches"]]
    return out


def test_every_layer_of_a_stack_passes_the_oracle_on_its_own_inputs():
    from muse_spark_open_challenge_b200 import layer, stack
    shape, weights = _stack()
    states = stack.prepare_stack([to_device(w, "cuda") for w in weights])
    step = _step(shape, [150, 77], [30, 0], seed=20)
    dev = _to_dev(step)
    seen = []

    def run(data, st, i):
        out = layer.kernel_fn(data, st)
        seen.append((data, out))
        return out

    hidden, stream, ids = stack.forward(dev, states, run_layer=run)
    torch.cuda.synchronize()
    for st in states:
        layer.check_status(st)
    assert len(ids) == N_LAYERS and hidden.shape == (227, shape.hidden)
    for i, (data, out) in enumerate(seen):
        cpu = {k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in data.items()}
        # the caches as the step found them (the kernel has since written the new rows into its copy)
        cpu["k_cache"], cpu["v_cache"] = step["k_caches"][i], step["v_caches"][i]
        d = L.dims_of(weights[i], cpu["config"])
        slots = L.new_slots(cpu).cuda()
        k_rows = data["k_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
        v_rows = data["v_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
        ok, msg, _ = L.check_layer(cpu, weights[i], out[0].cpu(), out[1].cpu(), out[2].cpu(), k_rows, v_rows)
        assert ok, f"layer {i}: {msg}"
    # layer i + 1 really consumed layer i's outputs
    assert seen[1][0]["attn_input"] is seen[0][1][0] and seen[2][0]["stream"] is seen[1][1][1]


def test_interleaved_micro_batches_equal_separate_runs_and_the_stack_is_capturable():
    from muse_spark_open_challenge_b200 import layer, stack
    shape, weights = _stack()
    states = stack.prepare_stack([to_device(w, "cuda") for w in weights])
    steps = [_step(shape, [150, 77], [30, 0], seed=20), _step(shape, [64, 200], [0, 128], seed=40)]
    alone = []
    for s in steps:
        h, r, ids = stack.forward(_to_dev(s), states)
        alone.append((h.clone(), r.clone(), [i.clone() for i in ids]))
    mb = stack.MicroBatches(states, 2)
    both = stack.forward_interleaved([_to_dev(s) for s in steps], mb)
    torch.cuda.synchronize()
    for sts in mb.states:
        for st in sts:
            layer.check_status(st)
    for (h0, r0, i0), (h1, r1, i1) in zip(alone, both):
        assert torch.equal(h0, h1) and torch.equal(r0, r1) and all(torch.equal(a, b) for a, b in zip(i0, i1))
    # one CUDA graph for the whole stack, replayed
    dev = _to_dev(steps[0])
    stack.forward(dev, states)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gh, gr, gi = stack.forward(dev, states)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(gh, alone[0][0]) and torch.equal(gr, alone[0][1])
