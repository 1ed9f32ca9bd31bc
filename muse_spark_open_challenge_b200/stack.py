"""A stack of decoder layers: layer i's outputs (hidden, stream) are layer i + 1's inputs
(attn_input, stream), as the reference's `ref_kernel` hands them on (reference.py:559-566: it returns
`hidden` as "the next attention input" and the updated residual `stream`).  The reference's harness
times one layer at a time; the stack exists to run the layers back to back as a model would, and, with
several GPUs, to overlap one micro-batch's expert exchange with another micro-batch's attention.

Every layer owns its paged K/V caches; the request geometry (positions, page table, sequence lengths)
is shared by all layers of a step.

Micro-batches: the requests of a step may be given as several `data` dicts (disjoint requests).
Each micro-batch runs on its own CUDA stream with its own scratch state (and, expert parallel, its
own peer slabs and barrier words), layer by layer; since a layer's MoE exchange (NVLink-bound
dispatch, barrier, combine) leaves the SMs mostly idle, another micro-batch's attention and dense
GEMMs fill them.  The streams are forked from and joined to the caller's stream by events, so a whole
step stays capturable in one CUDA graph.
"""
from __future__ import annotations

import torch

from . import layer

_SHARED_KEYS = ("positions", "cache_loc", "cache_seqlens", "seq_lens", "cu_seqlens_q", "page_table", "k_scale",
                "v_scale", "local_start", "config", "scheduler_metadata")


def prepare_stack(weights_per_layer, experts_nvfp4: bool = None) -> list:
    """`layer.prepare` for every layer of the stack."""
    return [layer.prepare(w, experts_nvfp4=experts_nvfp4) for w in weights_per_layer]


def clone_scratch(st: dict) -> dict:
    """A second state over the SAME prepared weights with its own scratch (slabs, counters, barrier words,
    status word, side stream): what a concurrent micro-batch needs."""
    dev = st["device"]
    out = {k: v for k, v in st.items() if k not in ("slab_x", "slab_i", "retired", "quant_x", "quant_i", "marks")}
    out["counts"] = torch.zeros_like(st["counts"])
    out["offsets"] = torch.zeros_like(st["offsets"])
    out["sync"] = torch.zeros_like(st["sync"])
    out["status"] = torch.zeros_like(st["status"])
    out["inv_freq"] = st["inv_freq"]                  # read-only cache, shared
    out["cap"] = 0
    out["side"] = torch.cuda.Stream(dev)
    return out


def layer_inputs(step: dict, index: int, hidden, stream) -> dict:
    """The `data` dict of layer `index`: the step's shared geometry, that layer's caches, and the
    activations handed on by the layer before (or the step's own for layer 0)."""
    d = {k: step[k] for k in _SHARED_KEYS if k in step}
    d["k_cache"], d["v_cache"] = step["k_caches"][index], step["v_caches"][index]
    d["attn_input"] = step["attn_input"] if hidden is None else hidden
    d["stream"] = step["stream"] if stream is None else stream
    return d


def forward(step: dict, states: list, run_layer=None):
    """One step through all layers on the current stream.  `step`: a layer `data` dict whose "k_cache" /
    "v_cache" are replaced by the lists "k_caches" / "v_caches" (one per layer).  Returns (hidden bf16,
    stream fp32, [expert ids per layer]).  `run_layer(data, state, index)` defaults to
    `layer.kernel_fn`."""
    hidden = stream = None
    ids = []
    for i, st in enumerate(states):
        data = layer_inputs(step, i, hidden, stream)
        hidden, stream, layer_ids = (layer.kernel_fn(data, st) if run_layer is None else run_layer(data, st, i))
        ids.append(layer_ids)
    return hidden, stream, ids


class MicroBatches:
    """Streams, events and per-stream states for `forward_interleaved`."""

    def __init__(self, states: list, n: int):
        dev = states[0]["device"]
        self.n = n
        self.streams = [torch.cuda.Stream(dev) for _ in range(n)]
        self.states = [states] + [[clone_scratch(st) for st in states] for _ in range(n - 1)]
        self.fork = torch.cuda.Event()
        self.join = [torch.cuda.Event() for _ in range(n)]


def forward_interleaved(steps: list, mb: MicroBatches, run_layer=None):
    """`forward` for several micro-batches at once, each on its own stream, issued layer by layer in
    round-robin order so that micro-batch b's layer i is in the queue next to micro-batch b + 1's.
    `run_layer(data, state, index, micro_batch)` defaults to `layer.kernel_fn`.  Returns one result
    triple per micro-batch; the caller's stream waits for all of them."""
    if len(steps) != mb.n:
        raise ValueError("one step per micro-batch")
    main = torch.cuda.current_stream()
    mb.fork.record(main)
    carry = [(None, None) for _ in steps]
    ids = [[] for _ in steps]
    for s in mb.streams:
        s.wait_event(mb.fork)
    n_layers = len(mb.states[0])
    for i in range(n_layers):
        for b, step in enumerate(steps):
            with torch.cuda.stream(mb.streams[b]):
                data = layer_inputs(step, i, *carry[b])
                st = mb.states[b][i]
                out = layer.kernel_fn(data, st) if run_layer is None else run_layer(data, st, i, b)
                carry[b] = (out[0], out[1])
                ids[b].append(out[2])
    results = []
    for b in range(mb.n):
        mb.join[b].record(mb.streams[b])
        main.wait_event(mb.join[b])
        for t in carry[b]:
            t.record_stream(main)
        results.append((carry[b][0], carry[b][1], ids[b]))
    return results
