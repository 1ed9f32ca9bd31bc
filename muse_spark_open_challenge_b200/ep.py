"""Expert-parallel form of the layer: one process per GPU, experts sharded contiguously
(rank r owns experts [r*E/W, (r+1)*E/W), the reference's `local_start` notion, reference.py:48-50,
466), requests sharded by rank, one exchange pair per layer over `torch.distributed`.

The reference replaces every cross-GPU step by the identity (reference.py:438,451,467); this module
supplies the exchange it leaves out:

    route over ALL experts -> rows grouped by expert (= grouped by owner rank)
    counts all-to-all -> row all-to-all (dispatch) -> local grouped GEMMs over (source, expert) groups
    -> row all-to-all back (combine) -> local weighted sum

Two transports:

* collective (`moe_stage`): the plan and both row exchanges are `torch.distributed` all-to-alls,
  device- and backend-agnostic (`gloo` on CPU in the tests, `nccl` on GPUs).  The split sizes are read
  on the host (one small synchronisation per layer).
* peer memory (`moe_stage_peer`, GPUs of one NVLink domain): every rank's row slab is mapped into
  every other rank; the dispatch kernel stores token rows straight into the owners' slabs and the
  combine kernel loads expert outputs straight from them, so both row exchanges are fused into the
  kernels either side of the expert GEMMs.  The route counts are all-gathered on the device and the
  row placement is computed there: no host synchronisation.  Three stream barriers per layer order
  the peer stores and loads.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import layer, ops
from ._lib import OUT_F32, OUT_SWIGLU_BF16


@dataclass
class ExchangePlan:
    send_splits: list      # rows this rank sends to each rank (its routes to that rank's experts)
    recv_splits: list      # rows this rank receives from each rank
    recv_counts: torch.Tensor   # i32 [world, local experts]: rows from source s for local expert e
    group_offsets: torch.Tensor  # i32 [world * local + 1]: row ranges of the (source, expert) groups

    @property
    def recv_rows(self):
        return sum(self.recv_splits)


def begin_plan(counts: torch.Tensor, world: int, group=None):
    """First half of the plan: the counts all-to-all and an asynchronous copy of the split sizes to
    the host.  counts: i32 [E] routes of this rank per global expert (rows of the send slab are
    ordered by expert).  Returns the pending pieces for `finish_plan`."""
    e = counts.numel()
    local = e // world
    mat = counts.view(world, local).contiguous()
    recv = torch.empty_like(mat)
    dist.all_to_all_single(recv, mat, group=group)
    both = torch.stack([mat.sum(1), recv.sum(1)])
    offs = torch.zeros(world * local + 1, dtype=torch.int32, device=counts.device)
    offs[1:] = torch.cumsum(recv.flatten(), 0).to(torch.int32)
    if both.is_cuda:
        host = torch.empty(both.shape, dtype=both.dtype, pin_memory=True)
        host.copy_(both, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
    else:
        host, done = both, None
    return host, done, recv, offs


def finish_plan(pending) -> ExchangePlan:
    """Second half: wait (on the host) for the split sizes only."""
    host, done, recv, offs = pending
    if done is not None:
        done.synchronize()                   # the one host synchronisation of the layer
    return ExchangePlan(host[0].tolist(), host[1].tolist(), recv, offs)


def make_plan(counts: torch.Tensor, world: int, group=None) -> ExchangePlan:
    """One all-to-all of the counts tells every rank what it will receive."""
    return finish_plan(begin_plan(counts, world, group))


def exchange_rows(send: torch.Tensor, out_rows: int, send_splits, recv_splits, out=None, group=None):
    """Variable-size all-to-all of rows (dim 0)."""
    if out is None:
        out = torch.empty((out_rows, send.shape[1]), dtype=send.dtype, device=send.device)
    dist.all_to_all_single(out[:out_rows], send, list(recv_splits), list(send_splits), group=group)
    return out


class ExpertParallel:
    """Per-rank context: world geometry plus grow-only receive buffers."""

    def __init__(self, st: dict, world: int, rank: int, n_experts: int, group=None):
        if n_experts % world:
            raise ValueError("the expert count must divide evenly over the ranks")
        if st["n_local"] != n_experts // world:
            raise ValueError("state holds a different number of local experts than n_experts / world")
        self.world, self.rank, self.n_experts, self.group = world, rank, n_experts, group
        self.zero = torch.zeros(1, dtype=torch.int32, device=st["device"])
        self.counts = torch.zeros(n_experts, dtype=torch.int32, device=st["device"])
        self.send_offsets = torch.zeros(n_experts + 1, dtype=torch.int32, device=st["device"])
        self.cap = 0
        self.recv_x = self.recv_i = None
        self.peer = None                       # set by enable_peer
        self.side = torch.cuda.Stream(st["device"]) if torch.device(st["device"]).type == "cuda" else None

    def buffers(self, st, rows):
        if rows > self.cap:
            rows_cap = int(rows * 1.25) + 128
            self.recv_x = torch.empty((rows_cap, st["moe_width"]), dtype=torch.bfloat16, device=st["device"])
            self.recv_i = torch.empty((rows_cap, st["inter"]), dtype=torch.bfloat16, device=st["device"])
            self.cap = rows_cap
        return self.recv_x, self.recv_i


class PeerSlabs:
    """Peer-mapped memory of one rank, allocated as symmetric memory and exchanged once: a bf16
    [cap, width] row slab (what the other ranks dispatch into and read expert outputs from) followed by
    `guard_rows` rows that nothing may touch (the tests check them) and the barrier's flag words; plus
    the device arrays of every rank's pointers to the slab and to the flag words."""

    FLAG_BYTES = 4096

    def __init__(self, ctx: "ExpertParallel", st: dict, cap: int, guard_rows: int = 0):
        dev = torch.device(st["device"])
        width = st["moe_width"]
        slab_bytes = cap * width * 2
        guard_bytes = guard_rows * width * 2
        flags_at = slab_bytes + guard_bytes
        if ctx.world > 1:
            import torch.distributed._symmetric_memory as symm

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer loads/stores only
            self.raw = symm.empty(flags_at + self.FLAG_BYTES, dtype=torch.uint8, device=dev)
            self.raw.zero_()
            group = ctx.group if ctx.group is not None else dist.group.WORLD
            self.handle = symm.rendezvous(self.raw, group)
            bases = [int(p) for p in self.handle.buffer_ptrs]
        else:                                  # a single rank is its own and only peer: ordinary memory will do
            self.raw = torch.zeros(flags_at + self.FLAG_BYTES, dtype=torch.uint8, device=dev)
            bases = [self.raw.data_ptr()]
        self.slab = self.raw[:slab_bytes].view(torch.bfloat16).view(cap, width)
        self.guard = self.raw[slab_bytes:flags_at]
        self.flags = self.raw[flags_at:flags_at + self.FLAG_BYTES].view(torch.int32)
        self.slab_ptrs = torch.tensor(bases, dtype=torch.int64, device=dev)
        self.flag_ptrs = torch.tensor([b + flags_at for b in bases], dtype=torch.int64, device=dev)
        self.cap = cap
        torch.cuda.synchronize(dev)
        if ctx.world > 1:
            dist.barrier(group=ctx.group)      # every rank's flag words are zero before the first barrier


def enable_peer(ctx: "ExpertParallel", st: dict, max_tokens: int, top_k: int, capacity_factor: float = 2.0,
                cap_rows: int = None, guard_rows: int = 0):
    """Switch `ctx` to the peer-memory transport.  Every rank's slab holds up to
    capacity_factor * max_tokens * top_k rows (never more than the worst case world * max_tokens *
    top_k; `cap_rows` sets the size directly); a layer whose routing needs more sets MSL_ERR_CAPACITY in
    the status word, the rows that do not fit are dropped, and no kernel addresses a row at or beyond
    the capacity.  The combine kernel loads the expert outputs from the owners' slabs.  (Returning
    the outputs from the down projection's epilogue instead, 64-byte stores over NVLink, was built and
    measured three times slower: 5.7 against 1.9 ms on two GPUs.  Not kept.)"""
    dev = st["device"]
    most = torch.tensor([max_tokens], dtype=torch.int64, device=dev)
    if ctx.world > 1:
        dist.all_reduce(most, op=dist.ReduceOp.MAX, group=ctx.group)   # slabs have one size on every rank
    cap = int(min(ctx.world, capacity_factor) * int(most.item()) * top_k) if cap_rows is None else int(cap_rows)
    cap = (cap + 255) // 256 * 256
    ctx.peer = PeerSlabs(ctx, st, cap, guard_rows)
    # the intermediate slab carries the same number of guard rows behind it
    ctx.recv_i_raw = torch.zeros((cap + guard_rows, st["inter"]), dtype=torch.bfloat16, device=dev)
    ctx.recv_i = ctx.recv_i_raw[:cap]
    ctx.counts_all = torch.zeros((ctx.world, ctx.n_experts), dtype=torch.int32, device=dev)
    ctx.dest_base = torch.zeros(ctx.n_experts, dtype=torch.int32, device=dev)
    ctx.group_offsets = torch.zeros(ctx.n_experts + 1, dtype=torch.int32, device=dev)
    return ctx


def moe_stage_peer(h, data, st, ctx: ExpertParallel):
    """Expert-parallel MoE stage over peer memory: dispatch and combine kernels move the rows."""
    cfg = data["config"]
    top_k, status = cfg["top_k"], st["status"]
    peer, local = ctx.peer, ctx.n_experts // ctx.world
    logits = ops.gemm(h, st["router_hilo"], out_mode=OUT_F32, k=h.shape[1], segs=2, a_seg_stride=0,
                      b_seg_stride=h.shape[1], status=status)
    layer._mark(st, "gemm_router")
    ctx.counts.zero_()
    ids, tw, _, slots = ops.route_topk(logits, st["router_bias"], layer.ROUTER_MULTIPLIER, ctx.zero, ctx.n_experts,
                                       top_k, ctx.n_experts, ctx.counts)
    layer._mark(st, "route_topk")
    # The plan and the NVLink-bound dispatch run on a side stream next to the compute-bound shared
    # expert (per-stage timing keeps one stream so that the marks mean something).
    main = torch.cuda.current_stream()
    fork = st.get("marks") is None and bool(st["shared"])
    if fork:
        ctx.side.wait_stream(main)
    with torch.cuda.stream(ctx.side if fork else main):
        if ctx.world > 1:
            dist.all_gather_into_tensor(ctx.counts_all.view(-1), ctx.counts, group=ctx.group)
        else:
            ctx.counts_all.view(-1).copy_(ctx.counts)
        ops.ep_plan(ctx.counts_all, ctx.rank, peer.cap, ctx.dest_base, ctx.group_offsets, status)
        # every rank has finished reading this rank's slab (the previous layer's combine) before new rows land
        ops.peer_barrier(peer.flag_ptrs.data_ptr(), ctx.rank, ctx.world, status)
        layer._mark(st, "plan")
        if st["pooled"]:
            p = ops.gemm(h, st["pooler"], status=status)
            rowmap = ops.dispatch_peer(p, st["w_pre_exp"], ids, slots, ctx.dest_base, peer.slab_ptrs.data_ptr(),
                                       local, peer.cap)
        else:
            rowmap = ops.dispatch_peer(h, None, ids, slots, ctx.dest_base, peer.slab_ptrs.data_ptr(), local,
                                       peer.cap)
        layer._mark(st, "dispatch")
    shared = None
    if st["shared"]:                           # also absorbs the skew between ranks ahead of the barrier
        s_inter = ops.gemm(h, st["shared_w13"], out_mode=OUT_SWIGLU_BF16, status=status)
        shared = ops.gemm(s_inter, st["shared_w2"], status=status)
        layer._mark(st, "shared_expert")
    if fork:
        main.wait_stream(ctx.side)
        rowmap.record_stream(main)             # allocated on the side stream, read on the main one
    ops.peer_barrier(peer.flag_ptrs.data_ptr(), ctx.rank, ctx.world, status)      # all rows have landed
    layer._mark(st, "barrier_rows")
    layer.expert_gemms(peer.slab, ctx.recv_i, ctx.group_offsets, st)      # x -> inter -> y, in place in the slab
    st["offsets"][-1:] = ctx.group_offsets[-1:]             # rows computed on this rank (for the bench's FLOP count)
    ops.peer_barrier(peer.flag_ptrs.data_ptr(), ctx.rank, ctx.world, status)      # all expert outputs are written
    layer._mark(st, "barrier_outputs")
    moe = ops.combine_peer(peer.slab_ptrs.data_ptr(), peer.cap, st["moe_width"], rowmap, tw, st["w_post_exp"],
                           addend=shared)
    layer._mark(st, "combine")
    if st["pooled"]:
        moe = layer.unpool(moe, st)
        layer._mark(st, "gemm_unpooler")
    return moe, ids


def moe_stage(h, data, st, ctx: ExpertParallel):
    """Expert-parallel counterpart of layer.moe_stage."""
    cfg = data["config"]
    top_k, status = cfg["top_k"], st["status"]
    tokens, hidden = h.shape
    logits = ops.gemm(h, st["router_hilo"], out_mode=OUT_F32, k=hidden, segs=2, a_seg_stride=0, b_seg_stride=hidden,
                      status=status)
    layer._mark(st, "gemm_router")
    ctx.counts.zero_()
    # every expert is a dispatch target here: rows come out grouped by global expert
    ids, tw, local_ids, slots = ops.route_topk(logits, st["router_bias"], layer.ROUTER_MULTIPLIER, ctx.zero,
                                               ctx.n_experts, top_k, ctx.n_experts, ctx.counts)
    layer._mark(st, "route_topk")
    send_x, _ = layer._scratch(st, tokens, top_k)
    if st["pooled"]:
        p = ops.gemm(h, st["pooler"], status=status)
        rowmap = ops.dispatch(p, st["w_pre_exp"], local_ids, slots, ctx.counts, send_x, ctx.send_offsets, status)
    else:
        rowmap = ops.dispatch(h, None, local_ids, slots, ctx.counts, send_x, ctx.send_offsets, status)
    layer._mark(st, "dispatch")
    # The split sizes travel to the host on a side stream; the row exchange then runs on that side
    # stream too, while the main stream computes the shared expert, which does not depend on the
    # routing.  The host wait (one event) does not drain the main stream.
    main = torch.cuda.current_stream()
    ctx.side.wait_stream(main)
    with torch.cuda.stream(ctx.side):
        pending = begin_plan(ctx.counts, ctx.world, ctx.group)
    plan = finish_plan(pending)
    recv_x, recv_i = ctx.buffers(st, max(plan.recv_rows, 1))
    with torch.cuda.stream(ctx.side):
        exchange_rows(send_x, plan.recv_rows, plan.send_splits, plan.recv_splits, out=recv_x, group=ctx.group)
    shared = None
    if st["shared"]:
        s_inter = ops.gemm(h, st["shared_w13"], out_mode=OUT_SWIGLU_BF16, status=status)
        shared = ops.gemm(s_inter, st["shared_w2"], status=status)
        layer._mark(st, "shared_expert")
    main.wait_stream(ctx.side)
    layer._mark(st, "a2a_dispatch")
    rows = max(plan.recv_rows, 1)
    layer.expert_gemms(recv_x[:rows], recv_i[:rows], plan.group_offsets, st)
    st["offsets"][-1:] = plan.group_offsets[-1:]            # rows computed on this rank (for the bench's FLOP count)
    exchange_rows(recv_x[:plan.recv_rows], tokens * top_k, plan.recv_splits, plan.send_splits, out=send_x,
                  group=ctx.group)
    layer._mark(st, "a2a_combine")
    moe = ops.combine(send_x, rowmap, tw, st["w_post_exp"], addend=shared, status=status)
    layer._mark(st, "combine")
    if st["pooled"]:
        moe = layer.unpool(moe, st)
        layer._mark(st, "gemm_unpooler")
    return moe, ids


class ChunkedSequence:
    """One sequence prefilled in pieces on several ranks in the same layer call (context parallel).
    Piece p, `lens[p]` tokens long, covers positions [sum(lens[:p]), +lens[p]) and runs on rank
    `owners[p]` of `group`; a rank gives its pieces, in increasing order, as separate requests whose
    cached context (`seq_lens[b]`) is the sum of all earlier pieces.  The earlier pieces' K/V rows do
    not exist in a request's pages until their owners have computed them in the same layer:
    `kv_handoff` brings them over.  `owners` defaults to one piece per rank in order; giving rank c the
    pieces c and 2 W - 1 - c (`zigzag_owners`) balances the causal attention work.
    The reference stands a synthetic cached context in for this (reference.py:195-224)."""

    def __init__(self, group, index: int, lens, hkv: int, head_dim: int, device, owners=None):
        self.group, self.index, self.lens = group, index, [int(n) for n in lens]
        self.owners = list(range(len(self.lens))) if owners is None else [int(o) for o in owners]
        if len(self.owners) != len(self.lens):
            raise ValueError("one owner per piece")
        self.world = max(self.owners) + 1
        self.starts = [sum(self.lens[:p]) for p in range(len(self.lens))]
        self.mine = [p for p, o in enumerate(self.owners) if o == index]          # this rank's requests
        # offset of piece p among its owner's tokens (requests are laid out in piece order)
        self.offset_in_owner = []
        seen = [0] * self.world
        for p, o in enumerate(self.owners):
            self.offset_in_owner.append(seen[o])
            seen[o] += self.lens[p]
        self.row_bytes = hkv * head_dim
        most = max(seen)
        self.most = most
        self.send = torch.empty((2, most, self.row_bytes), dtype=torch.uint8, device=device)
        self.recv = torch.empty((self.world, 2, most, self.row_bytes), dtype=torch.uint8, device=device)
        self._plans = {}

    def plan(self, page: int):
        """Index tensors of the hand-off, which depend on the sizes only and are built once per page
        size: for each of this rank's requests with a cached context, (page number and offset in the
        page of every context position, and for K and V the row of the receive buffer - viewed as
        [world * 2 * most, row_bytes] - that holds that position's row)."""
        if page not in self._plans:
            dev = self.recv.device
            out = []
            for p in self.mine:
                ctx_len = self.starts[p]
                if ctx_len == 0:
                    out.append(None)
                    continue
                pos = torch.arange(ctx_len, device=dev)
                src = [torch.cat([(self.owners[q] * 2 + which) * self.most + self.offset_in_owner[q]
                                  + torch.arange(self.lens[q], device=dev) for q in range(p)])
                       for which in range(2)]
                out.append((pos // page, pos % page, src[0], src[1]))
            self._plans[page] = out
        return self._plans[page]


def zigzag_owners(ranks: int):
    """Owners of 2 * ranks pieces: rank c takes pieces c and 2 * ranks - 1 - c."""
    return list(range(ranks)) + list(range(ranks - 1, -1, -1))


def kv_handoff(data: dict, st: dict, seq: ChunkedSequence):
    """After this rank's new K/V rows are in its paged cache: all-gather the new rows of every rank of
    the sequence, then, for each of this rank's requests, scatter the rows of all earlier pieces into
    the slots the request's page table gives their positions."""
    cfg = data["config"]
    if cfg["batch"] != len(seq.mine):
        raise ValueError("a rank's requests must be its pieces of the sequence, in order")
    n_mine = sum(seq.lens[p] for p in seq.mine)
    caches = [data[k].view(torch.uint8).view(-1, seq.row_bytes) for k in ("k_cache", "v_cache")]
    for which, cache in enumerate(caches):
        ops.kv_rows_copy(cache, seq.send[which], n_mine, src_idx=data["cache_loc"], status=st["status"])
    if seq.world > 1:
        dist.all_gather_into_tensor(seq.recv.view(-1), seq.send.view(-1), group=seq.group)
    else:
        seq.recv.view(-1).copy_(seq.send.view(-1))         # every piece runs on this rank
    page = cfg["page_size"]
    recv_rows = seq.recv.view(-1, seq.row_bytes)
    for b, plan in enumerate(seq.plan(page)):
        if plan is None:
            continue
        page_no, page_off, src_k, src_v = plan
        # where the request's page table puts positions 0 .. ctx-1 (the only data-dependent part)
        prefix_loc = data["page_table"][b].long()[page_no] * page + page_off
        for src, cache in zip((src_k, src_v), caches):
            ops.kv_rows_copy(recv_rows, cache, prefix_loc.numel(), src_idx=src, dst_idx=prefix_loc, status=st["status"])


def kernel_fn(data: dict, st: dict, ctx: ExpertParallel, seq: ChunkedSequence = None):
    """Same contract as layer.kernel_fn for this rank's requests; `st` holds this rank's slice of
    the expert banks.  With `seq` this rank's single request is one chunk of a longer sequence whose
    earlier chunks run on other ranks in the same call."""
    o_in = layer.attention_stage(data, st, (lambda: kv_handoff(data, st, seq)) if seq is not None else None)
    a = ops.gemm(o_in, st["o"], status=st["status"])
    layer._mark(st, "gemm_o")
    s1, h = ops.boundary(a, None, data["stream"], st["a1"], st["b1"], st["w_pre_ffn"], layer.POST_NORM_EPS,
                         layer.RMS_EPS)
    layer._mark(st, "boundary_attn")
    f, ids = (moe_stage_peer if ctx.peer is not None else moe_stage)(h, data, st, ctx)
    s2, hidden = ops.boundary(f, st["w_post_ffn"], s1, st["a2"], st["b2"], st["w_next"], layer.POST_NORM_EPS,
                              layer.RMS_EPS)
    layer._mark(st, "boundary_ffn")
    return hidden, s2, ids
