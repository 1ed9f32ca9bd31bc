"""Expert-parallel exchange logic on CPU ranks (gloo, world size 2 and 4): the plan built from
the per-expert counts, the row all-to-all out and back, and the (source, expert) group order the
grouped GEMM assumes.  The expert computation is replaced by `row * (1 + global expert id)`, so
every route must come back as its token's row times its expert's factor."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_experts, top_k, fail_rank):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from muse_spark_open_challenge_b200 import ep
        g = torch.Generator().manual_seed(100 + rank)
        tokens, width = 37 + 11 * rank, 8
        local = n_experts // world
        x = torch.randn((tokens, width), generator=g)
        ids = torch.stack([torch.randperm(n_experts, generator=g)[:top_k] for _ in range(tokens)])
        if rank == 0:
            ids[:, 0] = n_experts - 1          # skew: everything on rank 0 also goes to the last expert
        # CPU stand-in for route_topk + dispatch: rows ordered by expert, rowmap = row of each route
        flat = ids.flatten()
        order = torch.sort(flat, stable=True).indices
        rowmap = torch.empty_like(order)
        rowmap[order] = torch.arange(order.numel())
        send = x.repeat_interleave(top_k, 0)[order]
        counts = torch.bincount(flat, minlength=n_experts).int()
        plan = ep.make_plan(counts, world)
        assert sum(plan.send_splits) == tokens * top_k
        recv = ep.exchange_rows(send, plan.recv_rows, plan.send_splits, plan.recv_splits)
        # "experts": group g = (source, local expert), source-major; bank = g % local
        offs = plan.group_offsets.tolist()
        assert offs[-1] == plan.recv_rows and len(offs) == world * local + 1
        y = torch.empty_like(recv)
        for grp in range(world * local):
            e_global = rank * local + grp % local
            y[offs[grp]:offs[grp + 1]] = recv[offs[grp]:offs[grp + 1]] * (1 + e_global)
        back = ep.exchange_rows(y, tokens * top_k, plan.recv_splits, plan.send_splits)
        got = back[rowmap].view(tokens, top_k, width)
        want = x[:, None, :] * (1 + ids[:, :, None]).float()
        assert torch.equal(got, want)
        # totals agree across ranks
        tot = torch.tensor([plan.recv_rows, tokens * top_k])
        dist.all_reduce(tot)
        assert tot[0] == tot[1]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_experts,top_k", [(2, 8, 3), (4, 16, 4), (2, 2, 1)])
def test_expert_parallel_exchange_round_trip(world, n_experts, top_k):
    mp.spawn(_worker, args=(world, _free_port(), n_experts, top_k, -1), nprocs=world, join=True)


def test_expert_parallel_context_rejects_bad_geometry():
    from muse_spark_open_challenge_b200 import ep
    st = {"n_local": 4, "device": "cpu"}
    with pytest.raises(ValueError):
        ep.ExpertParallel(st, world=3, rank=0, n_experts=16)
    with pytest.raises(ValueError):
        ep.ExpertParallel(st, world=2, rank=0, n_experts=16)
    ctx = ep.ExpertParallel(st, world=4, rank=1, n_experts=16)
    assert ctx.counts.numel() == 16


def test_chunked_sequence_bookkeeping():
    """Pieces, their owners and where each piece sits among its owner's tokens (host logic only)."""
    from muse_spark_open_challenge_b200 import ep
    assert ep.zigzag_owners(4) == [0, 1, 2, 3, 3, 2, 1, 0]
    lens = [5, 7, 3, 9, 4, 6, 8, 2]
    seqs = [ep.ChunkedSequence(None, r, lens, hkv=2, head_dim=8, device="cpu", owners=ep.zigzag_owners(4))
            for r in range(4)]
    assert [s.mine for s in seqs] == [[0, 7], [1, 6], [2, 5], [3, 4]]
    s = seqs[1]
    assert s.starts == [0, 5, 12, 15, 24, 28, 34, 42]
    # rank 1 holds piece 1 (7 tokens) then piece 6 (8 tokens): piece 6 starts at row 7 of its rows
    assert s.offset_in_owner[1] == 0 and s.offset_in_owner[6] == 7
    assert s.offset_in_owner[0] == 0 and s.offset_in_owner[7] == 5
    # buffers hold the busiest rank's rows, K and V, for every rank
    most = max(lens[p] + lens[7 - p] for p in range(4))
    assert s.send.shape == (2, most, 16) and s.recv.shape == (4, 2, most, 16)
    # default: one piece per rank in order
    plain = ep.ChunkedSequence(None, 2, [4, 4, 4], hkv=1, head_dim=16, device="cpu")
    assert plain.owners == [0, 1, 2] and plain.mine == [2] and plain.starts == [0, 4, 8]
    with pytest.raises(ValueError):
        ep.ChunkedSequence(None, 0, [4, 4], hkv=1, head_dim=16, device="cpu", owners=[0])
