"""Expert parallelism on real GPUs (needs >= 2): every rank runs its own requests, experts are
sharded, rows travel by NCCL all-to-all or - fused into the dispatch and combine kernels - by
stores to and loads from the peers' memory; each rank's output must pass the reference's acceptance
check against the CPU oracle evaluated with ALL experts local."""
import dataclasses
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from muse_spark_open_challenge_b200 import ep, layer, synth
        from oracle import layer_ref as L
        from conftest import to_device
        shape = dataclasses.replace(synth.MID, hidden=1024, hq=8, hkv=2, n_experts=16, local_experts=16,
                                    moe_width=1024, inter=256, shared_inter=512)
        weights = synth.make_weights(shape, seed=5)                      # identical on every rank
        data = synth.make_input(shape, [150 + 40 * rank, 77], [30, 0], seed=20 + rank, page=64, kv_scale=0.5)
        local = shape.n_experts // world
        mine = dict(weights)
        for k in ("w13", "w13_sf", "w13_gs", "w2", "w2_sf", "w2_gs"):
            mine[k] = weights[k][rank * local:(rank + 1) * local]
        st = layer.prepare(to_device(mine, f"cuda:{rank}"))
        ctx = ep.ExpertParallel(st, world, rank, shape.n_experts)
        dev = to_device(data, f"cuda:{rank}")
        hidden, stream, ids = ep.kernel_fn(dev, st, ctx)
        hidden2, stream2, ids2 = ep.kernel_fn(dev, st, ctx)             # repeatable
        torch.cuda.synchronize()
        layer.check_status(st)
        assert torch.equal(hidden, hidden2) and torch.equal(ids, ids2)
        d = L.dims_of(weights, data["config"])
        slots = L.new_slots(data).cuda()
        k_rows = dev["k_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
        v_rows = dev["v_cache"].view(-1, d.hkv, d.head_dim)[slots].cpu()
        ok, msg, _ = L.check_layer(data, weights, hidden.cpu(), stream.cpu(), ids.cpu(), k_rows, v_rows)
        assert ok, f"rank {rank}: {msg}"
        # peer-memory transport: same rows in the same order through the same GEMMs; only the combine
        # kernel differs (it sums the same terms with another association), so ids are equal and the
        # outputs agree to fp32 rounding of a bf16 result
        ep.enable_peer(ctx, st, max_tokens=hidden.shape[0], top_k=shape.top_k)
        for _ in range(3):                                               # slab reuse across layers
            hidden3, stream3, ids3 = ep.kernel_fn(dev, st, ctx)
        torch.cuda.synchronize()
        layer.check_status(st)
        assert torch.equal(ids3, ids), f"rank {rank}: peer transport changed the routing"
        assert L.relative_l2(stream3, stream) < 1e-5 and L.relative_l2(hidden3.float(), hidden.float()) < 2e-3, \
            f"rank {rank}: peer transport differs"
        # a slab physically too small for the routing: reported, the rows that do not fit are dropped, and
        # neither the guard rows behind the slab and the intermediate buffer nor the flag words are touched
        tight = ep.ExpertParallel(st, world, rank, shape.n_experts)
        ep.enable_peer(tight, st, max_tokens=hidden.shape[0], top_k=shape.top_k, cap_rows=256, guard_rows=4096)
        tight.peer.guard.fill_(0x5A)
        tight.recv_i_raw[256:].fill_(3.0)
        dist.barrier()
        ep.kernel_fn(dev, st, tight)
        torch.cuda.synchronize()
        dist.barrier()
        with pytest.raises(Exception, match="out of range"):
            layer.check_status(st)
        st["status"].zero_()
        assert int(tight.group_offsets.max()) == 256
        assert bool((tight.peer.guard == 0x5A).all()) and bool((tight.recv_i_raw[256:] == 3.0).all())
        assert tight.peer.flags[:world + 1].tolist() == [3] * (world + 1)
        dist.barrier()
        # One sequence prefilled as two chunks, one per rank: the second rank's cached context is the
        # first rank's new K/V rows, handed over inside the layer call.
        lens = [190, 131]
        cdata = synth.make_input(shape, [lens[rank]], [sum(lens[:rank])], seed=50 + rank, page=64, kv_scale=0.5,
                                 fill_cache=False)
        cdev = to_device(cdata, f"cuda:{rank}")
        seq = ep.ChunkedSequence(None, rank, lens, shape.hkv, shape.head_dim, f"cuda:{rank}")
        c_hidden, c_stream, c_ids = ep.kernel_fn(cdev, st, ctx, seq)
        torch.cuda.synchronize()
        layer.check_status(st)
        c_slots = L.new_slots(cdata).cuda()
        rows = lambda name, idx: cdev[name].view(torch.uint8).view(-1, d.hkv * d.head_dim)[idx]   # noqa: E731
        mine = torch.zeros((2, max(lens), d.hkv * d.head_dim), dtype=torch.uint8, device=f"cuda:{rank}")
        mine[0, :lens[rank]], mine[1, :lens[rank]] = rows("k_cache", c_slots), rows("v_cache", c_slots)
        both = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(both, mine)
        if rank == 1:
            page, pos = 64, torch.arange(lens[0], device="cuda:1")
            prefix = cdev["page_table"][0].long()[pos // page] * page + pos % page
            assert torch.equal(rows("k_cache", prefix), both[0][0, :lens[0]]), "handed-over K rows differ"
            assert torch.equal(rows("v_cache", prefix), both[0][1, :lens[0]]), "handed-over V rows differ"
        after = dict(cdata)
        after["k_cache"], after["v_cache"] = cdev["k_cache"].cpu(), cdev["v_cache"].cpu()
        kc = cdev["k_cache"].view(-1, d.hkv, d.head_dim)[c_slots].cpu()
        vc = cdev["v_cache"].view(-1, d.hkv, d.head_dim)[c_slots].cpu()
        ok, msg, _ = L.check_layer(after, weights, c_hidden.cpu(), c_stream.cpu(), c_ids.cpu(), kc, vc)
        assert ok, f"rank {rank} (chunk {rank} of a split sequence): {msg}"
        dist.barrier()
        # The same with four pieces in zigzag order (rank 0: pieces 0 and 3, rank 1: pieces 1 and 2), two
        # requests per rank: balances the causal attention work between the ranks.
        lens4, owners = [70, 45, 83, 52], ep.zigzag_owners(world)
        starts4 = [sum(lens4[:p]) for p in range(4)]
        my = [p for p, o in enumerate(owners) if o == rank]
        zdata = synth.make_input(shape, [lens4[p] for p in my], [starts4[p] for p in my], seed=70 + rank, page=16,
                                 kv_scale=0.5, fill_cache=False)
        zdev = to_device(zdata, f"cuda:{rank}")
        zseq = ep.ChunkedSequence(None, rank, lens4, shape.hkv, shape.head_dim, f"cuda:{rank}", owners=owners)
        z_hidden, z_stream, z_ids = ep.kernel_fn(zdev, st, ctx, zseq)
        torch.cuda.synchronize()
        layer.check_status(st)
        z_slots = L.new_slots(zdata).cuda()
        zafter = dict(zdata)
        zafter["k_cache"], zafter["v_cache"] = zdev["k_cache"].cpu(), zdev["v_cache"].cpu()
        zk = zdev["k_cache"].view(-1, d.hkv, d.head_dim)[z_slots].cpu()
        zv = zdev["v_cache"].view(-1, d.hkv, d.head_dim)[z_slots].cpu()
        ok, msg, _ = L.check_layer(zafter, weights, z_hidden.cpu(), z_stream.cpu(), z_ids.cpu(), zk, zv)
        assert ok, f"rank {rank} (pieces {my} of a zigzag-split sequence): {msg}"
        # every cached context row of a request must be a row some rank computed: none left at zero
        for b, p in enumerate(my):
            if starts4[p]:
                pos = torch.arange(starts4[p], device=f"cuda:{rank}")
                loc = zdev["page_table"][b].long()[pos // 16] * 16 + pos % 16
                got = zdev["k_cache"].view(torch.uint8).view(-1, d.hkv * d.head_dim)[loc]
                assert bool((got != 0).any(dim=1).all()), f"rank {rank}: piece {p} has unfilled context rows"
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_layer_matches_oracle_on_two_gpus():
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
