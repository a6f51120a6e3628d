"""Two-GPU checks of the sharding layer with the real operators over NCCL: expert-parallel MoE against the
single-GPU layer, column- and row-parallel W4A16 linears against the unsharded one.  Skipped on one GPU."""

import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import torch.distributed as dist

    from emmy_b200 import ops, ops_moe as om, shard
    from oracle import synth
    from tests.test_gpu_moe import make_experts

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        e, h, inter, k, t = 8, 256, 128, 2, 40
        ex = make_experts(e, h, inter, seed=3)
        full = om.moe_repack(tuple(dev(a) for a in ex["gate_up"]), tuple(dev(a) for a in ex["down"]))
        per = e // world
        mine = slice(rank * per, (rank + 1) * per)
        local = om.moe_repack(tuple(dev(a[mine]) for a in ex["gate_up"]), tuple(dev(a[mine]) for a in ex["down"]))
        x = torch.from_numpy(synth.activations(t, h, "bf16", seed=50 + rank)).bfloat16().cuda()
        logits = torch.randn(t, e, generator=torch.Generator().manual_seed(60 + rank)).cuda()
        ref = om.moe_forward(x, logits, full, k).float()
        ids, scores = om.moe_route(logits, k)
        y = shard.ep_moe_forward(x, ids, scores, e, lambda rows, eid: om.moe_experts(rows, eid, local),
                                 lambda out_rows, sc: om.moe_combine(out_rows, sc, k)).float()
        ret[rank] = float((y - ref).abs().max() / ref.abs().max())

        # the same layer with the exchange done by the kernels over peer memory, twice (the epoch flags must carry over)
        ep = shard.EpMoe(None, 300, k, h, inter, per, torch.bfloat16, torch.device("cuda", rank))
        y1 = ep.forward(x, ids, scores, local).float()
        ep.status()
        ret[30 + rank] = float((y1 - ref).abs().max() / ref.abs().max())
        t2 = 300 - 7 * rank  # ranks need not hold the same number of tokens
        x2 = torch.from_numpy(synth.activations(t2, h, "bf16", seed=70 + rank)).bfloat16().cuda()
        logits2 = torch.randn(t2, e, generator=torch.Generator().manual_seed(80 + rank)).cuda()
        ref2 = om.moe_forward(x2, logits2, full, k).float()
        ids2, scores2 = om.moe_route(logits2, k)
        y2 = ep.forward(x2, ids2, scores2, local).float()
        ep.status()
        ret[40 + rank] = float((y2 - ref2).abs().max() / ref2.abs().max())

        # the pipelined form: three slices on three streams, each a complete exchange; twice, the second time with
        # fewer tokens than slices can be filled with (the last slice is empty on one rank)
        pipe = shard.EpMoePipelined(None, 300, k, h, inter, per, torch.bfloat16, torch.device("cuda", rank), chunks=3)
        y3 = pipe.forward(x2, ids2, scores2, local, check=True).float()
        ret[50 + rank] = float((y3 - ref2).abs().max() / ref2.abs().max())
        t3 = 150 if rank == 0 else 230
        y4 = pipe.forward(x2[:t3], ids2[:t3], scores2[:t3], local, check=True).float()
        ret[60 + rank] = float((y4 - ref2[:t3]).abs().max() / ref2[:t3].abs().max())

        # many experts, few tokens: the receive side runs eight-row blocks through the streaming tier
        e2, t4 = 64, 12
        ex2 = make_experts(e2, h, inter, seed=5)
        full2 = om.moe_repack(tuple(dev(a) for a in ex2["gate_up"]), tuple(dev(a) for a in ex2["down"]))
        per2 = e2 // world
        mine2 = slice(rank * per2, (rank + 1) * per2)
        local2 = om.moe_repack(tuple(dev(a[mine2]) for a in ex2["gate_up"]), tuple(dev(a[mine2]) for a in ex2["down"]))
        x4 = torch.from_numpy(synth.activations(t4, h, "bf16", seed=90 + rank)).bfloat16().cuda()
        logits4 = torch.randn(t4, e2, generator=torch.Generator().manual_seed(95 + rank)).cuda()
        ref4 = om.moe_forward(x4, logits4, full2, k).float()
        ids4, scores4 = om.moe_route(logits4, k)
        ep2 = shard.EpMoe(None, 16, k, h, inter, per2, torch.bfloat16, torch.device("cuda", rank))
        for _ in range(2):
            y5 = ep2.forward(x4, ids4, scores4, local2, check=True).float()
        ret[70 + rank] = float((y5 - ref4).abs().max() / ref4.abs().max())

        kk, n = 512, 256
        qw, qz, sc, gi = synth.gptq_linear(kk, n, seed=9)
        tq = [torch.from_numpy(a) for a in (qw, qz, sc, gi)]
        xx = torch.from_numpy(synth.activations(5, kk, "f16", seed=4)).half().cuda()
        whole = ops.w4a16_linear(xx, ops.w4_repack(*(a.cuda() for a in tq[:3]), 128, "gptq", g_idx=tq[3].cuda())).float()
        a, b, c, g = shard.column_slice_w4("gptq", *tq, rank, world)
        wcol = ops.w4_repack(a.cuda(), b.cuda(), c.cuda(), 128, "gptq", g_idx=g.cuda())
        ycol = shard.ColumnParallelLinear(lambda v: ops.w4a16_linear(v, wcol))(xx, gather=True).float()
        ret[10 + rank] = float((ycol - whole).abs().max() / whole.abs().max())
        a, b, c, g, rows = shard.row_slice_w4("gptq", *tq, 128, rank, world)
        wrow = ops.w4_repack(a.cuda(), b.cuda(), c.cuda(), 128, "gptq", g_idx=g.cuda())
        yrow = shard.RowParallelLinear(lambda v: ops.w4a16_linear(v, wrow), rows)(xx).float()
        ret[20 + rank] = float((yrow - whole).abs().max() / whole.abs().max())

        # the same sum by the peer-memory kernel: five calls (both buffer slots, reuse of each), then a larger bf16
        # result against the process group's f32 all-reduce, bit-identical on every rank, and replayed from a CUDA graph
        ar = shard.PeerAllReduce(None, 48 * 4096, torch.device("cuda", rank))
        rp = shard.RowParallelLinear(lambda v: ops.w4a16_linear(v, wrow), rows, reducer=ar)
        for _ in range(5):
            ypeer = rp(xx)
        ar.status()
        ret[80 + rank] = float((ypeer.float() - yrow).abs().max() / whole.abs().max())
        part = torch.randn(48, 4096, generator=torch.Generator().manual_seed(40 + rank)).bfloat16().cuda()
        assert ar.fits(part) and not ar.fits(torch.empty(49, 4096, dtype=torch.bfloat16, device="cuda"))
        want = part.float()
        dist.all_reduce(want)
        got = ar(part, check=True)
        ret[90 + rank] = float((got.float() - want).abs().max() / want.abs().max())
        theirs = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(theirs, got)
        ret[100 + rank] = float(sum((t != got).sum().item() for t in theirs))
        out = torch.empty_like(part)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ar(part, out=out)  # warm-up on the capture stream
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                ar(part, out=out)
            for _ in range(3):
                out.zero_()
                graph.replay()
            ar.status()
        torch.cuda.current_stream().wait_stream(side)
        ret[110 + rank] = float((out != got).sum().item())
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_paths_on_two_gpus():
    import torch.multiprocessing as mp

    world = 2
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
        out = dict(ret)
    assert all(out[r] < 1e-2 for r in range(world)), out            # EP == single device up to f32 summation order
    assert all(out[30 + r] < 1e-2 and out[40 + r] < 1e-2 for r in range(world)), out  # peer-memory exchange
    assert all(out[50 + r] < 1e-2 and out[60 + r] < 1e-2 for r in range(world)), out  # the same, sliced over streams
    assert all(out[70 + r] < 1e-2 for r in range(world)), out                          # streaming tier on the receive side
    assert all(out[10 + r] == 0.0 for r in range(world)), out      # column shards are the same columns
    assert all(out[20 + r] < 1e-2 for r in range(world)), out      # row partials summed in f32
    assert all(out[80 + r] < 2e-3 for r in range(world)), out      # the peer-memory sum: the same up to the order of the f32 adds
    assert all(out[90 + r] < 1e-2 for r in range(world)), out      # bf16, 48 x 4096, against the f32 all-reduce
    assert all(out[100 + r] == 0.0 and out[110 + r] == 0.0 for r in range(world)), out  # identical on all ranks, and from a graph
