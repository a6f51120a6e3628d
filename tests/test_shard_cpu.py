"""The sharding layer on CPU: slicing identities, and the expert-parallel / row-parallel exchange over two gloo
ranks with the oracle as the compute step."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from emmy_b200 import shard
from oracle import formats as fm
from oracle import moe as omoe
from oracle import synth


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_column_slices_concatenate_to_the_whole():
    for fmt in ("awq", "gptq"):
        if fmt == "awq":
            qw, qz, sc = synth.awq_linear(256, 128, seed=1)
            gi = None
        else:
            qw, qz, sc, gi = synth.gptq_linear(256, 128, seed=1)
        whole = fm.dequant_w4(qw, qz, sc, 128, fmt, gi)
        parts = []
        for r in range(4):
            a, b, c, g = shard.column_slice_w4(fmt, torch.from_numpy(qw), torch.from_numpy(qz), torch.from_numpy(sc),
                                               None if gi is None else torch.from_numpy(gi), r, 4)
            parts.append(fm.dequant_w4(a.numpy(), b.numpy(), c.numpy(), 128, fmt, None if g is None else g.numpy()))
        np.testing.assert_array_equal(np.concatenate(parts, axis=1), whole)


def test_row_slices_sum_to_the_whole_product():
    x = synth.activations(3, 512, "f16", seed=2).astype(np.float64)
    for fmt in ("awq", "gptq"):
        if fmt == "awq":
            qw, qz, sc = synth.awq_linear(512, 64, seed=3)
            gi = None
        else:
            qw, qz, sc, gi = synth.gptq_linear(512, 64, seed=3)
        whole = x @ fm.dequant_w4(qw, qz, sc, 128, fmt, gi).astype(np.float64)
        acc = np.zeros_like(whole)
        for r in range(2):
            a, b, c, g, rows = shard.row_slice_w4(fmt, torch.from_numpy(qw), torch.from_numpy(qz), torch.from_numpy(sc),
                                                  None if gi is None else torch.from_numpy(gi), 128, r, 2)
            w = fm.dequant_w4(a.numpy(), b.numpy(), c.numpy(), 128, fmt, None if g is None else g.numpy())
            acc += x[:, rows] @ w.astype(np.float64)
        np.testing.assert_allclose(acc, whole, rtol=1e-12, atol=1e-12)


def test_fp8_and_nvfp4_column_slices():
    bits, s = synth.fp8_weight(64, 128, seed=0)
    packed, sb, s2 = synth.nvfp4_weight(64, 128, seed=0)
    fp8_parts, fp4_parts = [], []
    for r in range(2):
        wb, ws = shard.column_slice_fp8(torch.from_numpy(bits), torch.from_numpy(s), r, 2)
        fp8_parts.append(fm.dequant_fp8(wb.numpy(), ws.numpy().reshape(-1, 1)))
        p, q, g = shard.column_slice_nvfp4(torch.from_numpy(packed), torch.from_numpy(sb), torch.from_numpy(s2), r, 2)
        fp4_parts.append(fm.dequant_nvfp4(p.numpy(), q.numpy(), g.numpy()))
    np.testing.assert_array_equal(np.concatenate(fp8_parts), fm.dequant_fp8(bits, s))
    np.testing.assert_array_equal(np.concatenate(fp4_parts), fm.dequant_nvfp4(packed, sb, s2))


def test_slicing_errors():
    qw, qz, sc = synth.awq_linear(256, 48, seed=1)
    with pytest.raises(ValueError):
        shard.column_slice_w4("awq", torch.from_numpy(qw), torch.from_numpy(qz), torch.from_numpy(sc), None, 0, 2)
    with pytest.raises(ValueError):
        shard.row_slice_w4("awq", torch.from_numpy(qw), torch.from_numpy(qz), torch.from_numpy(sc), None, 128, 0, 4)
    with pytest.raises(ValueError):
        shard.expert_owner(torch.tensor([1]), 10, 4)


def test_reference_intermediate_slices_sum_to_the_whole_expert():
    """tests/serving/test_expert_sharding.py:49-70: the per-rank partials of the reference's slicing add up."""
    g = torch.Generator().manual_seed(0)
    h, inter, world = 32, 16, 4
    w_gate_up = torch.randn(2 * inter, h, generator=g, dtype=torch.float64)
    w_down = torch.randn(h, inter, generator=g, dtype=torch.float64)
    x = torch.randn(5, h, generator=g, dtype=torch.float64)
    whole = omoe.expert_ffn(x, w_gate_up, w_down)
    parts = sum(
        omoe.expert_ffn(x, omoe.tp_expert_slice("w_gate_up", w_gate_up, r, world),
                        omoe.tp_expert_slice("w_down", w_down, r, world))
        for r in range(world)
    )
    torch.testing.assert_close(parts, whole, rtol=1e-5, atol=1e-5)
    scale = torch.ones(h, 1)  # a scale broadcast along the intermediate axis stays whole on every rank
    assert omoe.tp_expert_slice("w_down_scale", scale, 1, world) is scale


def test_single_row_path_equals_batch_path():
    """tests/serving/test_expert_sharding.py:101-165: routing a batch row by row gives bit for bit what routing the
    batch at once gives (the combine adds each row's picks in ascending expert order whatever else is in the batch)."""
    g = torch.Generator().manual_seed(3)
    e, h, inter, k, t = 8, 32, 16, 3, 7
    w_gu = (torch.randn(e, 2 * inter, h, generator=g) * 0.2).bfloat16()
    w_dn = (torch.randn(e, h, inter, generator=g) * 0.2).bfloat16()
    x = torch.randn(t, h, generator=g).bfloat16()
    logits = torch.randn(t, e, generator=g)
    whole = omoe.moe_layer(x, logits, w_gu, w_dn, k)
    rows = torch.cat([omoe.moe_layer(x[r : r + 1], logits[r : r + 1], w_gu, w_dn, k) for r in range(t)])
    assert torch.equal(whole, rows)
    # and the stacked form of the reference's slicing agrees with slicing expert by expert
    stacked = omoe.tp_expert_slice("w_gate_up", w_gu, 1, 2, stacked=True)
    assert torch.equal(stacked[3], omoe.tp_expert_slice("w_gate_up", w_gu[3], 1, 2))


def test_ep_default_cap_arithmetic():
    """The opt-in smaller receive capacity: twice the balanced share plus slack, never more than all picks."""
    assert shard.EpMoe.default_cap(4096, 8, 8) == 2 * 4096 * 8 // 8 + 256
    assert shard.EpMoe.default_cap(4, 8, 2) == 32  # small calls: all picks
    # a skewed routing that sends everything to one rank exceeds it; the default cap (all picks) cannot be exceeded
    picks = 4096 * 8
    assert picks > shard.EpMoe.default_cap(4096, 8, 8)


def _ep_worker(rank, world, port, e, h, inter, k, t, ret):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1)
        w_gu = torch.randn(e, 2 * inter, h, generator=g) * 0.1
        w_dn = torch.randn(e, h, inter, generator=g) * 0.1
        gt = torch.Generator().manual_seed(100 + rank)  # every rank has its own tokens
        x = torch.randn(t, h, generator=gt)
        logits = torch.randn(t, e, generator=gt)
        scores, ids = omoe.route_softmax_topk(logits, k)
        ids, by = ids.sort(dim=1, stable=True)
        scores = scores.gather(1, by)
        per = e // world
        lo = rank * per

        def experts_fn(rows, local_eid):
            out = torch.empty_like(rows)
            for le in torch.unique(local_eid).tolist():
                sel = (local_eid == le).nonzero().squeeze(1)
                out[sel] = omoe.expert_ffn(rows[sel], w_gu[lo + le], w_dn[lo + le])
            return out

        def combine_fn(out_rows, sc):
            return (out_rows.view(t, k, -1).float() * sc.unsqueeze(-1)).sum(dim=1)

        y = shard.ep_moe_forward(x, ids, scores, e, experts_fn, combine_fn)
        ref = omoe.moe_layer(x, logits, w_gu, w_dn, k)
        ret[rank] = float((y - ref).abs().max() / ref.abs().max())

        # row-parallel linear: partial products summed by all-reduce
        w = torch.randn(h, 24, generator=g, dtype=torch.float64)
        xx = torch.randn(3, h, generator=g, dtype=torch.float64)
        rows = slice(rank * h // world, (rank + 1) * h // world)
        rp = shard.RowParallelLinear(lambda xs: xs @ w[rows], rows, reduce_dtype=torch.float64)
        ret[10 + rank] = float((rp(xx) - xx @ w).abs().max())

        # a reducer takes the sum when the result fits it (here a stand-in built on the group's all-reduce that counts
        # its calls), the group's all-reduce otherwise; `sliced` inputs and `out=` on both routes
        class CountingReducer:
            calls = 0

            def __init__(self, limit):
                self.limit = limit

            def fits(self, partial):
                return partial.numel() <= self.limit

            def __call__(self, partial, out=None):
                CountingReducer.calls += 1
                acc = partial.clone()
                dist.all_reduce(acc)
                if out is None:
                    return acc
                out.copy_(acc)
                return out

        small = shard.RowParallelLinear(lambda xs: xs @ w[rows], rows, reduce_dtype=torch.float64, reducer=CountingReducer(3 * 24))
        big = shard.RowParallelLinear(lambda xs: xs @ w[rows], rows, reduce_dtype=torch.float64, reducer=CountingReducer(3 * 24 - 1))
        out = torch.empty(3, 24, dtype=torch.float64)
        err = float((small(xx[:, rows].contiguous(), sliced=True, out=out) - xx @ w).abs().max())
        took = CountingReducer.calls
        err = max(err, float((big(xx, out=out) - xx @ w).abs().max()), float((out - xx @ w).abs().max()))
        ret[30 + rank] = err if (took == 1 and CountingReducer.calls == 1) else 1.0
        cp = shard.ColumnParallelLinear(lambda xs: xs @ w[:, rank * 12 : (rank + 1) * 12])
        ret[20 + rank] = float((cp(xx, gather=True) - xx @ w).abs().max())
    finally:
        dist.destroy_process_group()


def test_expert_parallel_and_row_parallel_over_two_gloo_ranks():
    world = 2
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_ep_worker, args=(world, port, 8, 16, 8, 2, 11, ret), nprocs=world, join=True)
        assert all(ret[r] < 1e-5 for r in range(world)), dict(ret)
        assert all(ret[10 + r] < 1e-12 and ret[20 + r] < 1e-12 for r in range(world)), dict(ret)
        assert all(ret[30 + r] < 1e-12 for r in range(world)), dict(ret)  # reducer route and fallback agree
