"""MoE on W4A16 experts on the GPU against the CPU torch oracle, through the C ABI."""

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from oracle import synth

pytestmark = pytest.mark.gpu
TOL = 2e-2


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_experts(e, h, inter, seed=0):
    gu, dn = [], []
    for i in range(e):
        gu.append(synth.awq_linear(h, 2 * inter, seed=seed + 2 * i))
        dn.append(synth.awq_linear(inter, h, seed=seed + 2 * i + 1))
    stack = lambda parts, j: np.stack([p[j] for p in parts])
    gate_up = tuple(stack(gu, j) for j in range(3))
    down = tuple(stack(dn, j) for j in range(3))
    return {"gate_up": gate_up, "down": down}


def test_router_matches_oracle_and_breaks_ties_low():
    from emmy_b200 import ops_moe as om

    g = torch.Generator().manual_seed(0)
    logits = torch.randn(50, 128, generator=g)
    logits[3, 7] = logits[3, 90] = logits[3].max() + 1.0  # a tie at the top
    logits[4, :] = 0.25  # all equal: picks 0..7
    ids, scores = om.moe_route(logits.cuda(), 8)
    ref_s, ref_i = omoe.route_softmax_topk(logits, 8)
    ref_i_sorted, order = ref_i.sort(dim=1, stable=True)
    ref_s_sorted = ref_s.gather(1, order)
    np.testing.assert_array_equal(ids.cpu().numpy(), ref_i_sorted.numpy().astype(np.int32))
    np.testing.assert_allclose(scores.cpu().numpy(), ref_s_sorted.numpy(), rtol=2e-6, atol=1e-8)
    assert ids[4].tolist() == list(range(8)) and 7 in ids[3].tolist() and 90 in ids[3].tolist()
    np.testing.assert_allclose(scores.sum(dim=1).cpu().numpy(), 1.0, rtol=1e-5)


def test_experts_grouped_ffn_matches_per_expert_eager():
    from emmy_b200 import ops_moe as om

    e, h, inter = 8, 256, 128
    ex = make_experts(e, h, inter, seed=10)
    w = om.moe_repack(tuple(dev(a) for a in ex["gate_up"]), tuple(dev(a) for a in ex["down"]))
    wgu, wdn = omoe.dequant_expert_weights(ex, torch.bfloat16)
    rng = np.random.default_rng(0)
    r = 37
    x = torch.from_numpy(synth.activations(r, h, "bf16", seed=3)).bfloat16()
    eid = torch.from_numpy(rng.integers(0, e, r).astype(np.int32))
    eid[:3] = 5  # an expert with several rows, some with none
    out = om.moe_experts(x.cuda(), eid.cuda(), w).float().cpu()
    ref = torch.stack([omoe.expert_ffn(x[i : i + 1], wgu[int(eid[i])], wdn[int(eid[i])])[0] for i in range(r)]).float()
    assert float((out - ref).abs().max()) <= TOL * float(ref.abs().max())


@pytest.mark.parametrize("t", [1, 5, 64, 300])
def test_moe_layer_matches_oracle(t):
    from emmy_b200 import ops_moe as om

    e, h, inter, k = 16, 256, 128, 4
    ex = make_experts(e, h, inter, seed=100)
    w = om.moe_repack(tuple(dev(a) for a in ex["gate_up"]), tuple(dev(a) for a in ex["down"]))
    wgu, wdn = omoe.dequant_expert_weights(ex, torch.bfloat16)
    x = torch.from_numpy(synth.activations(t, h, "bf16", seed=t)).bfloat16()
    logits = torch.randn(t, e, generator=torch.Generator().manual_seed(t))
    ws = om.moe_workspace(t, w, k, torch.device("cuda"))
    y = om.moe_forward(x.cuda(), logits.cuda(), w, k, workspace=ws)
    om.moe_status(ws, t, w, k)
    ref = omoe.moe_layer(x, logits, wgu, wdn, k).float()
    got = y.float().cpu()
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max()) <= TOL * float(ref.abs().max())


def test_moe_layer_qwen3_shapes_decode():
    """128 experts, top-8, hidden 2048, intermediate 768, T = 1: the decode-shaped case at full width."""
    from emmy_b200 import ops_moe as om

    e, h, inter, k, t = 128, 2048, 768, 8, 1
    # weights are drawn once and shared by all experts but eight, to keep the CPU side short
    base = make_experts(2, h, inter, seed=7)
    idx = np.arange(e) % 2
    ex = {key: tuple(a[idx] for a in base[key]) for key in ("gate_up", "down")}
    w = om.moe_repack(tuple(dev(a) for a in ex["gate_up"]), tuple(dev(a) for a in ex["down"]))
    wgu2, wdn2 = omoe.dequant_expert_weights(base, torch.bfloat16)
    x = torch.from_numpy(synth.activations(t, h, "bf16", seed=1)).bfloat16()
    logits = torch.randn(t, e, generator=torch.Generator().manual_seed(5))
    y = om.moe_forward(x.cuda(), logits.cuda(), w, k).float().cpu()
    scores, ids = omoe.route_softmax_topk(logits, k)
    ref = omoe.combine_routed(x, scores, ids, lambda ee, rows: omoe.expert_ffn(x[rows], wgu2[ee % 2], wdn2[ee % 2])).float()
    assert float((y - ref).abs().max()) <= TOL * float(ref.abs().max())


def test_expert_ids_out_of_range_are_reported():
    from emmy_b200 import ops_moe as om
    from emmy_b200.lib import EmmyqError

    e, h, inter = 4, 128, 128
    ex = make_experts(e, h, inter, seed=1)
    w = om.moe_repack(tuple(dev(a) for a in ex["gate_up"]), tuple(dev(a) for a in ex["down"]))
    x = torch.zeros(3, h, dtype=torch.bfloat16, device="cuda")
    ws = om.moe_workspace(3, w, 1, x.device)
    om.moe_experts(x, torch.tensor([0, 9, 1], dtype=torch.int32, device="cuda"), w, workspace=ws)
    with pytest.raises(EmmyqError):
        om.moe_status(ws, 3, w, 1)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_moe_layer_tensor_path_ragged_shapes(dtype):
    """Enough rows per expert for the tcgen05 grouped GEMMs; widths that leave partial column tiles, experts with
    more than one 256-row block and experts with none."""
    from emmy_b200 import ops_moe as om

    e, h, inter, k, t = 8, 640, 384, 2, 1500
    ex = make_experts(e, h, inter, seed=300)
    w = om.moe_repack(tuple(dev(a) for a in ex["gate_up"]), tuple(dev(a) for a in ex["down"]))
    wgu, wdn = omoe.dequant_expert_weights(ex, dtype)
    name = "bf16" if dtype == torch.bfloat16 else "f16"
    x = torch.from_numpy(synth.activations(t, h, name, seed=t)).to(dtype)
    logits = torch.randn(t, e, generator=torch.Generator().manual_seed(t))
    logits[:, 5] = -50.0  # nobody picks expert 5
    logits[:, 2] += 2.0   # expert 2 is crowded
    ws = om.moe_workspace(t, w, k, torch.device("cuda"))
    y = om.moe_forward(x.cuda(), logits.cuda(), w, k, workspace=ws)
    om.moe_status(ws, t, w, k)
    ref = omoe.moe_layer(x, logits, wgu, wdn, k).float()
    got = y.float().cpu()
    assert torch.isfinite(got).all()
    assert float((got - ref).abs().max()) <= TOL * float(ref.abs().max())


def test_expert_parallel_wait_runs_out_and_reports():
    """One rank of a two-rank exchange calls alone: the peer's flag is never raised, the bounded waits run out (about
    a second each), the call returns, and the status word says so.  Both ranks' buffers are local allocations here."""
    import ctypes as C

    from emmy_b200 import lib as L
    from emmy_b200 import ops_moe as om
    from emmy_b200.ops import _DTYPE, _ptr, _stream

    e_local, h, inter, k, t, world = 4, 128, 128, 2, 8, 2
    ex = make_experts(e_local, h, inter, seed=11)
    w = om.moe_repack(tuple(dev(a) for a in ex["gate_up"]), tuple(dev(a) for a in ex["down"]))
    cap = t * k
    bufs = []
    peers = L.EpPeers()
    peers.world, peers.rank, peers.cap = world, 0, cap
    for r in range(world):
        recv_x = torch.zeros(world * cap * h, dtype=torch.bfloat16, device="cuda")
        meta = torch.zeros(world * cap * 2, dtype=torch.int32, device="cuda")
        count = torch.zeros(world * world * e_local, dtype=torch.int32, device="cuda")
        back = torch.zeros(t * k * h, dtype=torch.bfloat16, device="cuda")
        flags = torch.zeros(3 * world, dtype=torch.int32, device="cuda")
        bufs.append((recv_x, meta, count, back, flags))
        peers.recv_x[r], peers.recv_meta[r], peers.recv_count[r] = recv_x.data_ptr(), meta.data_ptr(), count.data_ptr()
        peers.back[r], peers.flags[r] = back.data_ptr(), flags.data_ptr()
    lib = L.load()
    ws = torch.zeros(lib.eq_ep_moe_workspace_bytes(world, cap, e_local, h, inter), dtype=torch.uint8, device="cuda")
    x = torch.randn(t, h, device="cuda").bfloat16()
    ids, scores = om.moe_route(torch.randn(t, e_local * world, device="cuda"), k)
    y = torch.empty(t, h, dtype=torch.bfloat16, device="cuda")
    L.check(lib.eq_ep_moe_w4a16(_ptr(w.gate_up), _ptr(w.down), _DTYPE[w.scale_dtype], e_local, k, h, inter, w.group, _ptr(x), _ptr(ids),
                                _ptr(scores), t, _DTYPE[x.dtype], _ptr(y), C.byref(peers), 0, _ptr(ws), ws.numel(), _stream()))
    with pytest.raises(L.EmmyqError) as err:
        L.check(lib.eq_ep_moe_status(_ptr(ws), world, cap, e_local, h, inter, _stream()))
    assert err.value.status_name == "EQ_ERR_TIMEOUT"
    # the context is still usable
    assert torch.isfinite(om.moe_forward(x, torch.randn(t, e_local, device="cuda"), w, k).float()).all()


def _local_ar_peers(world, rank, cap):
    """eq_ar_peers whose ranks' buffers are all local allocations (single-GPU tests of the peer-memory sum)."""
    from emmy_b200 import lib as L

    lib = L.load()
    peers = L.ArPeers()
    peers.world, peers.rank, peers.cap, peers.max_blocks = world, rank, cap, (cap + 2047) // 2048
    keep = []
    for r in range(world):
        recv = torch.zeros(lib.eq_peer_allreduce_recv_bytes(world, cap), dtype=torch.uint8, device="cuda")
        flags = torch.zeros(lib.eq_peer_allreduce_flag_bytes(world, cap), dtype=torch.uint8, device="cuda")
        keep.append((recv, flags))
        peers.recv[r], peers.flags[r] = recv.data_ptr(), flags.data_ptr()
    state = torch.zeros(lib.eq_peer_allreduce_state_bytes(), dtype=torch.uint8, device="cuda")
    return peers, state, keep


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_peer_allreduce_of_one_rank_is_the_identity(dtype):
    import ctypes as C

    from emmy_b200 import lib as L
    from emmy_b200.ops import _DTYPE, _ptr, _stream

    lib = L.load()
    peers, state, _keep = _local_ar_peers(1, 0, 4096 * 3)
    x = torch.randn(3, 4096, device="cuda").to(dtype)
    y = torch.empty_like(x)
    for _ in range(3):
        L.check(lib.eq_peer_allreduce(C.byref(peers), _ptr(x), x.numel(), _DTYPE[dtype], _ptr(y), _ptr(state), _stream()))
    L.check(lib.eq_peer_allreduce_status(_ptr(state), _stream()))
    assert torch.equal(x, y)
    assert state.view(torch.int32)[1].item() == 3  # the call counter on the device
    with pytest.raises(L.EmmyqError):  # more values than the buffers carry
        L.check(lib.eq_peer_allreduce(C.byref(peers), _ptr(x), 4096 * 3 + 8, _DTYPE[dtype], _ptr(y), _ptr(state), _stream()))


def test_peer_allreduce_wait_runs_out_and_reports():
    """One rank of two calls alone: the peer's flags are never raised, the bounded wait runs out (about a second), the
    call returns and the status word says so.  Both ranks' buffers are local allocations here."""
    import ctypes as C

    from emmy_b200 import lib as L
    from emmy_b200.ops import _DTYPE, _ptr, _stream

    lib = L.load()
    peers, state, _keep = _local_ar_peers(2, 0, 4096)
    x = torch.randn(1, 4096, device="cuda").half()
    y = torch.empty_like(x)
    L.check(lib.eq_peer_allreduce(C.byref(peers), _ptr(x), x.numel(), _DTYPE[x.dtype], _ptr(y), _ptr(state), _stream()))
    with pytest.raises(L.EmmyqError) as err:
        L.check(lib.eq_peer_allreduce_status(_ptr(state), _stream()))
    assert err.value.status_name == "EQ_ERR_TIMEOUT"
    # its own piece did reach the peer's buffer (slot 1 of the first call, source 0), and the context is still usable
    recv1 = _keep[1][0].view(torch.float16).view(2, 2, 4096)
    assert torch.equal(recv1[1, 0], x[0])
    assert torch.isfinite(x.float().sum())
