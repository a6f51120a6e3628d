"""Every benchmark shape a throughput figure is quoted on, checked against the CPU oracle through the C ABI.

The full outputs are too large to recompute on the host in a test, so each case checks a random SAMPLE of the output:
some rows of x against some output columns, with the oracle dequantising only those columns (the product of a row
and a column does not depend on the rest).  Weights are drawn with the configurations' distributions; where the host
quantizer would take minutes at full width (FP8, NVFP4: 89 M elements), a block of 1024 quantized output channels is
repeated along N, which changes nothing for the kernels (every row of the weight is streamed and multiplied).
Tolerance: max |err| <= 2e-2 * max |ref| over the sample (the bar the reference's own device tests use for expert
programs, tests/serving/generation/test_gen_runner_gpu.py:833-844; its NVFP4 staged tests hold 1e-3 / 6e-3 on the
weight-only path, tests/compiler/passes/test_nvfp4_staged.py:757-803).
"""

import numpy as np
import pytest
import torch

from oracle import activations as oact
from oracle import linear as ol
from oracle import moe as omoe
from oracle import synth

pytestmark = pytest.mark.gpu
TOL = 2e-2


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def sample(rng, extent, count, unit=1):
    """`count` distinct indices below `extent` in whole units, sorted."""
    blocks = np.sort(rng.choice(extent // unit, size=min(count // unit, extent // unit), replace=False))
    return (blocks[:, None] * unit + np.arange(unit)[None, :]).reshape(-1)


def close(got, ref):
    err = float(np.abs(got - ref).max())
    assert np.isfinite(got).all()
    assert err <= TOL * float(np.abs(ref).max()), f"max err {err:.4g} against max |ref| {float(np.abs(ref).max()):.4g}"


# ---------------------------------------------------------------------------------------------- NVFP4 W4A4 (config #4)


@pytest.fixture(scope="module")
def nvfp4_block():
    return synth.nvfp4_weight(1024, 5120, seed=4)


@pytest.mark.parametrize("m", [1, 128, 2048, 4096])
def test_nvfp4_k5120_n17408(m, nvfp4_block):
    """M = 2048 and 4096 run the 256 x 224 kernel through twenty K steps (its three-stage ring wraps six times)."""
    from emmy_b200 import ops_nvfp4 as o4

    n, k = 17408, 5120
    packed_b, sbits_b, s2 = nvfp4_block
    reps = n // 1024
    packed, sbits = np.tile(packed_b, (reps, 1)), np.tile(sbits_b, (reps, 1))
    x = synth.activations(m, k, "bf16", seed=40 + m)
    s2x = oact.nvfp4_global_scale(x)
    tiled = o4.nvfp4_tile_weight_scales(dev(sbits), k)
    ws = o4.nvfp4_workspace(m, k, torch.device("cuda"))
    y = o4.nvfp4_linear(dev(x).bfloat16(), dev(packed), tiled, dev(s2), torch.tensor([s2x], device="cuda"), workspace=ws)
    o4.nvfp4_status(ws, m, k)
    rng = np.random.default_rng(m)
    rows, cols = sample(rng, m, 48), sample(rng, n, 384)
    ref = ol.nvfp4_linear(x[rows], packed[cols], sbits[cols], s2, s2x)
    close(y.float().cpu().numpy()[np.ix_(rows, cols)], ref)


# ---------------------------------------------------------------------------------------------- FP8 W8A8 (config #3)


@pytest.fixture(scope="module")
def fp8_block():
    return synth.fp8_weight(1024, 5120, seed=3)


@pytest.mark.parametrize("n", [17408, 5120])
@pytest.mark.parametrize("m", [1, 32, 512, 8192])
def test_fp8_k5120(m, n, fp8_block):
    from emmy_b200 import ops

    k = 5120
    bits_b, scale_b = fp8_block
    reps = n // 1024
    bits, scale = np.tile(bits_b, (reps, 1)), np.tile(scale_b.reshape(-1), reps)
    x = synth.activations(m, k, "bf16", seed=30 + m)
    ws = ops.fp8_workspace(m, k, torch.device("cuda"))
    y = ops.fp8_linear(dev(x).bfloat16(), dev(bits), dev(scale), workspace=ws)
    ops.fp8_status(ws, m, k)
    rng = np.random.default_rng(m + n)
    rows, cols = sample(rng, m, 48), sample(rng, n, 384)
    ref = ol.fp8_linear(x[rows], bits[cols], scale[cols].reshape(-1, 1))
    close(y.float().cpu().numpy()[np.ix_(rows, cols)], ref)


# ---------------------------------------------------------------------------------------------- GPTQ act-order (config #2)


@pytest.fixture(scope="module", params=[(4096, 14336), (14336, 4096)], ids=["gate_up", "down"])
def gptq_weight(request):
    from emmy_b200 import ops

    k, n = request.param
    qw, qz, sc, gi = synth.gptq_linear(k, n, seed=2)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "gptq", g_idx=dev(gi))
    return k, n, qw, qz, sc, gi, w


@pytest.mark.parametrize("m", [1, 4, 16, 64, 256])
def test_gptq_llama_mlp(m, gptq_weight):
    """Both Llama-3.1-8B MLP shapes against the oracle's dequantize-then-matmul; K = 14336, N = 4096 at M = 64 is the
    split-K form of the tensor path (partial sums meet in the workspace)."""
    from emmy_b200 import ops

    k, n, qw, qz, sc, gi, w = gptq_weight
    x = synth.activations(m, k, "f16", seed=20 + m)
    ws = ops.w4a16_workspace(m, n, torch.device("cuda"), k)
    y = ops.w4a16_linear(dev(x).half(), w, workspace=ws)
    ops.w4a16_status(ws, m, n)
    rng = np.random.default_rng(m)
    rows, cols = sample(rng, m, 48), sample(rng, n, 256, unit=8)  # zero points are packed eight columns to a word
    ref = ol.w4a16_linear(x[rows], qw[:, cols], qz[:, cols[::8] // 8], sc[:, cols], 128, "gptq", "f16", gi)
    close(y.float().cpu().numpy()[np.ix_(rows, cols)], ref)


# ---------------------------------------------------------------------------------------------- AWQ (config #1)


@pytest.mark.parametrize("m", [1, 16])
def test_awq_4096(m):
    from emmy_b200 import ops

    k = n = 4096
    qw, qz, sc = synth.awq_linear(k, n, seed=1)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "awq")
    x = synth.activations(m, k, "f16", seed=10 + m)
    y = ops.w4a16_linear(dev(x).half(), w)
    rng = np.random.default_rng(m)
    cols = sample(rng, n, 512, unit=8)
    ref = ol.w4a16_linear(x, qw[:, cols[::8] // 8], qz[:, cols[::8] // 8], sc[:, cols], 128, "awq", "f16")
    close(y.float().cpu().numpy()[:, cols], ref)


# ---------------------------------------------------------------------------------------------- MoE (config #5)


@pytest.mark.parametrize("t", [1, 64, 4096])
def test_moe_qwen3_shapes(t):
    """128 experts, top-8, hidden 2048, intermediate 768.  Four weight blobs are shared by the experts (expert e uses
    blob e % 4) to keep the host side short; a sample of the tokens is checked against the oracle layer."""
    from emmy_b200 import ops_moe as om

    e, h, inter, k, blobs = 128, 2048, 768, 8, 4
    gu = [synth.awq_linear(h, 2 * inter, seed=50 + 2 * i) for i in range(blobs)]
    dn = [synth.awq_linear(inter, h, seed=51 + 2 * i) for i in range(blobs)]
    base = {"gate_up": tuple(np.stack([p[j] for p in gu]) for j in range(3)), "down": tuple(np.stack([p[j] for p in dn]) for j in range(3))}
    idx = np.arange(e) % blobs
    w = om.moe_repack(tuple(dev(a[idx]) for a in base["gate_up"]), tuple(dev(a[idx]) for a in base["down"]))
    wgu, wdn = omoe.dequant_expert_weights(base, torch.bfloat16)
    x = torch.from_numpy(synth.activations(t, h, "bf16", seed=60 + t)).bfloat16()
    logits = torch.randn(t, e, generator=torch.Generator().manual_seed(t))
    ws = om.moe_workspace(t, w, k, torch.device("cuda"))
    y = om.moe_forward(x.cuda(), logits.cuda(), w, k, workspace=ws)
    om.moe_status(ws, t, w, k)
    rows = torch.from_numpy(sample(np.random.default_rng(t), t, 24))
    xs, ls = x[rows], logits[rows]
    scores, ids = omoe.route_softmax_topk(ls, k)
    ref = omoe.combine_routed(xs, scores, ids, lambda ee, rr: omoe.expert_ffn(xs[rr], wgu[ee % blobs], wdn[ee % blobs])).float().numpy()
    close(y.float().cpu().numpy()[rows.numpy()], ref)
