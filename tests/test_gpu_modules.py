"""The nn.Module surface: checkpoint tensor names in, operator calls out, also under torch.compile."""

import numpy as np
import pytest
import torch

from oracle import activations as oact
from oracle import formats as fm
from oracle import linear as ol
from oracle import synth

pytestmark = pytest.mark.gpu


def test_w4_module_loads_checkpoint_names_and_matches_oracle():
    from emmy_b200.linear import W4A16Linear

    k, n = 512, 256
    qw, qz, sc, gi = synth.gptq_linear(k, n, seed=1)
    mod = W4A16Linear(k, n, 128, fmt="gptq", act_order=True)
    mod.load_state_dict({"qweight": torch.from_numpy(qw), "qzeros": torch.from_numpy(qz), "scales": torch.from_numpy(sc),
                         "g_idx": torch.from_numpy(gi)})
    mod = mod.cuda()
    w_ref = fm.cast_weight(fm.dequant_w4(qw, qz, sc, 128, "gptq", gi), "f16").T
    np.testing.assert_array_equal(mod.dequantized_weight().float().cpu().numpy(), w_ref)
    mod.finalize()
    x = synth.activations(6, k, "f16", seed=2)
    y = mod(torch.from_numpy(x).half().cuda().reshape(2, 3, k))
    ref = ol.w4a16_linear(x, qw, qz, sc, 128, "gptq", "f16", gi)
    assert y.shape == (2, 3, n)
    assert np.abs(y.reshape(6, n).float().cpu().numpy() - ref).max() <= 2e-2 * np.abs(ref).max()


def test_modules_trace_under_torch_compile():
    from emmy_b200.linear import FP8Linear, W4A16Linear

    k, n = 256, 256
    qw, qz, sc = synth.awq_linear(k, n, seed=3)
    a = W4A16Linear(k, n, 128, fmt="awq")
    a.load_state_dict({"qweight": torch.from_numpy(qw), "qzeros": torch.from_numpy(qz), "scales": torch.from_numpy(sc)})
    a = a.cuda().finalize()
    bits, sw = synth.fp8_weight(n, n, seed=4)
    b = FP8Linear(n, n).cuda()
    b.load_float8(torch.from_numpy(bits).cuda().view(torch.float8_e4m3fn), torch.from_numpy(sw).cuda())

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = a, b

        def forward(self, x):
            return self.b(torch.nn.functional.silu(self.a(x)).bfloat16()).float()

    blk = Block()
    x = torch.from_numpy(synth.activations(4, k, "f16", seed=5)).half().cuda()
    eager = blk(x)
    compiled = torch.compile(blk, fullgraph=True, backend="eager")(x)
    # tests/test_dynamo.py:22 tolerance of the reference's torch.compile entry
    torch.testing.assert_close(compiled, eager, atol=2e-3, rtol=2e-2)


def test_fused_forms_as_custom_ops_under_torch_compile():
    """emmyq::w4a16_gate_up_swiglu and emmyq::fp8_linear_rmsnorm trace under torch.compile (fake kernels give the shapes)
    and equal their unfused compositions."""
    import emmy_b200.linear  # noqa: F401  (registers the ops)
    from emmy_b200 import ops

    k, inter, n = 256, 384, 256
    parts = []
    for i in range(2):
        qw, qz, sc = synth.awq_linear(k, inter, seed=6 + i)
        parts.append(ops.w4_repack(torch.from_numpy(qw).cuda(), torch.from_numpy(qz).cuda(), torch.from_numpy(sc).cuda(), 128, "awq"))
    gu = ops.w4_concat(parts)
    bits, sw = synth.fp8_weight(n, inter, seed=8)
    wb, ws = torch.from_numpy(bits).cuda(), torch.from_numpy(sw.reshape(-1)).cuda()
    gamma = (1.0 + 0.1 * torch.randn(inter, generator=torch.Generator().manual_seed(1))).bfloat16().cuda()

    def fused(x):
        h = torch.ops.emmyq.w4a16_gate_up_swiglu(x, gu.wq, k, 2 * inter, 128, False)
        return torch.ops.emmyq.fp8_linear_rmsnorm(h.bfloat16(), gamma, 1e-6, wb, ws).float()

    def unfused(x):
        g, u = ops.w4a16_linear(x, parts[0]), ops.w4a16_linear(x, parts[1])
        h = (torch.nn.functional.silu(g) * u).bfloat16()
        hf = h.float()
        normed = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6)).bfloat16()
        return ops.fp8_linear(gamma * normed, wb, ws).float()

    for m in (3, 40):
        x = torch.from_numpy(synth.activations(m, k, "f16", seed=9 + m)).half().cuda()
        ref = unfused(x)
        got = torch.compile(fused, fullgraph=True, backend="eager")(x)
        assert got.shape == ref.shape
        assert float((got - ref).abs().max()) <= 2e-2 * float(ref.abs().max())


def test_nvfp4_module():
    from emmy_b200.linear import NVFP4Linear

    n, k = 256, 512
    packed, sbits, s2 = synth.nvfp4_weight(n, k, seed=6)
    x = synth.activations(9, k, "bf16", seed=7)
    s2x = oact.nvfp4_global_scale(x)
    mod = NVFP4Linear(k, n)
    mod.load_state_dict({"weight": torch.from_numpy(packed), "weight_scale": torch.from_numpy(sbits), "weight_scale_2": torch.from_numpy(s2),
                         "input_scale": torch.tensor([s2x])})
    y = mod.cuda()(torch.from_numpy(x).bfloat16().cuda()).float().cpu().numpy()
    ref = ol.nvfp4_linear(x, packed, sbits, s2, s2x)
    assert np.abs(y - ref).max() <= 2e-2 * np.abs(ref).max()
