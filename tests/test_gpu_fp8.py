"""FP8-E4M3 W8A8 on the GPU against the CPU oracle, through the C ABI."""

import numpy as np
import pytest
import torch

from oracle import activations as oact
from oracle import formats as fm
from oracle import linear as ol
from oracle import synth

pytestmark = pytest.mark.gpu
TOL = 2e-2


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_weight_dequant_golden_bit_exact(golden):
    from emmy_b200 import ops

    bits = dev(golden["fp8_bits"])
    for key, ref in (("fp8_scale_channel", "fp8_dequant_channel"), ("fp8_scale_block", "fp8_dequant_block")):
        out = ops.dequant_fp8(bits, dev(golden[key]), out_dtype=torch.float32).cpu().numpy()
        np.testing.assert_array_equal(out, golden[ref])
    out = ops.dequant_fp8(bits, dev(np.array([0.0625], np.float32)), out_dtype=torch.float32).cpu().numpy()
    np.testing.assert_array_equal(out, golden["fp8_dequant_tensor"])


def test_weight_dequant_all_codes_and_rounding():
    from emmy_b200 import ops

    codes = np.array([c for c in range(256) if c not in (0x7F, 0xFF)] * 2 + [0, 0, 0, 0], dtype=np.uint8).reshape(8, 64)
    s = np.random.default_rng(0).uniform(1e-3, 1.0, (8, 1)).astype(np.float32)
    ref = fm.dequant_fp8(codes, s)
    np.testing.assert_array_equal(ops.dequant_fp8(dev(codes), dev(s), torch.float32).cpu().numpy(), ref)
    np.testing.assert_array_equal(ops.dequant_fp8(dev(codes), dev(s), torch.bfloat16).float().cpu().numpy(), fm.round_bf16(ref))


def test_activation_quant_golden_bit_exact(golden):
    from emmy_b200 import ops

    q, s = ops.quant_fp8_per_token(dev(golden["act8_in"]))
    np.testing.assert_array_equal(q.cpu().numpy(), golden["act8_bits"])
    np.testing.assert_array_equal(s.cpu().numpy(), golden["act8_scale"])


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [(1, 5120), (33, 5120), (7, 256)])
def test_activation_quant_bit_exact(dtype, shape):
    from emmy_b200 import ops

    x = synth.activations(shape[0], shape[1], dtype, seed=shape[0])
    x[0, :16] *= 37.0  # a row with an outlier
    x = fm.round_bf16(x) if dtype == "bf16" else fm.round_f16(x)
    t = dev(x).bfloat16() if dtype == "bf16" else dev(x).half()
    q, s = ops.quant_fp8_per_token(t)
    rq, rs = oact.fp8_dynamic_per_token(x)
    np.testing.assert_array_equal(s.cpu().numpy(), rs)
    np.testing.assert_array_equal(q.cpu().numpy(), rq)


def test_activation_quant_zero_row_and_saturation():
    from emmy_b200 import ops

    x = np.zeros((2, 64), dtype=np.float32)
    x[1, 0], x[1, 1] = 448.0, -3.0
    q, s = ops.quant_fp8_per_token(dev(x))
    rq, rs = oact.fp8_dynamic_per_token(x)
    np.testing.assert_array_equal(q.cpu().numpy(), rq)
    np.testing.assert_array_equal(s.cpu().numpy(), rs)
    assert q[0].count_nonzero() == 0 and int(q[1, 0]) == 0x7E


def _check(x, bits, sw, dtype="bf16"):
    from emmy_b200 import ops

    t = dev(x).bfloat16() if dtype == "bf16" else dev(x).half()
    ws = ops.fp8_workspace(x.shape[0], x.shape[1], t.device)
    y = ops.fp8_linear(t, dev(bits), dev(sw.reshape(-1)), workspace=ws)
    ops.fp8_status(ws, x.shape[0], x.shape[1])
    got = y.float().cpu().numpy()
    ref = ol.fp8_linear(x, bits, sw, dtype)
    native = ol.fp8_linear_native(x, bits, sw)
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= TOL * np.abs(ref).max()
    # against the hoisted-scale product the kernel actually computes the gap is the output rounding only
    assert np.abs(got - native).max() <= 1e-2 * np.abs(native).max()


@pytest.mark.parametrize("m", [1, 5, 16, 32, 64])
def test_fp8_linear_decode_shaped(m):
    bits, sw = synth.fp8_weight(1024, 1280, seed=m)
    _check(synth.activations(m, 1280, "bf16", seed=100 + m), bits, sw)


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (128, 512, 1024), (200, 272, 384), (512, 1024, 5120)])
def test_fp8_linear_tensor_path(m, n, k):
    """tcgen05 path incl. ragged M (200) and N (272 = 256 + 16)."""
    bits, sw = synth.fp8_weight(n, k, seed=n)
    _check(synth.activations(m, k, "bf16", seed=m), bits, sw)


def test_fp8_linear_f16_output():
    bits, sw = synth.fp8_weight(256, 256, seed=2)
    _check(synth.activations(130, 256, "f16", seed=3), bits, sw, dtype="f16")
    _check(synth.activations(3, 256, "f16", seed=3), bits, sw, dtype="f16")


def test_fp8_linear_small_integer_known_answer():
    """Operands that are exact in e4m3 and sums that are exact in f32: the tensor path must reproduce them exactly."""
    from emmy_b200 import ops

    rng = np.random.default_rng(0)
    m, n, k = 128, 256, 256
    wv = rng.integers(-3, 4, (n, k)).astype(np.float32)
    xv = rng.integers(-2, 3, (m, k)).astype(np.float32)
    xv[:, 0] = 2.0  # every row's amax is 2 -> scale 2/448, x / s = 224 x: exact e4m3 values
    bits = fm.e4m3_encode(wv)
    sw = np.ones((n, 1), np.float32)
    y = ops.fp8_linear(dev(xv).bfloat16(), dev(bits), dev(sw.reshape(-1))).float().cpu().numpy()
    ref = fm.round_bf16(xv @ wv.T)
    np.testing.assert_array_equal(y, ref)


@pytest.mark.parametrize("n", [5120, 17408])
def test_fp8_linear_full_size_m1(n):
    bits, sw = synth.fp8_weight(n, 5120, seed=0)
    _check(synth.activations(1, 5120, "bf16", seed=1), bits, sw)


@pytest.mark.parametrize("m,n,k", [(3, 144, 128), (17, 144, 128), (33, 400, 1024), (48, 144, 640), (65, 272, 384), (100, 400, 256), (129, 144, 128), (257, 528, 640),
                                   (600, 784, 384)])
def test_fp8_linear_tile_edges(m, n, k):
    """Row counts on either side of the 16 / 32 / 64 / 128 / 256 boundaries where the kernel or the tiling changes, and widths
    that leave a partial 128- or 256-column tile."""
    bits, sw = synth.fp8_weight(n, k, seed=m)
    _check(synth.activations(m, k, "bf16", seed=n), bits, sw)


def test_fp8_linear_empty_batch():
    from emmy_b200 import ops

    bits, sw = synth.fp8_weight(64, 128, seed=0)
    y = ops.fp8_linear(torch.empty(0, 128, dtype=torch.bfloat16, device="cuda"), dev(bits), dev(sw.reshape(-1)))
    assert y.shape == (0, 64)


@pytest.mark.parametrize("m", [1, 20, 300])
def test_rmsnorm_inside_the_quantize(m):
    """y = fp8_linear(rmsnorm(x) * gamma) with the norm fused into the quantize kernel, against the oracle's eager RMSNorm
    followed by the oracle linear.  (The mean of squares is summed in another order than numpy's, so a normalised value
    may land one rounding step away; the linear's tolerance covers it.)"""
    from emmy_b200 import ops
    from oracle import activations as oact

    n, k = 384, 1280
    bits, sw = synth.fp8_weight(n, k, seed=m)
    x = synth.activations(m, k, "bf16", seed=200 + m) * 3.0
    x = fm.round_bf16(x)
    gamma = fm.round_bf16(1.0 + 0.1 * np.random.default_rng(m).standard_normal(k).astype(np.float32))
    ref = ol.fp8_linear(oact.rmsnorm(x, gamma, 1e-6, "bf16"), bits, sw)
    y = ops.fp8_linear(dev(x).bfloat16(), dev(bits), dev(sw.reshape(-1)), norm_weight=dev(gamma).bfloat16(), eps=1e-6)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max()
