"""NVFP4 W4A4 on the GPU against the CPU oracle, through the C ABI."""

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

    out = ops.dequant_nvfp4(dev(golden["nvfp4_packed"]), dev(golden["nvfp4_scale_bits"]), dev(golden["nvfp4_scale_2"]))
    np.testing.assert_array_equal(out.cpu().numpy(), golden["nvfp4_dequant"])
    out = ops.dequant_nvfp4(dev(golden["nvfp4_rand_packed"]), dev(golden["nvfp4_rand_scale_bits"]), dev(np.array([0.03125], np.float32)))
    np.testing.assert_array_equal(out.cpu().numpy(), golden["nvfp4_rand_dequant"])


def test_weight_dequant_hand_example():
    # tests/compiler/loader/test_quant.py:114-121
    from emmy_b200 import ops

    one, six = 0b0010, 0b0111
    packed = np.array([[one | one << 4] * 8 + [six | six << 4] * 8], dtype=np.uint8)
    sbits = np.array([[8 << 3, 7 << 3]], dtype=np.uint8)
    out = ops.dequant_nvfp4(dev(packed), dev(sbits), dev(np.array([2.0], np.float32))).cpu().numpy()
    np.testing.assert_array_equal(out, np.array([[4.0] * 16 + [12.0] * 16], dtype=np.float32))


def test_activation_quant_golden_bit_exact(golden):
    from emmy_b200 import ops_nvfp4 as o4

    codes, sf = o4.quant_nvfp4_act(dev(golden["act4_in"]), dev(golden["act4_s2"]))
    np.testing.assert_array_equal(sf.cpu().numpy(), golden["act4_scale_bits"])
    np.testing.assert_array_equal(codes.cpu().numpy(), golden["act4_packed"])


def test_activation_quant_midpoint_known_answer():
    # tests/compiler/loader/test_quant.py:1815-1836: scale byte 0x38, packed byte 0x47
    from emmy_b200 import ops_nvfp4 as o4

    x = np.zeros((4, 32), dtype=np.float32)
    x[0, :2] = (0.625, 0.25)
    codes, sf = o4.quant_nvfp4_act(dev(x), dev(np.array([0.1], np.float32)))
    assert int(sf[0, 0]) == 0x38 and int(codes[0, 0]) == 0x47
    assert int(codes[1:].count_nonzero()) == 0  # zero blocks stay zero, never NaN


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_activation_quant_and_global_scale_bit_exact(dtype):
    from emmy_b200 import ops_nvfp4 as o4

    x = synth.activations(37, 512, dtype, seed=5)
    x[3, 16:32] = 0.0
    t = dev(x).bfloat16() if dtype == "bf16" else dev(x).half()
    s2 = o4.nvfp4_global_scale(t)
    assert s2.cpu().numpy()[0] == oact.nvfp4_global_scale(x)
    codes, sf, tiled = o4.quant_nvfp4_act(t, s2, tiled=True)
    rc, rs = oact.nvfp4_static_act(x, oact.nvfp4_global_scale(x))
    np.testing.assert_array_equal(sf.cpu().numpy(), rs)
    np.testing.assert_array_equal(codes.cpu().numpy(), rc)
    # the tiled copy holds the same scales: atom byte (r % 32) * 16 + (r / 32) * 4 + i
    tl = tiled.cpu().numpy().reshape(-1, 512 // 64, 512)
    for r, b in ((0, 0), (36, 31), (33, 5)):
        assert tl[r // 128, b // 4, (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4] == rs[r, b]
    assert tl[0, 0, (37 % 32) * 16 + (37 // 32) * 4] == 0  # padding rows are zero


def test_tile_scales_layout():
    from emmy_b200 import ops_nvfp4 as o4

    rows, k = 200, 256
    sf = np.random.default_rng(0).integers(0, 127, (rows, k // 16)).astype(np.uint8)
    tl = o4.nvfp4_tile_scales(dev(sf), k).cpu().numpy().reshape(2, k // 64, 512)
    for r in (0, 31, 32, 127, 128, 199):
        for b in (0, 3, 4, 15):
            assert tl[r // 128, b // 4, (r % 32) * 16 + ((r % 128) // 32) * 4 + b % 4] == sf[r, b]
    assert tl[1, 0, (72 % 32) * 16 + (72 // 32) * 4] == 0  # row 200 = block 1, row 72: padding


def _check(m, n, k, seed=0, dtype="bf16"):
    from emmy_b200 import ops_nvfp4 as o4

    packed, sbits, s2w = synth.nvfp4_weight(n, k, seed=seed)
    x = synth.activations(m, k, dtype, seed=seed + 1)
    s2x = oact.nvfp4_global_scale(x)
    t = dev(x).bfloat16() if dtype == "bf16" else dev(x).half()
    ws = o4.nvfp4_workspace(m, k, t.device)
    y = o4.nvfp4_linear(t, dev(packed), o4.nvfp4_tile_weight_scales(dev(sbits), k), dev(s2w), dev(np.array([s2x], np.float32)), workspace=ws)
    o4.nvfp4_status(ws, m, k)
    got = y.float().cpu().numpy()
    ref = ol.nvfp4_linear(x, packed, sbits, s2w, s2x)
    assert np.isfinite(got).all()
    err = np.abs(got - ref).max() / np.abs(ref).max()
    assert err <= TOL, f"relative max error {err}"
    return err


@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (128, 256, 1024), (64, 512, 512), (1, 256, 512), (200, 264, 768), (128, 128, 256), (129, 224, 256), (300, 504, 512), (700, 1000, 1024),
                                   (2048, 17408, 256), (1900, 17400, 512),  # these two are large enough for the 256 x 224 tiling
                                   (5, 264, 2048), (16, 1000, 1280), (9, 136, 256), (2, 264, 1024), (1, 136, 256)])  # the decode tile: ragged N, ring wrap at K > 1280
def test_nvfp4_linear_tensor_path(m, n, k):
    _check(m, n, k, seed=m + n)


def test_nvfp4_linear_known_answer():
    """Codes and scales chosen so that every product and sum is exact: the block-scaled MMA must reproduce it."""
    from emmy_b200 import ops_nvfp4 as o4

    rng = np.random.default_rng(1)
    m, n, k = 128, 256, 256
    wc = rng.integers(0, 16, (n, k)).astype(np.uint8)
    wc[wc == 8] = 0  # no negative zero
    wpacked = (wc[:, 0::2] | (wc[:, 1::2] << 4)).astype(np.uint8)
    wsf = rng.choice(np.array([0x30, 0x38, 0x40], np.uint8), (n, k // 16))  # 0.5, 1, 2
    wval = fm.E2M1_VALUES[wc] * np.repeat(fm.e4m3_decode(wsf), 16, axis=1)
    # activations already on the grid: x = code * block scale with block amax 6 * scale -> quantizes to itself
    xc = rng.integers(1, 8, (m, k)).astype(np.uint8)
    xc[:, 0::16] = 7  # every block holds a 6.0 so that its scale is exactly amax / 6
    xsf = rng.choice(np.array([0.5, 1.0, 2.0], np.float32), (m, k // 16))
    xval = (fm.E2M1_VALUES[xc] * np.repeat(xsf, 16, axis=1)).astype(np.float32)
    s2x = np.float32(1.0)
    y = o4.nvfp4_linear(dev(xval).bfloat16(), dev(wpacked), o4.nvfp4_tile_weight_scales(dev(wsf), k), dev(np.array([1.0], np.float32)),
                        dev(np.array([s2x], np.float32))).float().cpu().numpy()
    ref = fm.round_bf16(xval @ wval.T)
    np.testing.assert_array_equal(y, ref)


@pytest.mark.parametrize("m", [1, 128, 300])
def test_nvfp4_linear_full_width(m):
    _check(m, 17408, 5120, seed=3)


def test_weight_quantizer_bit_exact():
    """eq_quant_nvfp4_weight against the oracle port of quantize_nvfp4 (itself pinned to the reference's output):
    N(0, 0.02) weights, a zero block, a block far below the tensor's range and one value at the tensor's maximum."""
    from emmy_b200 import ops_nvfp4 as o4
    from oracle import formats as fm

    rng = np.random.default_rng(11)
    w = (rng.standard_normal((96, 512)) * 0.02).astype(np.float32)
    w[3, 32:48] = 0.0
    w[5, 64:80] *= 1e-6
    w[7, 100] = 0.25
    packed, sbits, s2 = fm.quant_nvfp4(w)
    got = o4.quant_nvfp4_weight(torch.from_numpy(w).cuda())
    np.testing.assert_array_equal(got[2].cpu().numpy(), s2)
    np.testing.assert_array_equal(got[1].cpu().numpy(), sbits)
    np.testing.assert_array_equal(got[0].cpu().numpy(), packed)
    # an all-zero tensor: scale_2 floors at 1e-12 / (6 * 448), every code and scale is zero
    z = o4.quant_nvfp4_weight(torch.zeros(8, 64, device="cuda"))
    pz, sz, s2z = fm.quant_nvfp4(np.zeros((8, 64), np.float32))
    np.testing.assert_array_equal(z[2].cpu().numpy(), s2z)
    assert int(z[0].count_nonzero()) == 0 and int(z[1].count_nonzero()) == 0 and not pz.any() and not sz.any()


def test_mxfp4_decode_bit_exact(golden):
    """The MXFP4 decoder against the reference's own output (incl. a denormal result and the overflow to infinity) and,
    on a larger random tensor, against the oracle; f32 and bf16 outputs."""
    from emmy_b200 import ops

    blocks, scales = golden["mxfp4_blocks"], golden["mxfp4_scales"]
    got = ops.dequant_mxfp4(dev(blocks), dev(scales)).cpu().numpy()
    np.testing.assert_array_equal(got, golden["mxfp4_decoded"].T)
    rng = np.random.default_rng(7)
    blocks = rng.integers(0, 256, (300, 20, 16)).astype(np.uint8)
    scales = rng.integers(100, 150, (300, 20)).astype(np.uint8)
    ref = fm.dequant_mxfp4(blocks, scales).T
    np.testing.assert_array_equal(ops.dequant_mxfp4(dev(blocks), dev(scales)).cpu().numpy(), ref)
    got16 = ops.dequant_mxfp4(dev(blocks), dev(scales), torch.bfloat16).float().cpu().numpy()
    np.testing.assert_array_equal(got16, fm.round_bf16(ref))


@pytest.mark.parametrize("m", [1, 12, 200])
def test_rmsnorm_inside_the_quantize(m):
    """y = nvfp4_linear(rmsnorm(x) * gamma) with the norm fused into the static quantize kernel, against the oracle's eager
    RMSNorm followed by the oracle linear (decode tile, 128-row tile)."""
    from emmy_b200 import ops_nvfp4 as o4

    n, k = 264, 1024
    packed, sbits, s2 = synth.nvfp4_weight(n, k, seed=m)
    x = fm.round_bf16(synth.activations(m, k, "bf16", seed=300 + m) * 2.0)
    gamma = fm.round_bf16(1.0 + 0.1 * np.random.default_rng(m).standard_normal(k).astype(np.float32))
    h = oact.rmsnorm(x, gamma, 1e-6, "bf16")
    s2x = oact.nvfp4_global_scale(h)
    ref = ol.nvfp4_linear(h, packed, sbits, s2, s2x)
    tiled = o4.nvfp4_tile_weight_scales(dev(sbits), k)
    y = o4.nvfp4_linear(dev(x).bfloat16(), dev(packed), tiled, dev(s2), torch.tensor([s2x], device="cuda"), norm_weight=dev(gamma).bfloat16(), eps=1e-6)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max()
