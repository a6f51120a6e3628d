"""The CPU oracle against the reference: outputs captured from the reference's
own numpy functions (tests/golden/quant_golden.npz) and the known-answer
vectors its test-suite states."""

import numpy as np
import pytest

from oracle import activations as act
from oracle import formats as fm


def test_e4m3_table_matches_reference(golden):
    np.testing.assert_array_equal(fm.E4M3_TABLE, golden["e4m3_table"])
    # tests/compiler/loader/test_quant.py:64-68
    assert np.isnan(fm.E4M3_TABLE[0x7F]) and np.isnan(fm.E4M3_TABLE[0xFF])
    assert not np.isinf(fm.E4M3_TABLE).any()
    assert fm.E4M3_TABLE[0x7E] == 448.0 and fm.E4M3_TABLE[0xFE] == -448.0


def test_e4m3_table_matches_torch():
    torch = pytest.importorskip("torch")
    ref = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).float().numpy()
    np.testing.assert_array_equal(fm.E4M3_TABLE, ref)


def test_e4m3_encode_matches_reference(golden):
    np.testing.assert_array_equal(fm.e4m3_encode(golden["e4m3_encode_in"]), golden["e4m3_encode_out"])


def test_e4m3_encode_saturates_and_round_trips():
    assert fm.e4m3_encode(np.float32(500.0)) == 0x7E  # the reference saturates where torch's cast gives NaN
    codes = np.array([c for c in range(256) if c not in (0x7F, 0xFF)], dtype=np.uint8)
    np.testing.assert_array_equal(fm.e4m3_encode(fm.e4m3_decode(codes)), codes)


def test_e2m1_matches_reference(golden):
    np.testing.assert_array_equal(fm.e2m1_encode(golden["e2m1_encode_in"]), golden["e2m1_encode_out"])
    np.testing.assert_array_equal(fm.e2m1_decode_pairs(np.arange(256, dtype=np.uint8).reshape(1, 256)), golden["e2m1_pairs_decode"])


def test_e2m1_midpoints_go_to_even_code():
    # emmy/compiler/backend/torch_ref.py:119-129
    got = fm.e2m1_encode(np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 9.0], dtype=np.float32))
    np.testing.assert_array_equal(got, [0, 2, 2, 4, 4, 6, 6, 7])


def test_bf16_matches_reference(golden):
    np.testing.assert_array_equal(fm.bf16_bits(golden["bf16_in"]), golden["bf16_bits"])


def test_int4_shifts(golden):
    np.testing.assert_array_equal(fm.AWQ_SHIFTS, golden["awq_shifts"])
    np.testing.assert_array_equal(fm.GPTQ_SHIFTS, golden["gptq_shifts"])


@pytest.mark.parametrize("name", ["awq", "gptq", "awq_g32", "gptq_g32"])
def test_int4_unpack_and_dequant_match_reference(golden, name):
    fmt = name.split("_")[0]
    rows = fmt == "gptq"
    qw, qz, sc = golden[f"{name}_qweight"], golden[f"{name}_qzeros"], golden[f"{name}_scales"]
    np.testing.assert_array_equal(fm.unpack_int4(qw, fmt, along_rows=rows), golden[f"{name}_unpacked"])
    np.testing.assert_array_equal(fm.unpack_int4(qz, fmt), golden[f"{name}_zeros_unpacked"])
    np.testing.assert_array_equal(fm.dequant_w4(qw, qz, sc, int(golden[f"{name}_group"]), fmt), golden[f"{name}_dequant"])
    # pack is the inverse of unpack
    np.testing.assert_array_equal(fm.pack_int4(golden[f"{name}_unpacked"], fmt, along_rows=rows), qw)


def test_awq_unpack_reverses_gemm_pack_order():
    # tests/compiler/loader/test_quant.py:236-245, 972-974: order (0,2,4,6,1,3,5,7)
    values = np.arange(32, dtype=np.int32).reshape(2, 16) % 16
    packed = np.zeros((2, 2), dtype=np.uint32)
    for word in range(2):
        for slot, logical in enumerate((0, 2, 4, 6, 1, 3, 5, 7)):
            packed[:, word] |= values[:, word * 8 + logical].astype(np.uint32) << np.uint32(slot * 4)
    np.testing.assert_array_equal(fm.unpack_int4(packed.view(np.int32), "awq"), values)


def _fixture(k=8, n=16, g=4, zmod=16):
    ints = (np.arange(k * n, dtype=np.int32).reshape(k, n) * 7 + 3) % 16
    zeros = (np.arange((k // g) * n, dtype=np.int32).reshape(k // g, n) * 5 + 1) % zmod
    scales = ((np.arange((k // g) * n, dtype=np.float32).reshape(k // g, n) + 1) / 128).astype(np.float16)
    return ints, zeros, scales


def test_awq_fixture_group_formula():
    # tests/compiler/loader/test_quant.py:955-981
    ints, zeros, scales = _fixture()
    ref = (ints - np.repeat(zeros, 4, axis=0)) * np.repeat(scales.astype(np.float32), 4, axis=0)
    got = fm.dequant_w4(fm.pack_int4(ints, "awq"), fm.pack_int4(zeros, "awq"), scales, 4, "awq")
    np.testing.assert_array_equal(got, ref)


def test_gptq_fixture_adds_the_v1_zero_bias():
    # tests/compiler/loader/test_quant.py:1038-1072
    ints, zeros, scales = _fixture(zmod=15)
    ref = (ints - np.repeat(zeros + 1, 4, axis=0)) * np.repeat(scales.astype(np.float32), 4, axis=0)
    qw, qz = fm.pack_int4(ints, "gptq", along_rows=True), fm.pack_int4(zeros, "gptq")
    got = fm.dequant_w4(qw, qz, scales, 4, "gptq")
    np.testing.assert_array_equal(got, ref)
    identity = (np.arange(8) // 4).astype(np.int32)
    np.testing.assert_array_equal(fm.dequant_w4(qw, qz, scales, 4, "gptq", g_idx=identity), ref)


def test_gptq_act_order_is_a_group_gather():
    ints, zeros, scales = _fixture(k=16, zmod=15)
    qw, qz = fm.pack_int4(ints, "gptq", along_rows=True), fm.pack_int4(zeros, "gptq")
    g_idx = np.array([3, 3, 3, 3, 0, 0, 0, 0, 2, 2, 2, 2, 1, 1, 1, 1], dtype=np.int32)
    got = fm.dequant_w4(qw, qz, scales, 4, "gptq", g_idx=g_idx)
    ref = (ints - (zeros + 1)[g_idx]) * scales.astype(np.float32)[g_idx]
    np.testing.assert_array_equal(got, ref)


def test_int4_geometry_errors():
    ints, zeros, scales = _fixture()
    qw, qz = fm.pack_int4(ints, "awq"), fm.pack_int4(zeros, "awq")
    with pytest.raises(ValueError):
        fm.dequant_w4(qw, qz, scales, 3, "awq")
    with pytest.raises(ValueError):
        fm.dequant_w4(qw, qz, scales[:, :8], 4, "awq")
    with pytest.raises(ValueError):
        fm.unpack_int4(qw.astype(np.int64), "awq")


def test_fp8_weight_dequant_matches_reference(golden):
    b = golden["fp8_bits"]
    np.testing.assert_array_equal(fm.dequant_fp8(b, golden["fp8_scale_channel"]), golden["fp8_dequant_channel"])
    np.testing.assert_array_equal(fm.dequant_fp8(b, golden["fp8_scale_block"]), golden["fp8_dequant_block"])
    np.testing.assert_array_equal(fm.dequant_fp8(b, np.array([0.0625], np.float32)), golden["fp8_dequant_tensor"])
    with pytest.raises(ValueError):
        fm.dequant_fp8(b, np.ones((3, 1), np.float32))


def test_nvfp4_hand_example():
    # tests/compiler/loader/test_quant.py:114-121: values 1.0 then 6.0, block scales 2.0 then 1.0, scale_2 = 2
    one, six = 0b0010, 0b0111
    packed = np.array([[one | one << 4] * 8 + [six | six << 4] * 8], dtype=np.uint8)
    sbits = np.array([[8 << 3, 7 << 3]], dtype=np.uint8)
    out = fm.dequant_nvfp4(packed, sbits, np.array(2.0, np.float32))
    np.testing.assert_array_equal(out, np.array([[4.0] * 16 + [12.0] * 16], dtype=np.float32))


def test_nvfp4_matches_reference(golden):
    packed, sbits, s2 = fm.quant_nvfp4(golden["nvfp4_in"])
    np.testing.assert_array_equal(packed, golden["nvfp4_packed"])
    np.testing.assert_array_equal(sbits, golden["nvfp4_scale_bits"])
    np.testing.assert_array_equal(s2, golden["nvfp4_scale_2"])
    np.testing.assert_array_equal(fm.dequant_nvfp4(packed, sbits, s2), golden["nvfp4_dequant"])
    np.testing.assert_array_equal(fm.nvfp4_fused_scale(sbits, s2), golden["nvfp4_fused"])
    got = fm.dequant_nvfp4(golden["nvfp4_rand_packed"], golden["nvfp4_rand_scale_bits"], np.array(0.03125, np.float32))
    np.testing.assert_array_equal(got, golden["nvfp4_rand_dequant"])


def test_nvfp4_quantize_properties():
    # tests/compiler/loader/test_quant.py:2238-2294
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((3, 64)) * np.array([[0.01], [1.0], [80.0]])).astype(np.float32)
    packed, sbits, s2 = fm.quant_nvfp4(x)
    assert (packed.dtype, packed.shape) == (np.uint8, (3, 32))
    assert (sbits.dtype, sbits.shape) == (np.uint8, (3, 4)) and not (sbits >> 7).any()
    back = fm.dequant_nvfp4(packed, sbits, s2)
    amax = np.abs(x).reshape(3, 4, 16).max(axis=-1).repeat(16, axis=-1).reshape(3, 64)
    assert (np.abs(back - x) <= amax / 6 + 1e-6).all()
    once = fm.dequant_nvfp4(*fm.quant_nvfp4(np.random.default_rng(1).standard_normal((2, 32)).astype(np.float32)))
    np.testing.assert_array_equal(fm.dequant_nvfp4(*fm.quant_nvfp4(once)), once)  # idempotent on the grid
    assert not fm.dequant_nvfp4(*fm.quant_nvfp4(np.zeros((1, 16), np.float32))).any()
    for mag in (0.0, 1e-42, 1e-30):
        p, s, g = fm.quant_nvfp4(np.full((1, 16), mag, np.float32))
        assert g[0] > 0 and np.isfinite(fm.dequant_nvfp4(p, s, g)).all()
    with pytest.raises(AssertionError):
        fm.quant_nvfp4(np.zeros((1, 20), np.float32))
    with pytest.raises(AssertionError):
        fm.quant_nvfp4(np.full((1, 16), 3e38, np.float32))


def test_static_nvfp4_activation_matches_reference(golden):
    packed, sbits = act.nvfp4_static_act(golden["act4_in"], golden["act4_s2"][0])
    np.testing.assert_array_equal(packed, golden["act4_packed"])
    np.testing.assert_array_equal(sbits, golden["act4_scale_bits"])
    np.testing.assert_array_equal(act.nvfp4_static_round_trip(golden["act4_in"], golden["act4_s2"][0]), golden["act4_round_trip"])
    assert act.nvfp4_global_scale(golden["act4_in"]) == golden["act4_s2"][0]


def test_static_nvfp4_midpoint_known_answer():
    # tests/compiler/loader/test_quant.py:1815-1836: scale byte 0x38 (1.0), packed byte 0x47 (codes [6, 2])
    x = np.zeros((4, 32), dtype=np.float32)
    x[0, :2] = (0.625, 0.25)
    packed, sbits = act.nvfp4_static_act(x, 0.1)
    assert int(sbits[0, 0]) == 0x38 and int(packed[0, 0]) == 0x47


def test_dynamic_fp8_activation_matches_reference(golden):
    bits, s = act.fp8_dynamic_per_token(golden["act8_in"])
    np.testing.assert_array_equal(bits, golden["act8_bits"])
    np.testing.assert_array_equal(s, golden["act8_scale"])


def test_dynamic_fp8_activation_matches_eager_hook():
    # tests/compiler/loader/test_quant.py:2114-2120, in f32
    torch = pytest.importorskip("torch")
    x = torch.randn(6, 80, generator=torch.Generator().manual_seed(3))
    scale = x.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12) / 448.0
    ref = (x / scale).to(torch.float8_e4m3fn).float() * scale
    np.testing.assert_array_equal(act.fp8_dynamic_round_trip(x.numpy()), ref.numpy())


def test_mxfp4_decode_matches_reference(golden):
    """decode_mxfp4 of the reference on random blocks, incl. the smallest exponent (a denormal result), 2^0 and the
    largest one (overflow to infinity, as the reference's cast does)."""
    got = fm.dequant_mxfp4(golden["mxfp4_blocks"], golden["mxfp4_scales"])
    assert got.shape == golden["mxfp4_decoded"].shape and got.dtype == np.float32
    np.testing.assert_array_equal(got, golden["mxfp4_decoded"])


def test_mxfp4_hand_example():
    """0x21: low nibble 1 -> 0.5 (even position), high nibble 2 -> 1.0 (odd position); scale 128 -> x2."""
    blocks = np.zeros((1, 1, 16), np.uint8)
    blocks[0, 0, 0] = 0x21
    blocks[0, 0, 15] = 0xF7  # 6.0 and -6.0
    out = fm.dequant_mxfp4(blocks, np.array([[128]], np.uint8))
    assert out.shape == (32, 1)
    assert out[0, 0] == 1.0 and out[1, 0] == 2.0 and out[30, 0] == 12.0 and out[31, 0] == -12.0
    assert not out[2:30].any()
