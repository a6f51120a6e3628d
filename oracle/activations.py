"""Activation quantizers of the W8A8 / W4A4 paths, in numpy (test infrastructure)."""

from __future__ import annotations

import numpy as np

from .formats import (
    dequant_nvfp4,
    e2m1_encode_pairs,
    e4m3_decode,
    e4m3_encode,
    quant_fp8_rows,
)


def fp8_dynamic_per_token(x) -> tuple[np.ndarray, np.ndarray]:
    """x [M, K] (values already rounded to the activation dtype) -> (bits u8
    [M, K], scale f32 [M, 1]).  Per token: s = max(amax|x|, 1e-12) / 448 in
    f32, bits = e4m3_rne_satfinite(x / s) with an f32 division
    (emmy/compiler/loader/quant.py:1655-1735; eager mirror
    tests/compiler/loader/test_quant.py:2114-2120)."""
    return quant_fp8_rows(x)


def fp8_dynamic_round_trip(x) -> np.ndarray:
    """The value a consumer of the dynamic FP8 activation reads: dec(bits) * s
    (emmy/compiler/loader/quant.py:1747-1768), in f32."""
    bits, s = fp8_dynamic_per_token(x)
    return e4m3_decode(bits) * s


def fp8_dynamic_per_group(x, group: int = 128) -> tuple[np.ndarray, np.ndarray]:
    """The dynamic rule per token AND per `group` elements of K: x [M, K] -> (bits u8 [M, K], scale f32 [M, K / group]);
    what a `weight_block_size` declaration selects (emmy/compiler/loader/quant.py:1581-1593, 1655-1717)."""
    xf = np.asarray(x, dtype=np.float32)
    m, k = xf.shape
    bits, s = quant_fp8_rows(xf.reshape(m * (k // group), group))
    return bits.reshape(m, k), s.reshape(m, k // group)


def nvfp4_global_scale(x) -> np.float32:
    """The calibrated-on-the-sample input scale: max(amax, 1e-12) / (6 * 448)
    (emmy/compiler/loader/synthesize.py:181-183)."""
    amax = max(float(np.abs(np.asarray(x, dtype=np.float32)).max()), 1e-12)
    return np.float32(amax / (6.0 * 448.0))


def nvfp4_static_act(x, s2) -> tuple[np.ndarray, np.ndarray]:
    """Static-scale NVFP4 activation quantize: x [M, K] -> (packed u8 [M, K/2],
    scale_bits u8 [M, K/16]).  Per 16-block: ratio = (amax * f32(1/6)) *
    f32(1/s2); scale_bits = e4m3(ratio); fused32 = dec(scale_bits) * s2;
    codes = e2m1(block / max(fused32, 1e-12)), every step in f32 with
    round-to-nearest division.  Follows
    tests/compiler/loader/test_quant.py:1776-1784 (`_static_quantize_ref`),
    which pins emmy/compiler/loader/quant.py:1968-2139."""
    xf = np.asarray(x, dtype=np.float32)
    s2 = np.float32(s2)
    blocks = xf.reshape(*xf.shape[:-1], -1, 16)
    ratio = (np.abs(blocks).max(axis=-1) * (np.float32(1) / np.float32(6))) * (np.float32(1) / s2)
    scale_bits = e4m3_encode(ratio)
    fused = e4m3_decode(scale_bits) * s2
    quot = blocks / np.maximum(fused[..., None], np.float32(1e-12))
    return e2m1_encode_pairs(quot.reshape(xf.shape)), scale_bits


def nvfp4_static_round_trip(x, s2) -> np.ndarray:
    """Quantize then reconstruct with the f16 fused scale, in f32."""
    packed, scale_bits = nvfp4_static_act(x, s2)
    return dequant_nvfp4(packed, scale_bits, np.float32(s2).reshape(1))


def rmsnorm(x, gamma, eps: float, dtype: str = "bf16") -> np.ndarray:
    """The model's RMSNorm as its eager module computes it (the HF Llama / Qwen3 form the reference traces): the mean of
    squares and the reciprocal root in f32, the normalised value rounded to the activation dtype, then the weight's
    product rounded again.  x and gamma hold values representable in `dtype`; returns such values as f32."""
    from . import formats as fm

    rnd = fm.round_bf16 if dtype == "bf16" else fm.round_f16
    xf = np.asarray(x, dtype=np.float32)
    var = np.mean(xf * xf, axis=-1, keepdims=True, dtype=np.float32)
    normed = rnd(xf * (np.float32(1) / np.sqrt(var + np.float32(eps))))
    return rnd(normed * np.asarray(gamma, dtype=np.float32))
