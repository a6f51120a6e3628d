"""Dequantize-then-matmul references for every linear family (test infrastructure).

Each function returns the f32 result of the reference's eager path
(emmy/compiler/trace/huggingface.py:2877-2920: decode the weight with numpy,
round it once to the model dtype, ordinary linear with f32 accumulation) and
leaves the final rounding to the caller's comparison.
"""

from __future__ import annotations

import numpy as np

from . import activations as act
from . import formats as fm


def _matmul_f32(x: np.ndarray, w_kn: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32) @ np.asarray(w_kn, dtype=np.float32)


def w4a16_linear(x, qweight, qzeros, scales, group_size, fmt, dtype, g_idx=None) -> np.ndarray:
    """y[M,N] = x @ dtype((q - z) * s): config #1/#2's eager path.  `x` holds
    values already representable in `dtype` ("f16" or "bf16")."""
    w = fm.cast_weight(fm.dequant_w4(qweight, qzeros, scales, group_size, fmt, g_idx), dtype)
    return _matmul_f32(x, w)


def w4a16_gate_up_swiglu(x, qweight, qzeros, scales, group_size, fmt, dtype, g_idx=None) -> np.ndarray:
    """act(silu(gate)) * up for a [gate | up] weight (gate columns, then up columns): both projections rounded to the
    activation dtype, silu in f32 rounded to the dtype, the product rounded again -- the eager form's roundings
    (emmy/compiler/trace/huggingface.py:1663-1669).  Returns f32 values representable in `dtype`."""
    rnd = fm.round_f16 if dtype == "f16" else fm.round_bf16
    gu = rnd(w4a16_linear(x, qweight, qzeros, scales, group_size, fmt, dtype, g_idx))
    inter = gu.shape[1] // 2
    gate, up = gu[:, :inter].astype(np.float32), gu[:, inter:].astype(np.float32)
    act = rnd(gate / (np.float32(1) + np.exp(-gate, dtype=np.float32)))
    return rnd(act * up)


def fp8_linear(x, w_bits, w_scale, dtype="bf16") -> np.ndarray:
    """W8A8 value path: x_hat = dtype(dec(q_x) * s_x), w_hat = dtype(dec(w) *
    s_w), ordinary linear (emmy/compiler/loader/quant.py:1655-1768)."""
    rnd = fm.round_bf16 if dtype == "bf16" else fm.round_f16
    xh = rnd(act.fp8_dynamic_round_trip(x))
    wh = rnd(fm.dequant_fp8(w_bits, w_scale))
    return _matmul_f32(xh, wh.T)


def fp8_linear_native(x, w_bits, w_scale) -> np.ndarray:
    """The hoisted-scale W8A8 product the reference's own k32 tensor path
    computes (tests/compiler/passes/test_fp8_mma.py:111-120):
    (sum_k q_x q_w) * s_x[m] * s_w[n], f32."""
    bits, sx = act.fp8_dynamic_per_token(x)
    acc = fm.e4m3_decode(bits).astype(np.float32) @ fm.e4m3_decode(w_bits).astype(np.float32).T
    return acc * sx * np.asarray(w_scale, dtype=np.float32).reshape(1, -1)


def fp8_block_linear(x, w_bits, w_scale_blocks, dtype="bf16") -> np.ndarray:
    """Block-scaled W8A8 value path: activations round-tripped per token and per 128 elements of K, weight
    dequantized by its 2-D block scales, both rounded to the model dtype, ordinary linear
    (emmy/compiler/loader/quant.py:147-170, 1655-1717)."""
    rnd = fm.round_bf16 if dtype == "bf16" else fm.round_f16
    bits, s = act.fp8_dynamic_per_group(x)
    xh = rnd(fm.e4m3_decode(bits) * np.repeat(s, 128, axis=1))
    wh = rnd(fm.dequant_fp8(w_bits, w_scale_blocks))
    return _matmul_f32(xh, wh.T)


def nvfp4_linear(x, w_packed, w_scale_bits, w_scale_2, input_scale) -> np.ndarray:
    """W4A4: static-quantized activation round trip times the dequantized
    weight (tests/compiler/loader/test_quant.py:1809-1812)."""
    xh = act.nvfp4_static_round_trip(x, input_scale)
    wh = fm.dequant_nvfp4(w_packed, w_scale_bits, w_scale_2)
    return _matmul_f32(xh, wh.T)
