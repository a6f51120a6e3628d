"""Number formats and weight decoders of the quantized-linear path, in numpy.

Test infrastructure: a CPU restatement of the reference's value math, never
imported by the shipped package.  Each function names the reference code it
follows (paths are relative to the reference project's root).
"""

from __future__ import annotations

import numpy as np

# ---------------------------------------------------------------------------
# bf16 / fp16 rounding
# ---------------------------------------------------------------------------


def bf16_bits(values) -> np.ndarray:
    """f32 -> bf16 bit patterns (uint16), round to nearest even.

    Follows emmy/compiler/dtype.py:147-156 (add 0x7FFF plus the kept LSB, then
    drop the low half)."""
    u = np.ascontiguousarray(np.asarray(values, dtype=np.float32)).view(np.uint32)
    keep_lsb = (u >> np.uint32(16)) & np.uint32(1)
    return ((u + np.uint32(0x7FFF) + keep_lsb) >> np.uint32(16)).astype(np.uint16)


def bf16_value(bits) -> np.ndarray:
    """bf16 bit patterns -> f32 values (emmy/compiler/dtype.py:159-163)."""
    wide = np.asarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)
    return wide.view(np.float32)


def round_bf16(values) -> np.ndarray:
    """f32 values rounded once to bf16, returned as f32."""
    return bf16_value(bf16_bits(values))


def round_f16(values) -> np.ndarray:
    """f32 values rounded once to fp16 (numpy's cast is RNE), returned as f32."""
    return np.asarray(values, dtype=np.float32).astype(np.float16).astype(np.float32)


# ---------------------------------------------------------------------------
# FP8 e4m3fn
# ---------------------------------------------------------------------------

E4M3_MAX = 448.0


def _build_e4m3_table() -> np.ndarray:
    """All 256 e4m3fn values: bias 7, subnormals at exponent field 0, no
    infinities, NaN only at 0x7F / 0xFF (emmy/compiler/dtype.py:204-233)."""
    table = np.empty(256, dtype=np.float64)
    for code in range(256):
        e = (code >> 3) & 0xF
        m = code & 0x7
        mag = (m / 8.0) * 2.0**-6 if e == 0 else (1.0 + m / 8.0) * 2.0 ** (e - 7)
        if e == 0xF and m == 0x7:
            mag = np.nan
        table[code] = -mag if code & 0x80 else mag
    return table.astype(np.float32)


E4M3_TABLE = _build_e4m3_table()


def e4m3_decode(bits) -> np.ndarray:
    """uint8 e4m3fn codes -> f32 (emmy/compiler/dtype.py:236-238)."""
    return E4M3_TABLE[np.asarray(bits).astype(np.uint8, copy=False)]


def e4m3_encode(values) -> np.ndarray:
    """f32 -> e4m3fn codes: round to nearest even on the representable set,
    saturate to +-448, NaN -> 0x7F (emmy/compiler/dtype.py:250-270).

    Stated arithmetically rather than by table search: a magnitude with binary
    exponent e (floored at the subnormal exponent -6) sits on a grid of pitch
    2^(e-3); rint() onto that grid is round-to-nearest-even because adjacent
    codes alternate in their low mantissa bit."""
    with np.errstate(invalid="ignore"):
        x = np.asarray(values, dtype=np.float64)
    nan = np.isnan(x)
    a = np.where(nan, 0.0, np.abs(x))
    _, ex = np.frexp(a)  # a = m * 2^ex, m in [0.5, 1)  ->  floor(log2 a) = ex - 1
    e = np.maximum(ex - 1, -6)
    pitch = np.ldexp(1.0, e - 3)
    r = np.minimum(np.rint(a / pitch) * pitch, E4M3_MAX)
    # value -> code
    _, rex = np.frexp(r)
    re = np.maximum(rex - 1, -6)
    steps = np.rint(r / np.ldexp(1.0, re - 3)).astype(np.int64)  # 0..15: mantissa with the implicit bit
    normal = steps >= 8
    code = np.where(normal, ((re + 7) << 3) | (steps - 8), steps).astype(np.uint8)
    code = code | (np.signbit(x).astype(np.uint8) << 7)
    return np.where(nan, np.uint8(0x7F), code).astype(np.uint8)


# ---------------------------------------------------------------------------
# FP4 e2m1 (packed pairs)
# ---------------------------------------------------------------------------

E2M1_VALUES = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0], dtype=np.float32
)


def e2m1_decode_pairs(packed) -> np.ndarray:
    """uint8 byte = code(even k) | code(odd k) << 4 -> f32 values, last axis
    doubled (emmy/compiler/dtype.py:301-311)."""
    b = np.asarray(packed)
    assert b.dtype == np.uint8
    out = np.empty((*b.shape[:-1], b.shape[-1] * 2), dtype=np.float32)
    out[..., 0::2] = E2M1_VALUES[b & 0xF]
    out[..., 1::2] = E2M1_VALUES[b >> 4]
    return out


def e2m1_encode(values) -> np.ndarray:
    """f32 -> e2m1 codes 0..15: round to nearest, ties to the even code,
    saturate at +-6 (emmy/compiler/dtype.py:319-337).

    The grid pitch is 0.5 below 2, 1 on [2,4) and 2 on [4,8); rint() on the
    pitch is ties-to-even-code for the same reason as in e4m3_encode."""
    x = np.asarray(values, dtype=np.float64)
    assert not np.isnan(x).any(), "e2m1 has no NaN code"
    a = np.abs(x)
    pitch = np.where(a < 2.0, 0.5, np.where(a < 4.0, 1.0, 2.0))
    r = np.minimum(np.rint(a / pitch) * pitch, 6.0)
    code = np.searchsorted(E2M1_VALUES[:8].astype(np.float64), r).astype(np.uint8)  # exact hits only
    return (code | (np.signbit(x).astype(np.uint8) << 3)).astype(np.uint8)


def e2m1_encode_pairs(values) -> np.ndarray:
    """f32 -> packed e2m1 pairs, last axis halved (emmy/compiler/dtype.py:340-345)."""
    c = e2m1_encode(values)
    assert c.shape[-1] % 2 == 0
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


# ---------------------------------------------------------------------------
# packed int4 (AWQ / GPTQ)
# ---------------------------------------------------------------------------

# Bit offset of logical slot i inside an int32 word
# (emmy/compiler/loader/quant.py:86-133: AWQ is two interleaved lanes of four
# -- pack order 0,2,4,6,1,3,5,7 -- GPTQ one sequential lane of eight).
AWQ_SHIFTS = (0, 16, 4, 20, 8, 24, 12, 28)
GPTQ_SHIFTS = (0, 4, 8, 12, 16, 20, 24, 28)
FORMATS = {
    # name: (shifts, qweight packed along K rows?, zero bias)
    "awq": (AWQ_SHIFTS, False, 0),
    "gptq": (GPTQ_SHIFTS, True, 1),
    # compressed-tensors pack-quantized int4 once its three tensors are transposed into GPTQ's orientation:
    # sequential nibbles down K, zero point as stored (emmy/compiler/loader/quant.py:119-133)
    "ct": (GPTQ_SHIFTS, True, 0),
}


def unpack_int4(words, fmt: str, *, along_rows: bool = False) -> np.ndarray:
    """int32 words -> int8 nibbles in [0,15], eight per word.

    `along_rows` spreads a word down the row axis (GPTQ qweight, [K/8,N] ->
    [K,N]); otherwise along the column axis (AWQ qweight and both families'
    qzeros).  Follows emmy/compiler/loader/quant.py:515-530."""
    w = np.asarray(words)
    if w.ndim != 2 or w.dtype not in (np.dtype(np.int32), np.dtype(np.uint32)):
        raise ValueError(f"packed int4 tensor must be rank-2 int32, got {w.shape} {w.dtype}")
    u = w.view(np.uint32) if w.dtype == np.int32 else w
    shifts = FORMATS[fmt][0]
    rows, cols = u.shape
    if along_rows:
        out = np.empty((rows, 8, cols), dtype=np.int8)
        for i, s in enumerate(shifts):
            out[:, i, :] = (u >> np.uint32(s)) & np.uint32(0xF)
        return out.reshape(rows * 8, cols)
    out = np.empty((rows, cols, 8), dtype=np.int8)
    for i, s in enumerate(shifts):
        out[:, :, i] = (u >> np.uint32(s)) & np.uint32(0xF)
    return out.reshape(rows, cols * 8)


def pack_int4(values, fmt: str, *, along_rows: bool = False) -> np.ndarray:
    """Inverse of unpack_int4 (the packers of the reference's test fixtures,
    tests/compiler/loader/test_quant.py:236-245 and :1025-1036)."""
    v = np.asarray(values).astype(np.uint32)
    shifts = FORMATS[fmt][0]
    if along_rows:
        k, n = v.shape
        assert k % 8 == 0
        g = v.reshape(k // 8, 8, n)
        out = np.zeros((k // 8, n), dtype=np.uint32)
        for i, s in enumerate(shifts):
            out |= g[:, i, :] << np.uint32(s)
    else:
        r, n = v.shape
        assert n % 8 == 0
        g = v.reshape(r, n // 8, 8)
        out = np.zeros((r, n // 8), dtype=np.uint32)
        for i, s in enumerate(shifts):
            out |= g[:, :, i] << np.uint32(s)
    return out.view(np.int32)


def dequant_w4(qweight, qzeros, scales, group_size: int, fmt: str, g_idx=None) -> np.ndarray:
    """Packed int4 linear -> f32 value matrix W[k, n] (the transpose of the HF
    weight): (q - (z + bias)) * s with one group of scales/zeros per
    `group_size` input rows.  Follows emmy/compiler/loader/quant.py:533-555;
    `scales` may be fp16 or bf16-as-f32.

    `g_idx` (int32 [K]) selects the group of every input row explicitly, as a
    GPTQ act-order checkpoint does.  The reference refuses such checkpoints
    (quant.py:384-407), so that branch is PARITY UNPINNED; with g_idx = k //
    group_size it is identical to the pinned branch."""
    _, rows, bias = FORMATS[fmt]
    q = unpack_int4(qweight, fmt, along_rows=rows).astype(np.float32)
    k, n = q.shape
    z = unpack_int4(qzeros, fmt).astype(np.float32) + np.float32(bias)
    s = np.asarray(scales).astype(np.float32)
    groups = z.shape[0]
    g = k if int(group_size) == -1 else int(group_size)
    if g <= 0 or groups * g != k:
        raise ValueError(f"group geometry {groups} x {g} does not cover K={k}")
    if z.shape[1] != n or s.shape != (groups, n):
        raise ValueError(f"sibling geometry mismatch: q={q.shape} z={z.shape} s={s.shape}")
    if g_idx is None:
        return (q - np.repeat(z, g, axis=0)) * np.repeat(s, g, axis=0)
    gi = np.asarray(g_idx).astype(np.int64)
    if gi.shape != (k,) or gi.min() < 0 or gi.max() >= groups:
        raise ValueError("g_idx must be [K] with entries in [0, K/group)")
    return (q - z[gi]) * s[gi]


def cast_weight(w_kn: np.ndarray, dtype: str) -> np.ndarray:
    """The eager path's one rounding of the exact f32 product to the model
    dtype (emmy/compiler/trace/huggingface.py:2908-2910).  Returns the rounded
    values as f32, still in [K, N] orientation."""
    return round_f16(w_kn) if dtype == "f16" else round_bf16(w_kn)


# ---------------------------------------------------------------------------
# FP8 weights
# ---------------------------------------------------------------------------


def dequant_fp8(bits, scale) -> np.ndarray:
    """e4m3 weight [N, K] times a multiplier scale whose shape divides the
    weight's: per tensor, per output channel [N,1] or 2-D blocks
    (emmy/compiler/loader/quant.py:147-170)."""
    w = e4m3_decode(bits)
    s = np.asarray(scale, dtype=np.float32)
    if s.size == 1:
        return w * s.reshape(())
    if s.ndim != w.ndim:
        raise ValueError(f"scale rank {s.ndim} != weight rank {w.ndim}")
    reps = []
    for wd, sd in zip(w.shape, s.shape):
        if sd == 0 or wd % sd:
            raise ValueError(f"scale shape {s.shape} does not divide weight shape {w.shape}")
        reps.append(wd // sd)
    full = s
    for axis, r in enumerate(reps):
        full = np.repeat(full, r, axis=axis)
    return w * full


def quant_fp8_rows(values) -> tuple[np.ndarray, np.ndarray]:
    """Per-row e4m3 quantization: s = max(amax, 1e-12) / 448 (f32), bits =
    e4m3(x / s) with an f32 division.  This is the dynamic activation rule of
    emmy/compiler/loader/quant.py:1655-1768 and, applied to a weight's rows,
    the per-output-channel weight quantizer the synthetic FP8 inputs use."""
    x = np.asarray(values, dtype=np.float32)
    amax = np.maximum(np.abs(x).max(axis=-1, keepdims=True), np.float32(1e-12)).astype(np.float32)
    s = (amax / np.float32(448.0)).astype(np.float32)
    return e4m3_encode((x / s).astype(np.float32)), s


# ---------------------------------------------------------------------------
# NVFP4
# ---------------------------------------------------------------------------

NVFP4_BLOCK = 16


def nvfp4_fused_scale(scale_bits, scale_2) -> np.ndarray:
    """f16( e4m3(scale_bits) * scale_2 ): the single rounding of the two-level
    scale (emmy/compiler/loader/quant.py:173-186)."""
    s2 = np.asarray(scale_2, dtype=np.float32).reshape(())
    return (e4m3_decode(scale_bits) * s2).astype(np.float16)


def dequant_nvfp4(packed, scale_bits, scale_2) -> np.ndarray:
    """NVFP4 weight [N, K/2] bytes + [N, K/16] e4m3 scales + f32 global ->
    f32 values [N, K], exact (emmy/compiler/loader/quant.py:189-197)."""
    vals = e2m1_decode_pairs(packed)
    fused = nvfp4_fused_scale(scale_bits, scale_2).astype(np.float32)
    return vals * np.repeat(fused, NVFP4_BLOCK, axis=-1)


def dequant_mxfp4(blocks, scales) -> np.ndarray:
    """Native MXFP4 storage -> its logical (..., in, out) f32 matrix (emmy/compiler/loader/quant.py:477-496).
    blocks uint8 (..., out, groups, 16): a byte holds the even value in its low nibble and the odd one in its high
    nibble, 32 values to a group; scales uint8 (..., out, groups): a power of two, exponent biased by 127.  The e2m1
    value table is NVFP4's; the product with the power of two is exact, then one cast to f32 (the largest exponents
    overflow to infinity, as in the reference)."""
    b = np.asarray(blocks)
    sc = np.asarray(scales)
    if b.dtype != np.uint8 or sc.dtype != np.uint8:
        raise ValueError("MXFP4 blocks and scales are uint8")
    if b.ndim < 3 or b.shape[-1] != 16 or sc.shape != b.shape[:-1]:
        raise ValueError(f"MXFP4 storage geometry mismatch: blocks {b.shape}, scales {sc.shape}")
    vals = e2m1_decode_pairs(b).astype(np.float64)  # (..., out, groups, 32)
    with np.errstate(over="ignore"):
        dense = np.ldexp(vals, sc.astype(np.int32)[..., None] - 127).reshape(*b.shape[:-2], b.shape[-2] * 32).astype(np.float32)
    return np.swapaxes(dense, -2, -1)


def quant_nvfp4(values) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """f32 [.., K] -> (packed u8 [.., K/2], scale_bits u8 [.., K/16], scale_2
    f32 [1]), the weight quantizer of emmy/compiler/loader/quant.py:206-237:
    scale_2 = max(amax,1e-12)/(6*448); block scale = block amax / 6 stored as
    e4m3 relative to scale_2; codes = e2m1(block / fused), 0 where fused == 0."""
    x = np.asarray(values, dtype=np.float32)
    assert x.shape[-1] % NVFP4_BLOCK == 0
    blocks = x.reshape(*x.shape[:-1], x.shape[-1] // NVFP4_BLOCK, NVFP4_BLOCK)
    amax = max(float(np.abs(x).max()), 1e-12)
    assert amax / 6.0 <= 65504.0, "tensor too large for an f16 fused scale"
    scale_2 = np.float32(amax / (6.0 * 448.0))
    block_scale = np.abs(blocks).max(axis=-1) / 6.0
    scale_bits = e4m3_encode(block_scale / scale_2)
    fused = nvfp4_fused_scale(scale_bits, scale_2).astype(np.float32)[..., None]
    quot = np.divide(blocks, fused, out=np.zeros_like(blocks), where=fused != 0)
    packed = e2m1_encode_pairs(quot).reshape(*x.shape[:-1], x.shape[-1] // 2)
    return packed, scale_bits, np.asarray(scale_2, dtype=np.float32).reshape(1)
