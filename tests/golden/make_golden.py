"""Regenerate tests/golden/quant_golden.npz from the reference's own numpy code.

Run in a container where the reference project is checked out:

    python tests/golden/make_golden.py /path/to/reference

Only two reference files are needed, emmy/compiler/dtype.py and
emmy/compiler/loader/quant.py; they are loaded by path behind empty stand-ins
for the packages they import (the rest of the reference needs native
extensions that are not built here).  The inputs are seeded, the outputs are
whatever the reference's functions return, unmodified.  The result is a small
.npz the test-suite reads; the reference itself is never needed at test time.
"""

from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np


def load_reference(root: Path):
    def stub(name, **attrs):
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        m.__path__ = []  # behaves as a package
        sys.modules[name] = m
        return m

    for pkg in ("emmy", "emmy.compiler", "emmy.compiler.ir", "emmy.compiler.loader"):
        stub(pkg)

    class Wire:
        def __init_subclass__(cls, **kw):
            pass

    stub("emmy.compiler.wire", Wire=Wire)
    stub("emmy.compiler.graph", Graph=type("Graph", (), {}))
    stub("emmy.compiler.ir.base", ConstantOp=type("ConstantOp", (), {}))
    stub("emmy.compiler.loader.exl3", HAD_BLOCK=128, decode_trellis=None, fold_hadamard=None)

    def by_path(name, rel):
        spec = importlib.util.spec_from_file_location(name, root / rel)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
        return mod

    d = by_path("emmy.compiler.dtype", "emmy/compiler/dtype.py")
    q = by_path("emmy.compiler.loader.quant", "emmy/compiler/loader/quant.py")
    return d, q


def pack(values, shifts, along_rows):
    v = np.asarray(values).astype(np.uint32)
    if along_rows:
        g = v.reshape(v.shape[0] // 8, 8, v.shape[1])
        out = np.zeros((g.shape[0], g.shape[2]), np.uint32)
        for i, s in enumerate(shifts):
            out |= g[:, i, :] << np.uint32(s)
    else:
        g = v.reshape(v.shape[0], v.shape[1] // 8, 8)
        out = np.zeros(g.shape[:2], np.uint32)
        for i, s in enumerate(shifts):
            out |= g[:, :, i] << np.uint32(s)
    return out.view(np.int32)


def main(root: str) -> None:
    d, q = load_reference(Path(root))
    rng = np.random.default_rng(2024)
    out: dict[str, np.ndarray] = {}

    # --- codecs -----------------------------------------------------------
    out["e4m3_table"] = d.decode_f8(np.arange(256, dtype=np.uint8), "f8e4m3")
    edge = np.array(
        [0.0, -0.0, 2.0**-9, 2.0**-10, 1.5 * 2.0**-10, 2.0**-6, 17.0, 18.0, 19.0, 447.9, 448.0, 463.9, 464.0, 500.0, 1e9, -1e9, np.nan],
        dtype=np.float32,
    )
    enc_in = np.concatenate(
        [edge, (rng.standard_normal(4096) * 100).astype(np.float32), (rng.standard_normal(2048) * 0.01).astype(np.float32),
         np.linspace(-470, 470, 4001, dtype=np.float32)]
    )
    out["e4m3_encode_in"] = enc_in
    out["e4m3_encode_out"] = d.encode_f8(enc_in, "f8e4m3")
    f4_in = np.concatenate([np.linspace(-7, 7, 1121, dtype=np.float32), (rng.standard_normal(2048) * 2).astype(np.float32)])
    out["e2m1_encode_in"] = f4_in
    out["e2m1_encode_out"] = d.encode_f4(f4_in)
    bytes_ = np.arange(256, dtype=np.uint8).reshape(1, 256)
    out["e2m1_pairs_decode"] = d.decode_f4x2(bytes_)
    bf_in = np.concatenate([(rng.standard_normal(4096) * 3).astype(np.float32), np.array([1.00390625, 1.01171875, 3.3895e38], np.float32)])
    out["bf16_in"] = bf_in
    out["bf16_bits"] = d.encode_bf16(bf_in)

    # --- packed int4 ------------------------------------------------------
    out["awq_shifts"] = np.array(q._AWQ4.shifts, dtype=np.int32)
    out["gptq_shifts"] = np.array(q._GPTQ4.shifts, dtype=np.int32)
    for name, layout, k, n, g in (("awq", q._AWQ4, 256, 64, 128), ("gptq", q._GPTQ4, 256, 64, 128), ("awq_g32", q._AWQ4, 64, 32, 32), ("gptq_g32", q._GPTQ4, 64, 32, 32)):
        ints = rng.integers(0, 16, (k, n))
        zeros = rng.integers(0, 15 if layout.zero_bias else 16, (k // g, n))
        scales = rng.uniform(1e-3, 2e-2, (k // g, n)).astype(np.float16)
        qw = pack(ints, layout.shifts, layout.rows)
        qz = pack(zeros, layout.shifts, False)
        out[f"{name}_qweight"], out[f"{name}_qzeros"], out[f"{name}_scales"] = qw, qz, scales
        out[f"{name}_group"] = np.array(g)
        out[f"{name}_unpacked"] = q.unpack_int4(qw, layout, rows=layout.rows)
        out[f"{name}_zeros_unpacked"] = q.unpack_int4(qz, layout)
        out[f"{name}_dequant"] = q.dequantize_packed_int4(qw, qz, scales, g, layout=layout)

    # --- fp8 weights ------------------------------------------------------
    bits = rng.integers(0, 256, (16, 64)).astype(np.uint8)
    bits[bits == 0x7F] = 0
    bits[bits == 0xFF] = 0x80
    s_ch = rng.uniform(1e-4, 1e-2, (16, 1)).astype(np.float32)
    s_blk = rng.uniform(1e-4, 1e-2, (2, 4)).astype(np.float32)
    out["fp8_bits"], out["fp8_scale_channel"], out["fp8_scale_block"] = bits, s_ch, s_blk
    out["fp8_dequant_channel"] = q.dequantize(d.decode_f8(bits, "f8e4m3"), s_ch)
    out["fp8_dequant_block"] = q.dequantize(d.decode_f8(bits, "f8e4m3"), s_blk)
    out["fp8_dequant_tensor"] = q.dequantize(d.decode_f8(bits, "f8e4m3"), np.array([0.0625], np.float32))

    # --- nvfp4 ------------------------------------------------------------
    w = (rng.standard_normal((12, 128)) * 0.02).astype(np.float32)
    w[3, 16:32] = 0.0
    packed, sbits, s2 = q.quantize_nvfp4(w)
    out["nvfp4_in"], out["nvfp4_packed"], out["nvfp4_scale_bits"], out["nvfp4_scale_2"] = w, packed, sbits, s2
    out["nvfp4_dequant"] = q.dequantize_nvfp4(packed, sbits, s2)
    out["nvfp4_fused"] = q.fuse_nvfp4_scales(sbits, s2)
    rpacked = rng.integers(0, 256, (6, 32)).astype(np.uint8)
    rsb = rng.integers(0, 0x7F, (6, 4)).astype(np.uint8)
    out["nvfp4_rand_packed"], out["nvfp4_rand_scale_bits"] = rpacked, rsb
    out["nvfp4_rand_dequant"] = q.dequantize_nvfp4(rpacked, rsb, np.array(0.03125, np.float32))

    # --- static NVFP4 activation quantize, composed from the reference's
    #     primitives in the order tests/compiler/loader/test_quant.py:1776-1784 uses
    x = rng.standard_normal((8, 64)).astype(np.float32)
    x[1, :16] = 0.0
    s2a = np.float32(max(float(np.abs(x).max()), 1e-12) / (6.0 * 448.0))
    blocks = x.reshape(8, -1, 16)
    ratio = (np.abs(blocks).max(axis=-1) * (np.float32(1) / np.float32(6))) * (np.float32(1) / s2a)
    a_sbits = d.encode_f8(ratio, "f8e4m3")
    fused = d.decode_f8(a_sbits, "f8e4m3") * s2a
    quot = blocks / np.maximum(fused[..., None], np.float32(1e-12))
    a_packed = d.encode_f4x2(quot.reshape(x.shape))
    out["act4_in"], out["act4_s2"] = x, np.array([s2a], np.float32)
    out["act4_packed"], out["act4_scale_bits"] = a_packed, a_sbits
    out["act4_round_trip"] = q.dequantize_nvfp4(a_packed, a_sbits, s2a.reshape(1))

    # --- dynamic FP8 activation, composed from the reference's primitives in
    #     the order emmy/compiler/loader/quant.py:1684-1735 spells them
    xa = rng.standard_normal((8, 96)).astype(np.float32)
    xa[2] = 0.0
    amax = np.maximum(np.abs(xa).max(axis=-1, keepdims=True), np.float32(1e-12))
    sx = (amax / np.float32(448.0)).astype(np.float32)
    out["act8_in"], out["act8_scale"] = xa, sx
    out["act8_bits"] = d.encode_f8((xa / sx).astype(np.float32), "f8e4m3")

    # --- MXFP4 (own generator: the arrays above keep their values) ------------
    rng4 = np.random.default_rng(1234)
    mx_blocks = rng4.integers(0, 256, (24, 6, 16)).astype(np.uint8)   # (out, groups, 16): 24 channels, 192 inputs
    mx_scales = rng4.integers(112, 136, (24, 6)).astype(np.uint8)
    mx_scales[0, 0], mx_scales[1, 1], mx_scales[2, 2] = 0, 254, 127   # the smallest and the largest exponent, and 2^0
    out["mxfp4_blocks"], out["mxfp4_scales"] = mx_blocks, mx_scales
    out["mxfp4_decoded"] = q.decode_mxfp4(mx_blocks, mx_scales)          # (in, out) f32

    dest = Path(__file__).with_name("quant_golden.npz")
    np.savez_compressed(dest, **out)
    print(f"wrote {dest} ({dest.stat().st_size} bytes, {len(out)} arrays)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to a checkout of the reference project>")
    main(sys.argv[1])
