"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (test infrastructure; stand-ins for real checkpoints)."""

from __future__ import annotations

import numpy as np

from . import formats as fm


def awq_linear(k: int, n: int, group: int = 128, seed: int = 0, scale_dtype=np.float16):
    """int4 weights and zero points uniform 0..15 in AWQ order, scales uniform
    [1e-3, 2e-2]."""
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 16, (k, n), dtype=np.int32)
    z = rng.integers(0, 16, (k // group, n), dtype=np.int32)
    s = rng.uniform(1e-3, 2e-2, (k // group, n)).astype(np.float32)
    s = s.astype(scale_dtype) if scale_dtype is np.float16 else fm.round_bf16(s)
    return fm.pack_int4(q, "awq"), fm.pack_int4(z, "awq"), s


def gptq_linear(k: int, n: int, group: int = 128, seed: int = 0, act_order: bool = True):
    """GPTQ v1, symmetric (stored zero 7 = true zero 8), sequential packing
    down K; g_idx[k] = perm[k // group] with perm a random permutation of the
    groups when act_order."""
    rng = np.random.default_rng(seed)
    q = rng.integers(0, 16, (k, n), dtype=np.int32)
    z = np.full((k // group, n), 7, dtype=np.int32)
    s = rng.uniform(1e-3, 2e-2, (k // group, n)).astype(np.float32).astype(np.float16)
    perm = rng.permutation(k // group) if act_order else np.arange(k // group)
    g_idx = perm[np.arange(k) // group].astype(np.int32)
    return fm.pack_int4(q, "gptq", along_rows=True), fm.pack_int4(z, "gptq"), s, g_idx


def activations(m: int, k: int, dtype: str, seed: int = 1) -> np.ndarray:
    """x ~ N(0,1) rounded to the activation dtype, returned as f32."""
    x = np.random.default_rng(seed).standard_normal((m, k)).astype(np.float32)
    return fm.round_f16(x) if dtype == "f16" else fm.round_bf16(x)


def fp8_weight(n: int, k: int, seed: int = 0):
    """W ~ N(0, 0.02) quantized per output channel."""
    w = (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)
    return fm.quant_fp8_rows(w)


def nvfp4_weight(n: int, k: int, seed: int = 0):
    w = (np.random.default_rng(seed).standard_normal((n, k)) * 0.02).astype(np.float32)
    return fm.quant_nvfp4(w)
