"""NVFP4 W4A4 operator calls on torch CUDA tensors (one C-ABI call each)."""

from __future__ import annotations

import torch

from . import lib as L
from .ops import _DTYPE, _need_cuda, _ptr, _stream


def nvfp4_global_scale(x: torch.Tensor) -> torch.Tensor:
    """max(amax |x|, 1e-12) / (6 * 448) as a device f32 [1]."""
    _need_cuda(x)
    m, k = x.shape
    out = torch.empty(1, dtype=torch.float32, device=x.device)
    scratch = torch.empty(1, dtype=torch.int32, device=x.device)
    L.check(L.load().eq_nvfp4_global_scale(_ptr(x), m, k, _DTYPE[x.dtype], _ptr(out), _ptr(scratch), _stream()))
    return out


def quant_nvfp4_weight(values: torch.Tensor):
    """values [N, K] (f32 / f16 / bf16) -> (packed uint8 [N, K/2], scale_bits uint8 [N, K/16], scale_2 f32 [1]): the
    reference's weight quantizer, on the device."""
    _need_cuda(values)
    n, k = values.shape
    packed = torch.empty((n, k // 2), dtype=torch.uint8, device=values.device)
    sf = torch.empty((n, k // 16), dtype=torch.uint8, device=values.device)
    s2 = torch.empty(1, dtype=torch.float32, device=values.device)
    scratch = torch.empty(1, dtype=torch.int32, device=values.device)
    L.check(L.load().eq_quant_nvfp4_weight(_ptr(values), n, k, _DTYPE[values.dtype], _ptr(packed), _ptr(sf), _ptr(s2), _ptr(scratch), _stream()))
    return packed, sf, s2


def quant_nvfp4_act(x: torch.Tensor, input_scale: torch.Tensor, tiled: bool = False):
    """x [M, K] -> (codes uint8 [M, K/2], scale_bits uint8 [M, K/16][, tiled scales])."""
    _need_cuda(x, input_scale)
    m, k = x.shape
    codes = torch.empty((m, k // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty((m, k // 16), dtype=torch.uint8, device=x.device)
    sft = None
    if tiled:
        sft = torch.empty(L.load().eq_nvfp4_tiled_scale_bytes(m, k), dtype=torch.uint8, device=x.device)
    L.check(
        L.load().eq_quant_nvfp4_act(_ptr(x), m, k, _DTYPE[x.dtype], _ptr(input_scale), _ptr(codes), _ptr(sf), _ptr(sft), _stream())
    )
    return (codes, sf, sft) if tiled else (codes, sf)


def nvfp4_tile_scales(scale_bits: torch.Tensor, k: int) -> torch.Tensor:
    """weight_scale [N, K/16] -> the tiled order the tensor path reads (load time)."""
    _need_cuda(scale_bits)
    rows = scale_bits.shape[0]
    out = torch.empty(L.load().eq_nvfp4_tiled_scale_bytes(rows, k), dtype=torch.uint8, device=scale_bits.device)
    L.check(L.load().eq_nvfp4_tile_scales(_ptr(scale_bits), rows, k, _ptr(out), _stream()))
    return out


def nvfp4_tile_weight_scales(scale_bits: torch.Tensor, k: int) -> torch.Tensor:
    """weight_scale [N, K/16] -> the scale blob eq_nvfp4_linear reads (both tile groupings; load time)."""
    _need_cuda(scale_bits)
    rows = scale_bits.shape[0]
    out = torch.empty(L.load().eq_nvfp4_weight_scale_bytes(rows, k), dtype=torch.uint8, device=scale_bits.device)
    L.check(L.load().eq_nvfp4_tile_weight_scales(_ptr(scale_bits), rows, k, _ptr(out), _stream()))
    return out


def nvfp4_workspace(m: int, k: int, device) -> torch.Tensor:
    return torch.zeros(max(L.load().eq_nvfp4_workspace_bytes(m, k), 256), dtype=torch.uint8, device=device)


def nvfp4_linear(x, weight, weight_scale_tiled, weight_scale_2, input_scale, workspace=None, out=None, norm_weight=None, eps: float = 1e-6):
    """y[M, N] for packed e2m1 weight [N, K/2], tiled block scales, f32 weight_scale_2 [1] and input_scale [1].
    `norm_weight` ([K], x's dtype): the model's RMSNorm runs inside the quantize kernel, y = linear(rmsnorm(x) * norm_weight),
    and input_scale is the global scale of those normalised activations."""
    _need_cuda(x, weight, weight_scale_tiled, weight_scale_2, input_scale, norm_weight)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] * 2 != k:
        raise ValueError(f"x has {k} features, the weight takes {weight.shape[1] * 2}")
    y = out if out is not None else torch.empty((m, n), dtype=x.dtype, device=x.device)
    ws = workspace if workspace is not None else nvfp4_workspace(m, k, x.device)
    if norm_weight is not None:
        if norm_weight.dtype != x.dtype or norm_weight.numel() != k:
            raise ValueError("nvfp4_linear: norm_weight is [K] in x's dtype")
        L.check(
            L.load().eq_nvfp4_linear_rmsnorm(
                _ptr(weight), _ptr(weight_scale_tiled), _ptr(weight_scale_2), n, k, _ptr(x), _ptr(norm_weight), float(eps), _ptr(input_scale), m,
                _DTYPE[x.dtype], _ptr(y), _ptr(ws), ws.numel(), _stream(),
            )
        )
        return y
    L.check(
        L.load().eq_nvfp4_linear(
            _ptr(weight), _ptr(weight_scale_tiled), _ptr(weight_scale_2), n, k, _ptr(x), _ptr(input_scale), m, _DTYPE[x.dtype],
            _ptr(y), _ptr(ws), ws.numel(), _stream(),
        )
    )
    return y


def nvfp4_status(workspace: torch.Tensor, m: int, k: int) -> None:
    L.check(L.load().eq_nvfp4_status(_ptr(workspace), m, k, _stream()))
