"""Mixture-of-experts operator calls on torch CUDA tensors (W4A16 experts)."""

from __future__ import annotations

import ctypes as C

import torch

from . import lib as L
from .ops import _DTYPE, _FMT, _need_cuda, _ptr, _stream


class MoEWeights:
    """E experts' repacked int4 weights, stacked expert-major on the device.

    gate_up: K = hidden, N = 2 * intermediate (gate columns then up columns, the w_gate_up layout of
    emmy/compiler/trace/huggingface.py:2110-2141 transposed to [K, N]); down: K = intermediate, N = hidden."""

    __slots__ = ("gate_up", "down", "experts", "hidden", "inter", "group", "scale_dtype")


def _repack_stack(qweight, qzeros, scales, group, fmt):
    """qweight [E, ...], qzeros [E, ...], scales [E, K/G, N] -> one uint8 blob of E repacked experts."""
    lib = L.load()
    e = qweight.shape[0]
    if fmt == "awq":
        k, n = qweight.shape[1], qweight.shape[2] * 8
    else:
        k, n = qweight.shape[1] * 8, qweight.shape[2]
    a, c = C.c_size_t(), C.c_size_t()
    L.check(lib.eq_w4_repack_sizes(k, n, group, C.byref(a), C.byref(c)))
    blob = torch.empty(e * a.value, dtype=torch.uint8, device=qweight.device)
    # the whole stack in two launches
    L.check(lib.eq_w4_repack_stack(_FMT[fmt], _ptr(qweight.contiguous()), _ptr(qzeros.contiguous()), _ptr(scales.contiguous()), e, k, n, group,
                                   _ptr(blob), _stream()))
    return blob, k, n


def moe_repack(gate_up, down, group: int = 128, fmt: str = "awq") -> MoEWeights:
    """gate_up / down: (qweight, qzeros, scales) with a leading expert axis, checkpoint layouts otherwise."""
    for t in (*gate_up, *down):
        _need_cuda(t)
    w = MoEWeights()
    w.gate_up, h, n2 = _repack_stack(*gate_up, group, fmt)
    w.down, i, h2 = _repack_stack(*down, group, fmt)
    if h != h2 or n2 != 2 * i:
        raise ValueError(f"expert shapes do not chain: gate_up {h}x{n2}, down {i}x{h2}")
    w.experts, w.hidden, w.inter, w.group, w.scale_dtype = gate_up[0].shape[0], h, i, group, gate_up[2].dtype
    return w


def moe_route(logits: torch.Tensor, topk: int, renorm: bool = True):
    """logits f32 [T, E] -> (ids int32 [T, k], scores f32 [T, k]), picks sorted by ascending expert id."""
    _need_cuda(logits)
    t, e = logits.shape
    ids = torch.empty((t, topk), dtype=torch.int32, device=logits.device)
    scores = torch.empty((t, topk), dtype=torch.float32, device=logits.device)
    L.check(L.load().eq_moe_route(_ptr(logits), t, e, topk, int(renorm), _ptr(ids), _ptr(scores), _stream()))
    return ids, scores


def moe_workspace(t: int, w: MoEWeights, topk: int, device) -> torch.Tensor:
    need = L.load().eq_moe_workspace_bytes(t, w.experts, topk, w.hidden, w.inter)
    return torch.zeros(max(need, 256), dtype=torch.uint8, device=device)


def moe_experts(x, expert_ids, w: MoEWeights, src_row=None, workspace=None, out=None):
    """Grouped expert FFN: row r = expert expert_ids[r] applied to x[src_row[r]] (or x[r])."""
    _need_cuda(x, expert_ids, src_row)
    r = expert_ids.numel()
    y = out if out is not None else torch.empty((r, w.hidden), dtype=x.dtype, device=x.device)
    ws = workspace if workspace is not None else moe_workspace(r, w, 1, x.device)
    L.check(
        L.load().eq_moe_experts_w4a16(
            _ptr(w.gate_up), _ptr(w.down), _DTYPE[w.scale_dtype], w.experts, w.hidden, w.inter, w.group, _ptr(x), _ptr(src_row),
            _ptr(expert_ids), r, _DTYPE[x.dtype], _ptr(y), _ptr(ws), ws.numel(), _stream(),
        )
    )
    return y


def moe_combine(out_rows, scores, topk: int, out=None):
    _need_cuda(out_rows, scores)
    t, h = scores.shape[0], out_rows.shape[1]
    y = out if out is not None else torch.empty((t, h), dtype=out_rows.dtype, device=out_rows.device)
    L.check(L.load().eq_moe_combine(_ptr(out_rows), _ptr(scores), t, topk, h, _DTYPE[out_rows.dtype], _ptr(y), _stream()))
    return y


def moe_forward(x, router_logits, w: MoEWeights, topk: int, workspace=None, out=None):
    """One routed MoE layer: y[T, H] from x[T, H] and f32 router logits [T, E]."""
    _need_cuda(x, router_logits)
    t = x.shape[0]
    y = out if out is not None else torch.empty((t, w.hidden), dtype=x.dtype, device=x.device)
    ws = workspace if workspace is not None else moe_workspace(t, w, topk, x.device)
    L.check(
        L.load().eq_moe_w4a16(
            _ptr(w.gate_up), _ptr(w.down), _DTYPE[w.scale_dtype], w.experts, topk, w.hidden, w.inter, w.group, _ptr(x),
            _ptr(router_logits), t, _DTYPE[x.dtype], _ptr(y), _ptr(ws), ws.numel(), _stream(),
        )
    )
    return y


def moe_status(workspace, t: int, w: MoEWeights, topk: int) -> None:
    L.check(L.load().eq_moe_status(_ptr(workspace), t, w.experts, topk, w.hidden, w.inter, _stream()))
