"""Operator-level calls on torch CUDA tensors, each one C-ABI call.

Tensors are lent to the library as raw device pointers on torch's current
stream, as the reference's torch.compile entry lends caller memory by
(name, data_ptr, nbytes) (emmy/dynamo.py:58-68).  Outputs are allocated here
with torch.empty; the kernels allocate nothing.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import lib as L

_DTYPE = {torch.float16: L.EQ_F16, torch.bfloat16: L.EQ_BF16, torch.float32: L.EQ_F32}
_FMT = {"awq": L.EQ_W4_AWQ, "gptq": L.EQ_W4_GPTQ, "ct": L.EQ_W4_CT}


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("emmy_b200 operators take CUDA tensors only; there is no CPU path")
        if t is not None and not t.is_contiguous():
            raise ValueError("emmy_b200 operators take contiguous tensors")


def unpack_int4(words: torch.Tensor, fmt: str, along_rows: bool = False) -> torch.Tensor:
    _need_cuda(words)
    rows, cols = words.shape
    out = torch.empty((rows * 8, cols) if along_rows else (rows, cols * 8), dtype=torch.uint8, device=words.device)
    L.check(L.load().eq_unpack_int4(_FMT[fmt], int(along_rows), _ptr(words), rows, cols, _ptr(out), _stream()))
    return out


def dequant_w4(qweight, qzeros, scales, group_size, fmt, g_idx=None, out_dtype=torch.float16, transpose=False):
    """-> W[K, N] (or the HF orientation [N, K] when `transpose`), rounded once to out_dtype."""
    _need_cuda(qweight, qzeros, scales, g_idx)
    if fmt == "awq":
        k, n = qweight.shape[0], qweight.shape[1] * 8
    else:  # "gptq", and "ct" (compressed-tensors int4 already transposed into GPTQ's orientation)
        k, n = qweight.shape[0] * 8, qweight.shape[1]
    out = torch.empty((n, k) if transpose else (k, n), dtype=out_dtype, device=qweight.device)
    L.check(
        L.load().eq_dequant_w4(
            _FMT[fmt], _ptr(qweight), _ptr(qzeros), _ptr(scales), _DTYPE[scales.dtype], _ptr(g_idx), k, n, group_size,
            _DTYPE[out_dtype], int(transpose), _ptr(out), _stream(),
        )
    )
    return out


def dequant_fp8(bits, scale, out_dtype=torch.float32):
    _need_cuda(bits, scale)
    n, k = bits.shape
    s = scale.reshape(1, 1) if scale.numel() == 1 else scale
    if s.dim() == 1:
        s = s.reshape(-1, 1)
    out = torch.empty((n, k), dtype=out_dtype, device=bits.device)
    L.check(L.load().eq_dequant_fp8(_ptr(bits), _ptr(s), n, k, s.shape[0], s.shape[1], _DTYPE[out_dtype], _ptr(out), _stream()))
    return out


def dequant_nvfp4(packed, scale_bits, scale_2, out_dtype=torch.float32):
    _need_cuda(packed, scale_bits, scale_2)
    n, k = packed.shape[0], packed.shape[1] * 2
    out = torch.empty((n, k), dtype=out_dtype, device=packed.device)
    L.check(L.load().eq_dequant_nvfp4(_ptr(packed), _ptr(scale_bits), _ptr(scale_2), n, k, _DTYPE[out_dtype], _ptr(out), _stream()))
    return out


def dequant_mxfp4(blocks, scales, out_dtype=torch.float32):
    """Native MXFP4 storage (blocks uint8 [N, K/32, 16], scales uint8 [N, K/32]) -> [N, K] values, the stored orientation
    (the reference's decode_mxfp4 returns the transpose)."""
    _need_cuda(blocks, scales)
    if blocks.dim() != 3 or blocks.shape[-1] != 16 or tuple(scales.shape) != tuple(blocks.shape[:-1]):
        raise ValueError(f"MXFP4 storage geometry mismatch: blocks {tuple(blocks.shape)}, scales {tuple(scales.shape)}")
    n, k = blocks.shape[0], blocks.shape[1] * 32
    out = torch.empty((n, k), dtype=out_dtype, device=blocks.device)
    L.check(L.load().eq_dequant_mxfp4(_ptr(blocks.contiguous()), _ptr(scales.contiguous()), n, k, _DTYPE[out_dtype], _ptr(out), _stream()))
    return out


class W4Weight:
    """A repacked int4 weight resident on the device."""

    __slots__ = ("wq", "perm", "k", "n", "group", "scale_dtype", "fmt")

    def nbytes(self) -> int:
        return self.wq.numel() + (self.perm.numel() * 4 if self.perm is not None else 0)


def w4_repack(qweight, qzeros, scales, group_size, fmt, g_idx=None) -> W4Weight:
    _need_cuda(qweight, qzeros, scales, g_idx)
    lib = L.load()
    if fmt == "awq":
        k, n = qweight.shape[0], qweight.shape[1] * 8
    else:
        k, n = qweight.shape[0] * 8, qweight.shape[1]
    a, c = C.c_size_t(), C.c_size_t()
    L.check(lib.eq_w4_repack_sizes(k, n, group_size, C.byref(a), C.byref(c)))
    dev = qweight.device
    w = W4Weight()
    w.wq = torch.empty(a.value, dtype=torch.uint8, device=dev)
    perm = torch.empty(c.value // 4, dtype=torch.int32, device=dev) if g_idx is not None else None
    uses = C.c_int(0)
    L.check(
        lib.eq_w4_repack(
            _FMT[fmt], _ptr(qweight), _ptr(qzeros), _ptr(scales), _ptr(g_idx), k, n, group_size, _ptr(w.wq), _ptr(perm),
            C.byref(uses), _stream(),
        )
    )
    w.perm = perm if uses.value else None
    w.k, w.n, w.group, w.scale_dtype, w.fmt = k, n, (k if group_size == -1 else group_size), scales.dtype, fmt
    return w


def w4_concat(weights: list[W4Weight]) -> W4Weight:
    """Several repacked linears that read the same activations (gate and up, or q / k / v) as ONE linear whose output
    is their outputs side by side: the repacked stream is [column tile][K run], so concatenating along N is concatenating
    the blobs.  One launch then streams all of them behind one prologue -- the reference stores `[gate | up]` as one
    tensor for the same reason (emmy/compiler/trace/huggingface.py:2110-2141).  The parts must agree in K, group size
    and scale dtype, and none may carry a row permutation (scattered act-order groups differ per linear)."""
    first = weights[0]
    for w in weights:
        if (w.k, w.group, w.scale_dtype) != (first.k, first.group, first.scale_dtype) or w.perm is not None:
            raise ValueError("w4_concat: the parts must share K, group size and scale dtype and carry no row permutation")
    out = W4Weight()
    out.wq = torch.cat([w.wq for w in weights])
    out.perm, out.k, out.n, out.group, out.scale_dtype, out.fmt = None, first.k, sum(w.n for w in weights), first.group, first.scale_dtype, first.fmt
    return out


def w4_unpack_repacked(w: W4Weight) -> torch.Tensor:
    out = torch.empty((w.k, w.n), dtype=torch.uint8, device=w.wq.device)
    L.check(L.load().eq_w4_unpack_repacked(_ptr(w.wq), w.k, w.n, _ptr(out), _stream()))
    return out


_workspaces: dict = {}


def w4a16_workspace(m: int, n: int, device, k: int = 1) -> torch.Tensor:
    """A zeroed scratch buffer per (device, stream); grown on demand, reused by calls on that stream."""
    need = L.load().eq_w4a16_workspace_bytes(m, n, k)
    key = (device.index if device.index is not None else torch.cuda.current_device(), torch.cuda.current_stream().cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def w4a16_linear(x: torch.Tensor, w: W4Weight, workspace: torch.Tensor | None = None, out: torch.Tensor | None = None):
    """y[M, N] = x[M, K] @ W, x and y in f16 or bf16."""
    _need_cuda(x)
    m, k = x.shape
    if k != w.k:
        raise ValueError(f"x has {k} features, the weight takes {w.k}")
    y = out if out is not None else torch.empty((m, w.n), dtype=x.dtype, device=x.device)
    ws = workspace if workspace is not None else w4a16_workspace(m, w.n, x.device, w.k)
    L.check(
        L.load().eq_w4a16_linear(
            _ptr(w.wq), _DTYPE[w.scale_dtype], _ptr(w.perm), w.k, w.n, w.group, _ptr(x), m, _DTYPE[x.dtype],
            _ptr(y), _ptr(ws), ws.numel(), _stream(),
        )
    )
    return y


def w4a16_gate_up_swiglu(x: torch.Tensor, w: W4Weight, workspace: torch.Tensor | None = None, out: torch.Tensor | None = None):
    """h[M, I] = act(silu(gate)) * up for a [gate | up] weight (`w4_concat([gate, up])`, or a checkpoint that stores the two
    projections as one tensor): one call, and above 16 rows one kernel (the activation sits in the GEMM's epilogue)."""
    _need_cuda(x)
    m, k = x.shape
    if k != w.k or w.n % 32:
        raise ValueError(f"x has {k} features, the weight {w.k}; the [gate | up] width {w.n} must be a multiple of 32")
    inter = w.n // 2
    h = out if out is not None else torch.empty((m, inter), dtype=x.dtype, device=x.device)
    need = L.load().eq_w4a16_gate_up_workspace_bytes(m, inter, k)
    ws = workspace if workspace is not None else torch.zeros(max(need, 256), dtype=torch.uint8, device=x.device)
    L.check(L.load().eq_w4a16_gate_up_swiglu(_ptr(w.wq), _DTYPE[w.scale_dtype], _ptr(w.perm), w.k, inter, w.group, _ptr(x), m, _DTYPE[x.dtype],
                                             _ptr(h), _ptr(ws), ws.numel(), _stream()))
    return h


def w4a16_status(workspace: torch.Tensor, m: int, n: int) -> None:
    """Raises EmmyqError(EQ_ERR_TIMEOUT) if a bounded device-side wait of an earlier call ran out."""
    L.check(L.load().eq_w4a16_status(_ptr(workspace), m, n, _stream()))


def w4a16_linear_noalloc(x: torch.Tensor, w: W4Weight, out: torch.Tensor):
    """The W4A16 linear for callers that may not allocate: scratch lives inside the library (M <= 16, N <= 32768)
    and `out` must be given.  Calls on one device must not overlap."""
    _need_cuda(x, out)
    m, k = x.shape
    if k != w.k:
        raise ValueError(f"x has {k} features, the weight takes {w.k}")
    L.check(
        L.load().eq_w4a16_linear_noalloc(
            _ptr(w.wq), _DTYPE[w.scale_dtype], _ptr(w.perm), w.k, w.n, w.group, _ptr(x), m, _DTYPE[x.dtype], _ptr(out),
            _stream(),
        )
    )
    return out


# ---------------------------------------------------------------------------------------------- FP8 W8A8


def quant_fp8_per_token(x: torch.Tensor):
    """x [M, K] (f16 / bf16 / f32) -> (bits uint8 [M, K], scale f32 [M, 1])."""
    _need_cuda(x)
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.uint8, device=x.device)
    s = torch.empty((m, 1), dtype=torch.float32, device=x.device)
    L.check(L.load().eq_quant_fp8_per_token(_ptr(x), m, k, _DTYPE[x.dtype], _ptr(q), _ptr(s), _stream()))
    return q, s


def fp8_workspace(m: int, k: int, device) -> torch.Tensor:
    need = L.load().eq_fp8_workspace_bytes(m, k)
    return torch.zeros(max(need, 256), dtype=torch.uint8, device=device)


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, workspace=None, out=None, input_scale=None,
               norm_weight: torch.Tensor | None = None, eps: float = 1e-6):
    """y[M, N] = x @ (weight * scale).T with x quantized per token (or with the static `input_scale`, f32 [1]);
    weight uint8 e4m3 bits [N, K], scale f32 [N].  `norm_weight` ([K], x's dtype): the model's RMSNorm runs inside the
    quantize kernel, y = linear(rmsnorm(x) * norm_weight)."""
    _need_cuda(x, weight, weight_scale, input_scale, norm_weight)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise ValueError(f"x has {k} features, the weight takes {weight.shape[1]}")
    y = out if out is not None else torch.empty((m, n), dtype=x.dtype, device=x.device)
    ws = workspace if workspace is not None else fp8_workspace(m, k, x.device)
    if norm_weight is not None:
        if input_scale is not None or norm_weight.dtype != x.dtype or norm_weight.numel() != k:
            raise ValueError("fp8_linear: norm_weight is [K] in x's dtype and excludes a static input_scale")
        L.check(
            L.load().eq_fp8_linear_rmsnorm(
                _ptr(weight), _ptr(weight_scale), n, k, _ptr(x), _ptr(norm_weight), float(eps), m, _DTYPE[x.dtype], _ptr(y), _ptr(ws), ws.numel(), _stream()
            )
        )
        return y
    if input_scale is not None:
        L.check(
            L.load().eq_fp8_linear_static(
                _ptr(weight), _ptr(weight_scale), n, k, _ptr(x), _ptr(input_scale), m, _DTYPE[x.dtype], _ptr(y), _ptr(ws), ws.numel(), _stream()
            )
        )
        return y
    L.check(
        L.load().eq_fp8_linear(
            _ptr(weight), _ptr(weight_scale), n, k, _ptr(x), m, _DTYPE[x.dtype], _ptr(y), _ptr(ws), ws.numel(), _stream()
        )
    )
    return y


def fp8_status(workspace: torch.Tensor, m: int, k: int) -> None:
    L.check(L.load().eq_fp8_status(_ptr(workspace), m, k, _stream()))


def quant_fp8_per_group(x: torch.Tensor):
    """x [M, K] -> (bits uint8 [M, K], scale f32 [M, K / 128]): the dynamic rule per token and per 128 elements of K."""
    _need_cuda(x)
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.uint8, device=x.device)
    s = torch.empty((m, k // 128), dtype=torch.float32, device=x.device)
    L.check(L.load().eq_quant_fp8_per_group(_ptr(x), m, k, _DTYPE[x.dtype], _ptr(q), _ptr(s), _stream()))
    return q, s


def fp8_block_linear(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, workspace=None, out=None):
    """Block-scaled W8A8: weight uint8 e4m3 bits [N, K], weight_scale f32 [N / 128, K / 128] (a multiplier)."""
    _need_cuda(x, weight, weight_scale)
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or tuple(weight_scale.shape) != (n // 128, k // 128):
        raise ValueError(f"block-scaled FP8: x {tuple(x.shape)}, weight {tuple(weight.shape)}, scale {tuple(weight_scale.shape)} do not fit")
    y = out if out is not None else torch.empty((m, n), dtype=x.dtype, device=x.device)
    need = L.load().eq_fp8_block_workspace_bytes(m, k)
    ws = workspace if workspace is not None else torch.empty(max(need, 256), dtype=torch.uint8, device=x.device)
    L.check(L.load().eq_fp8_block_linear(_ptr(weight), _ptr(weight_scale), n, k, _ptr(x), m, _DTYPE[x.dtype], _ptr(y), _ptr(ws), ws.numel(), _stream()))
    return y


def fp8_block_status(workspace: torch.Tensor, m: int, k: int) -> None:
    L.check(L.load().eq_fp8_block_status(_ptr(workspace), m, k, _stream()))
