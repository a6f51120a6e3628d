"""Modules that take a quantized checkpoint's tensors under their own names and run the C-ABI operators.

The reference recognizes a quantized linear by its sibling tensors (`qweight` / `qzeros` / `scales` [/ `g_idx`] for
AWQ and GPTQ, `weight` + `weight_scale` for FP8, `weight` + `weight_scale` + `weight_scale_2` + `input_scale` for
NVFP4: emmy/compiler/loader/quant.py:99-144, 1120-1194) and rewrites the traced graph around them.  Here the same
tensors load into an `nn.Module` whose forward is one operator call; output dtype = activation dtype, as there.
Each forward goes through a `torch.library` custom op with a fake (meta) kernel, so `torch.compile` traces through
the modules without graph breaks (the reference's own entry is the dynamo backend of emmy/dynamo.py:26-70).
"""

from __future__ import annotations

import torch
from torch import nn

from . import ops, ops_moe, ops_nvfp4

# The custom ops take the repacked weights as TENSORS (plus plain ints), never as process-local handles: the packed
# blobs are module buffers, so they follow module.to(), are freed with the module, and a traced graph holds nothing
# but tensors and shapes.


def _w4_weight(wq, perm, k, n, group, scale_bf16) -> ops.W4Weight:
    w = ops.W4Weight()
    w.wq, w.perm, w.k, w.n, w.group = wq, (perm if perm is not None and perm.numel() else None), k, n, group
    w.scale_dtype, w.fmt = (torch.bfloat16 if scale_bf16 else torch.float16), "packed"
    return w


@torch.library.custom_op("emmyq::w4a16_linear", mutates_args=(), device_types="cuda")
def _w4a16_op(x: torch.Tensor, wq: torch.Tensor, perm: torch.Tensor, k: int, n: int, group: int, scale_bf16: bool) -> torch.Tensor:
    return ops.w4a16_linear(x.contiguous(), _w4_weight(wq, perm, k, n, group, scale_bf16))


@_w4a16_op.register_fake
def _(x, wq, perm, k, n, group, scale_bf16):
    return x.new_empty((x.shape[0], n))


@torch.library.custom_op("emmyq::fp8_linear", mutates_args=(), device_types="cuda")
def _fp8_op(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor) -> torch.Tensor:
    return ops.fp8_linear(x.contiguous(), weight, weight_scale)


@_fp8_op.register_fake
def _(x, weight, weight_scale):
    return x.new_empty((x.shape[0], weight.shape[0]))


@torch.library.custom_op("emmyq::fp8_linear_static", mutates_args=(), device_types="cuda")
def _fp8_static_op(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor, input_scale: torch.Tensor) -> torch.Tensor:
    return ops.fp8_linear(x.contiguous(), weight, weight_scale, input_scale=input_scale)


@_fp8_static_op.register_fake
def _(x, weight, weight_scale, input_scale):
    return x.new_empty((x.shape[0], weight.shape[0]))


@torch.library.custom_op("emmyq::fp8_linear_rmsnorm", mutates_args=(), device_types="cuda")
def _fp8_rmsnorm_op(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, weight: torch.Tensor, weight_scale: torch.Tensor) -> torch.Tensor:
    return ops.fp8_linear(x.contiguous(), weight, weight_scale, norm_weight=norm_weight, eps=eps)


@_fp8_rmsnorm_op.register_fake
def _(x, norm_weight, eps, weight, weight_scale):
    return x.new_empty((x.shape[0], weight.shape[0]))


@torch.library.custom_op("emmyq::w4a16_gate_up_swiglu", mutates_args=(), device_types="cuda")
def _w4_gate_up_op(x: torch.Tensor, wq: torch.Tensor, k: int, n: int, group: int, scale_bf16: bool) -> torch.Tensor:
    w = ops.W4Weight()
    w.wq, w.perm, w.k, w.n, w.group, w.scale_dtype, w.fmt = wq, None, k, n, group, torch.bfloat16 if scale_bf16 else torch.float16, "gptq"
    return ops.w4a16_gate_up_swiglu(x.contiguous(), w)


@_w4_gate_up_op.register_fake
def _(x, wq, k, n, group, scale_bf16):
    return x.new_empty((x.shape[0], n // 2))


@torch.library.custom_op("emmyq::fp8_block_linear", mutates_args=(), device_types="cuda")
def _fp8_block_op(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor) -> torch.Tensor:
    return ops.fp8_block_linear(x.contiguous(), weight, weight_scale)


@_fp8_block_op.register_fake
def _(x, weight, weight_scale):
    return x.new_empty((x.shape[0], weight.shape[0]))


@torch.library.custom_op("emmyq::nvfp4_linear", mutates_args=(), device_types="cuda")
def _nvfp4_op(x: torch.Tensor, weight: torch.Tensor, scale_tiled: torch.Tensor, scale_2: torch.Tensor, input_scale: torch.Tensor) -> torch.Tensor:
    return ops_nvfp4.nvfp4_linear(x.contiguous(), weight, scale_tiled, scale_2, input_scale)


@_nvfp4_op.register_fake
def _(x, weight, scale_tiled, scale_2, input_scale):
    return x.new_empty((x.shape[0], weight.shape[0]))


@torch.library.custom_op("emmyq::moe_w4a16", mutates_args=(), device_types="cuda")
def _moe_op(x: torch.Tensor, router_logits: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, experts: int, hidden: int,
            inter: int, group: int, scale_bf16: bool, topk: int) -> torch.Tensor:
    w = ops_moe.MoEWeights()
    w.gate_up, w.down, w.experts, w.hidden, w.inter, w.group = gate_up, down, experts, hidden, inter, group
    w.scale_dtype = torch.bfloat16 if scale_bf16 else torch.float16
    return ops_moe.moe_forward(x.contiguous(), router_logits.float().contiguous(), w, topk)


@_moe_op.register_fake
def _(x, router_logits, gate_up, down, experts, hidden, inter, group, scale_bf16, topk):
    return torch.empty_like(x)


def _flat(x):
    return x.reshape(-1, x.shape[-1]), x.shape[:-1]


class W4A16Linear(nn.Module):
    """AWQ (`fmt="awq"`), GPTQ (`fmt="gptq"`, optional act-order `g_idx`) or compressed-tensors (`fmt="ct"`: its three
    tensors already transposed into GPTQ's orientation) int4 linear.

    Buffers keep the checkpoint names and layouts; `finalize()` repacks them once on the device (load time) and
    frees the originals unless `keep_checkpoint=True`."""

    def __init__(self, in_features: int, out_features: int, group_size: int = 128, fmt: str = "awq", act_order: bool = False,
                 scale_dtype=torch.float16):
        super().__init__()
        if fmt not in ("awq", "gptq", "ct"):
            raise ValueError(f"unknown packed-int4 family {fmt!r}")
        g = in_features if group_size == -1 else group_size
        self.in_features, self.out_features, self.group_size, self.fmt = in_features, out_features, group_size, fmt
        qshape = (in_features, out_features // 8) if fmt == "awq" else (in_features // 8, out_features)
        self.register_buffer("qweight", torch.zeros(qshape, dtype=torch.int32))
        self.register_buffer("qzeros", torch.zeros((in_features // g, out_features // 8), dtype=torch.int32))
        self.register_buffer("scales", torch.zeros((in_features // g, out_features), dtype=scale_dtype))
        if act_order:
            self.register_buffer("g_idx", torch.arange(in_features, dtype=torch.int32) // g)
        else:
            self.g_idx = None
        # the repacked stream (and the row order of scattered act-order groups): derived data, not part of the state dict
        self.register_buffer("packed_wq", None, persistent=False)
        self.register_buffer("packed_perm", None, persistent=False)
        self._scale_bf16 = scale_dtype == torch.bfloat16

    def finalize(self, keep_checkpoint: bool = False) -> "W4A16Linear":
        """Repack on the device (the checkpoint buffers must already be there)."""
        if self.qweight is None:
            raise RuntimeError("W4A16Linear.finalize: the checkpoint tensors were already released")
        if not self.qweight.is_cuda:
            raise RuntimeError("W4A16Linear.finalize: move the module to a CUDA device first; there is no CPU path")
        packed = ops.w4_repack(self.qweight, self.qzeros, self.scales, self.group_size, self.fmt, g_idx=self.g_idx)
        self.packed_wq = packed.wq
        self.packed_perm = packed.perm if packed.perm is not None else torch.empty(0, dtype=torch.int32, device=packed.wq.device)
        self._scale_bf16 = packed.scale_dtype == torch.bfloat16
        if not keep_checkpoint:
            self.qweight = self.qzeros = self.scales = self.g_idx = None
        return self

    def dequantized_weight(self, dtype=torch.float16) -> torch.Tensor:
        """The HF-orientation weight the reference's eager twin would load, bit for bit."""
        return ops.dequant_w4(self.qweight, self.qzeros, self.scales, self.group_size, self.fmt, g_idx=self.g_idx, out_dtype=dtype,
                              transpose=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.packed_wq is None:
            self.finalize(keep_checkpoint=True)
        x2, lead = _flat(x)
        g = self.in_features if self.group_size == -1 else self.group_size
        y = _w4a16_op(x2, self.packed_wq, self.packed_perm, self.in_features, self.out_features, g, self._scale_bf16)
        return y.reshape(*lead, self.out_features)


class FP8Linear(nn.Module):
    """FP8-E4M3 W8A8 linear: `weight` e4m3 bits [N, K] (uint8 carrier), `weight_scale` f32 [N] multiplier, the
    activation quantized per token inside the call."""

    def __init__(self, in_features: int, out_features: int):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight", torch.zeros((out_features, in_features), dtype=torch.uint8))
        self.register_buffer("weight_scale", torch.ones(out_features, dtype=torch.float32))

    def load_float8(self, weight_f8: torch.Tensor, weight_scale: torch.Tensor) -> "FP8Linear":
        self.weight = weight_f8.view(torch.uint8).contiguous()
        self.weight_scale = weight_scale.reshape(-1).float().contiguous()
        return self

    def set_static_input_scale(self, input_scale: torch.Tensor) -> "FP8Linear":
        """A checkpoint's calibrated `input_scale` / `activation_scale` (one f32): activations are then encoded as
        x / scale instead of with a per-token scale (emmy/compiler/loader/quant.py:1818-1905)."""
        self.register_buffer("input_scale", input_scale.float().reshape(1).to(self.weight.device))
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, lead = _flat(x)
        if getattr(self, "input_scale", None) is not None:
            return _fp8_static_op(x2, self.weight, self.weight_scale, self.input_scale).reshape(*lead, self.out_features)
        return _fp8_op(x2, self.weight, self.weight_scale).reshape(*lead, self.out_features)


class FP8BlockLinear(nn.Module):
    """Block-scaled FP8 W8A8 linear (the official 128 x 128 `weight_block_size` form): `weight` e4m3 bits [N, K],
    `weight_scale_inv` f32 [N / 128, K / 128] used as a multiplier, activations quantized per token and per 128
    elements of K inside the call."""

    def __init__(self, in_features: int, out_features: int, block=(128, 128)):
        super().__init__()
        if tuple(block) != (128, 128):
            raise ValueError(f"block-scaled FP8 kernels take 128 x 128 weight blocks, got {tuple(block)}")
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight", torch.zeros((out_features, in_features), dtype=torch.uint8))
        self.register_buffer("weight_scale_inv", torch.ones((out_features // 128, in_features // 128), dtype=torch.float32))

    def load_float8(self, weight_f8: torch.Tensor, weight_scale: torch.Tensor) -> "FP8BlockLinear":
        self.weight = weight_f8.view(torch.uint8).contiguous()
        self.weight_scale_inv = weight_scale.float().contiguous()
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, lead = _flat(x)
        return _fp8_block_op(x2, self.weight, self.weight_scale_inv).reshape(*lead, self.out_features)


class NVFP4Linear(nn.Module):
    """NVFP4 W4A4 linear: `weight` packed e2m1 [N, K/2], `weight_scale` e4m3 bits [N, K/16], `weight_scale_2` and
    `input_scale` f32 scalars."""

    def __init__(self, in_features: int, out_features: int):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("weight", torch.zeros((out_features, in_features // 2), dtype=torch.uint8))
        self.register_buffer("weight_scale", torch.zeros((out_features, in_features // 16), dtype=torch.uint8))
        self.register_buffer("weight_scale_2", torch.ones(1, dtype=torch.float32))
        self.register_buffer("input_scale", torch.ones(1, dtype=torch.float32))
        self.register_buffer("scale_tiled", None, persistent=False)  # weight_scale in the tensor core's atom order

    def finalize(self) -> "NVFP4Linear":
        if not self.weight_scale.is_cuda:
            raise RuntimeError("NVFP4Linear.finalize: move the module to a CUDA device first; there is no CPU path")
        self.scale_tiled = ops_nvfp4.nvfp4_tile_weight_scales(self.weight_scale, self.in_features)
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.scale_tiled is None:
            self.finalize()
        x2, lead = _flat(x)
        y = _nvfp4_op(x2, self.weight, self.scale_tiled, self.weight_scale_2.reshape(1), self.input_scale.reshape(1))
        return y.reshape(*lead, self.out_features)


class QuantMoE(nn.Module):
    """Routed MoE block on AWQ experts.  Expert program inputs keep the reference's names and meaning
    (`w_gate_up` = gate rows then up rows, `w_down`; emmy/compiler/trace/huggingface.py:1702-1717), here as the
    stacked int4 triplets of each."""

    def __init__(self, top_k: int):
        super().__init__()
        self.top_k = top_k
        self.register_buffer("packed_gate_up", None, persistent=False)
        self.register_buffer("packed_down", None, persistent=False)
        self._geometry = None

    def load_experts(self, w_gate_up, w_down, group_size: int = 128, fmt: str = "awq") -> "QuantMoE":
        w = ops_moe.moe_repack(w_gate_up, w_down, group_size, fmt)
        self.packed_gate_up, self.packed_down = w.gate_up, w.down
        self._geometry = (w.experts, w.hidden, w.inter, w.group, w.scale_dtype == torch.bfloat16)
        return self

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        if self._geometry is None:
            raise RuntimeError("QuantMoE.forward: load_experts() has not been called")
        x2, lead = _flat(x)
        y = _moe_op(x2, router_logits.reshape(-1, router_logits.shape[-1]), self.packed_gate_up, self.packed_down, *self._geometry, self.top_k)
        return y.reshape(*lead, x.shape[-1])
