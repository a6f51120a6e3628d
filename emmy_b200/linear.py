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

_REGISTRY: dict[int, object] = {}


def _register(obj) -> int:
    key = id(obj)
    _REGISTRY[key] = obj
    return key


@torch.library.custom_op("emmyq::w4a16_linear", mutates_args=(), device_types="cuda")
def _w4a16_op(x: torch.Tensor, handle: int) -> torch.Tensor:
    return ops.w4a16_linear(x.contiguous(), _REGISTRY[handle])


@_w4a16_op.register_fake
def _(x, handle):
    return x.new_empty((x.shape[0], _REGISTRY[handle].n))


@torch.library.custom_op("emmyq::fp8_linear", mutates_args=(), device_types="cuda")
def _fp8_op(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor) -> torch.Tensor:
    return ops.fp8_linear(x.contiguous(), weight, weight_scale)


@_fp8_op.register_fake
def _(x, weight, weight_scale):
    return x.new_empty((x.shape[0], weight.shape[0]))


@torch.library.custom_op("emmyq::nvfp4_linear", mutates_args=(), device_types="cuda")
def _nvfp4_op(x: torch.Tensor, weight: torch.Tensor, scale_tiled: torch.Tensor, scale_2: torch.Tensor, input_scale: torch.Tensor) -> torch.Tensor:
    return ops_nvfp4.nvfp4_linear(x.contiguous(), weight, scale_tiled, scale_2, input_scale)


@_nvfp4_op.register_fake
def _(x, weight, scale_tiled, scale_2, input_scale):
    return x.new_empty((x.shape[0], weight.shape[0]))


@torch.library.custom_op("emmyq::moe_w4a16", mutates_args=(), device_types="cuda")
def _moe_op(x: torch.Tensor, router_logits: torch.Tensor, handle: int, topk: int) -> torch.Tensor:
    return ops_moe.moe_forward(x.contiguous(), router_logits.float().contiguous(), _REGISTRY[handle], topk)


@_moe_op.register_fake
def _(x, router_logits, handle, topk):
    return torch.empty_like(x)


def _flat(x):
    return x.reshape(-1, x.shape[-1]), x.shape[:-1]


class W4A16Linear(nn.Module):
    """AWQ (`fmt="awq"`) or GPTQ (`fmt="gptq"`, optional act-order `g_idx`) int4 linear.

    Buffers keep the checkpoint names and layouts; `finalize()` repacks them once on the device (load time) and
    frees the originals unless `keep_checkpoint=True`."""

    def __init__(self, in_features: int, out_features: int, group_size: int = 128, fmt: str = "awq", act_order: bool = False,
                 scale_dtype=torch.float16):
        super().__init__()
        if fmt not in ("awq", "gptq"):
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
        self._packed = None
        self._handle = None

    def finalize(self, keep_checkpoint: bool = False) -> "W4A16Linear":
        self._packed = ops.w4_repack(self.qweight, self.qzeros, self.scales, self.group_size, self.fmt, g_idx=self.g_idx)
        self._handle = _register(self._packed)
        if not keep_checkpoint:
            self.qweight = self.qzeros = self.scales = None
        return self

    def dequantized_weight(self, dtype=torch.float16) -> torch.Tensor:
        """The HF-orientation weight the reference's eager twin would load, bit for bit."""
        return ops.dequant_w4(self.qweight, self.qzeros, self.scales, self.group_size, self.fmt, g_idx=self.g_idx, out_dtype=dtype,
                              transpose=True)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._packed is None:
            self.finalize(keep_checkpoint=True)
        x2, lead = _flat(x)
        return _w4a16_op(x2, self._handle).reshape(*lead, self.out_features)


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

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x2, lead = _flat(x)
        return _fp8_op(x2, self.weight, self.weight_scale).reshape(*lead, self.out_features)


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
        self._tiled = None

    def finalize(self) -> "NVFP4Linear":
        self._tiled = ops_nvfp4.nvfp4_tile_weight_scales(self.weight_scale, self.in_features)
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._tiled is None:
            self.finalize()
        x2, lead = _flat(x)
        y = _nvfp4_op(x2, self.weight, self._tiled, self.weight_scale_2.reshape(1), self.input_scale.reshape(1))
        return y.reshape(*lead, self.out_features)


class QuantMoE(nn.Module):
    """Routed MoE block on AWQ experts.  Expert program inputs keep the reference's names and meaning
    (`w_gate_up` = gate rows then up rows, `w_down`; emmy/compiler/trace/huggingface.py:1702-1717), here as the
    stacked int4 triplets of each."""

    def __init__(self, top_k: int):
        super().__init__()
        self.top_k = top_k
        self._weights = None
        self._handle = None

    def load_experts(self, w_gate_up, w_down, group_size: int = 128, fmt: str = "awq") -> "QuantMoE":
        self._weights = ops_moe.moe_repack(w_gate_up, w_down, group_size, fmt)
        self._handle = _register(self._weights)
        return self

    def forward(self, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        x2, lead = _flat(x)
        return _moe_op(x2, router_logits.reshape(-1, router_logits.shape[-1]), self._handle, self.top_k).reshape(*lead, x.shape[-1])
