"""Checkpoint-facing loader: safetensors shards -> quantized-linear modules on the device.

The reference recognizes a quantized checkpoint from `config.json`'s `quantization_config` and from the sibling tensors
stored beside each weight, and decides per tensor which family it is
(emmy/compiler/loader/quant.py:240-474 the declarations, :782-806 the skip rules, :809-933 the per-key pairing, :1545-1557
the NVFP4 trio before the FP8 pair).  This module restates those rules over a safetensors directory and hands every
recognized linear to the operators of this package:

    packed int4   `<m>.qweight` / `qzeros` / `scales` [/ `g_idx`]   (AWQ GEMM, GPTQ v1)  -> W4A16Linear
                  `<m>.weight_packed` / `weight_zero_point` / `weight_scale`  (compressed-tensors int4, stored transposed)
    NVFP4         `<key>` uint8 + `<key>_scale` (e4m3 bits) + `<key>_scale_2` (f32) [+ `<m>.input_scale`]  -> NVFP4Linear
    FP8           `<key>` float8_e4m3fn + `<key>_scale` | `<key>_scale_inv` (always a multiplier) [+ static
                  `<m>.input_scale` | `<m>.activation_scale`]  -> FP8Linear (per-tensor / per-channel scales) or
                  FP8BlockLinear (2-D block scales)
    routed experts  per-expert `gate_proj` / `up_proj` / `down_proj` modules, or fused `gate_up_proj` tensors with gate and
                  up interleaved on even / odd columns (de-interleaved at load) -> stacked [gate | up] and down, QuantMoE

`scan()` works on the host alone (it reads headers, not tensors) and returns one `LinearSpec` per recognized linear;
`load_linear()` / `load_experts()` read the tensors and build the modules on a CUDA device.  One difference from the
reference, on purpose: a GPTQ checkpoint with `desc_act: true` is refused there (quant.py:384-407) and loaded here, since
the act-order gather is part of this package's W4A16 path.
"""

from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from pathlib import Path

import torch

SKIP_KEYS = ("ignored_layers", "modules_to_not_convert", "ignore")
PACKED_LEAVES = {
    "awq": ("qweight", "qzeros", "scales"),
    "gptq": ("qweight", "qzeros", "scales"),
    "ct": ("weight_packed", "weight_zero_point", "weight_scale"),
}


# ---------------------------------------------------------------------------------------------- declarations


def quantization_config(model_dir) -> dict | None:
    """`config.json`'s `quantization_config`, or None when the checkpoint declares none."""
    cfg = Path(model_dir) / "config.json"
    if not cfg.exists():
        return None
    qc = json.loads(cfg.read_text()).get("quantization_config")
    return qc if isinstance(qc, dict) else None


def _group_weights(qc: dict):
    for entry in (qc.get("config_groups") or {}).values():
        if isinstance(entry, dict) and isinstance(entry.get("weights"), dict):
            yield entry["weights"]


def _has_group(qc: dict, bits: int, kind: str, group_size: int | None = None) -> bool:
    """Whether ANY config group quantizes weights as `kind` at this width (a checkpoint may mix schemes per leaf)."""
    for w in _group_weights(qc):
        if w.get("type") == kind and int(w.get("num_bits") or 0) == bits and (group_size is None or int(w.get("group_size") or 0) == group_size):
            return True
    return False


def declares_fp8(qc: dict | None) -> bool:
    """`quant_method: fp8`, or compressed-tensors / modelopt MIXED_PRECISION with an 8-bit float weight group."""
    if not qc:
        return False
    method = qc.get("quant_method")
    if method == "fp8":
        return True
    if method == "modelopt" and qc.get("quant_algo") != "MIXED_PRECISION":
        return False
    return method in ("compressed-tensors", "modelopt") and _has_group(qc, 8, "float")


def declares_nvfp4(qc: dict | None) -> bool:
    """modelopt NVFP4 (or MIXED_PRECISION with a 4-bit float group of 16), or compressed-tensors with such a group.
    The group size keeps 32-element 4-bit families (MXFP4) out."""
    if not qc:
        return False
    method = qc.get("quant_method")
    if method == "modelopt":
        algo = qc.get("quant_algo")
        return algo == "NVFP4" or (algo == "MIXED_PRECISION" and _has_group(qc, 4, "float", 16))
    return method == "compressed-tensors" and _has_group(qc, 4, "float", 16)


def declares_mxfp4(qc: dict | None) -> bool:
    """The checkpoint's native MXFP4 declaration, `quant_method: mxfp4` (gpt-oss; emmy/compiler/loader/quant.py:330-342).
    This library decodes such tensors (`ops.dequant_mxfp4`) but has no MXFP4 linear."""
    return bool(qc) and qc.get("quant_method") == "mxfp4"


def packed_int4_family(qc: dict | None) -> tuple[str, int] | None:
    """(family, group_size) of a packed-int4 declaration, None when there is none; unsupported variants raise instead
    of loading wrongly, as in the reference (an off-by-one zero convention would shift every weight by a scale unit)."""
    if not qc:
        return None
    method = qc.get("quant_method")
    if method == "awq":
        bits = int(qc.get("bits", qc.get("w_bit", 0)) or 0)
        version = str(qc.get("version", "gemm")).lower()
        if bits != 4 or version != "gemm" or qc.get("zero_point", True) is not True:
            raise ValueError(f"unsupported AWQ checkpoint: needs GEMM int4 with explicit zero points (bits={bits}, version={version!r}, "
                             f"zero_point={qc.get('zero_point')!r})")
        return "awq", int(qc.get("group_size", qc.get("q_group_size", -1)))
    if method == "gptq":
        bits = int(qc.get("bits", 0) or 0)
        fmt = str(qc.get("checkpoint_format", qc.get("format", "gptq"))).lower()
        if bits != 4 or fmt != "gptq" or qc.get("sym", False) is not True:
            raise ValueError(f"unsupported GPTQ checkpoint: needs the symmetric 4-bit v1 layout (bits={bits}, format={fmt!r}, sym={qc.get('sym')!r})")
        return "gptq", int(qc.get("group_size", -1))
    if method == "compressed-tensors":
        group = next((w for w in _group_weights(qc) if w.get("type") == "int" and int(w.get("num_bits") or 0) == 4), None)
        if group is None:
            return None
        fmt = str(qc.get("format", "")).lower()
        gs = int(group.get("group_size") or 0)
        if fmt != "pack-quantized" or gs <= 0 or group.get("symmetric", True) is not False:
            raise ValueError(f"unsupported compressed-tensors int4 checkpoint: needs the asymmetric pack-quantized layout over a positive "
                             f"group (format={fmt!r}, group_size={gs}, symmetric={group.get('symmetric')!r})")
        return "ct", gs
    return None


def skip_patterns(qc: dict | None) -> list[str]:
    """The module patterns a declaration leaves unquantized, every spelling pooled."""
    return [pat for key in SKIP_KEYS for pat in ((qc or {}).get(key) or [])]


def is_skipped(weight_key: str, patterns: list[str]) -> bool:
    """Whether the weight's module is excluded: `re:` entries are regexes on the module path; plain entries match the
    path exactly, as a dotted suffix, or as a parent module."""
    module = weight_key.rsplit(".", 1)[0]
    for pat in patterns:
        if pat.startswith("re:"):
            if re.match(pat[3:], module):
                return True
        elif module == pat or module.endswith("." + pat) or module.startswith(pat + "."):
            return True
    return False


# ---------------------------------------------------------------------------------------------- index and specs


class CheckpointIndex:
    """Key -> shard of a safetensors directory (`model.safetensors.index.json` when present, else every `*.safetensors`),
    with header-only shape / dtype queries and tensor reads."""

    def __init__(self, model_dir):
        from safetensors import safe_open

        self.dir = Path(model_dir)
        self._open = safe_open
        self.shard_of: dict[str, Path] = {}
        idx = self.dir / "model.safetensors.index.json"
        if idx.exists():
            for key, shard in json.loads(idx.read_text())["weight_map"].items():
                self.shard_of[key] = self.dir / shard
        else:
            for shard in sorted(self.dir.glob("*.safetensors")):
                with safe_open(str(shard), framework="pt") as f:
                    for key in f.keys():
                        self.shard_of[key] = shard
        self._meta: dict[str, tuple[str, tuple[int, ...]]] = {}

    def __contains__(self, key: str) -> bool:
        return key in self.shard_of

    def keys(self):
        return self.shard_of.keys()

    def meta(self, key: str) -> tuple[str, tuple[int, ...]]:
        """(safetensors dtype tag, shape) from the shard header."""
        if key not in self._meta:
            with self._open(str(self.shard_of[key]), framework="pt") as f:
                sl = f.get_slice(key)
                self._meta[key] = (sl.get_dtype(), tuple(int(d) for d in sl.get_shape()))
        return self._meta[key]

    def tensor(self, key: str) -> torch.Tensor:
        with self._open(str(self.shard_of[key]), framework="pt") as f:
            return f.get_tensor(key)


@dataclass
class LinearSpec:
    """One recognized quantized linear: its family, the checkpoint keys of its tensors, and its geometry."""

    module: str                       # module path ("model.layers.0.mlp.down_proj")
    family: str                       # "awq" | "gptq" | "ct" | "fp8" | "fp8_block" | "nvfp4"
    keys: dict = field(default_factory=dict)
    in_features: int = 0
    out_features: int = 0
    group_size: int = 0               # packed int4 only
    block: tuple[int, int] | None = None  # fp8_block only: (rows, cols) of one scale block


def _fp8_spec(index, key, scale_key) -> LinearSpec:
    n, k = index.meta(key)[1]
    sshape = index.meta(scale_key)[1]
    count = 1
    for d in sshape:
        count *= d
    module = key.rsplit(".", 1)[0]
    spec = LinearSpec(module, "fp8", {"weight": key, "weight_scale": scale_key}, k, n)
    if count not in (1, n):
        if len(sshape) != 2 or n % sshape[0] or k % sshape[1]:
            raise ValueError(f"FP8 scale {scale_key!r} of shape {sshape} does not divide the weight's {(n, k)}")
        spec.family, spec.block = "fp8_block", (n // sshape[0], k // sshape[1])
    for leaf in ("input_scale", "activation_scale"):
        if f"{module}.{leaf}" in index:
            spec.keys["input_scale"] = f"{module}.{leaf}"
            break
    return spec


def scan(model_dir, index: CheckpointIndex | None = None) -> dict[str, LinearSpec]:
    """Every quantized 2-D linear of the checkpoint, by module path.  Reads headers only."""
    qc = quantization_config(model_dir)
    index = index or CheckpointIndex(model_dir)
    packed = packed_int4_family(qc)
    fp8, fp4 = declares_fp8(qc), declares_nvfp4(qc)
    patterns = skip_patterns(qc)
    specs: dict[str, LinearSpec] = {}
    for key in index.keys():
        if packed is not None and key.endswith("." + PACKED_LEAVES[packed[0]][0]):
            family, group = packed
            leaves = PACKED_LEAVES[family]
            module = key[: -len("." + leaves[0])]
            zeros, scales = f"{module}.{leaves[1]}", f"{module}.{leaves[2]}"
            if zeros not in index or scales not in index:
                raise ValueError(f"packed int4 linear {module!r} is missing {leaves[1]} or {leaves[2]}")
            shape = index.meta(key)[1]
            if family == "awq":
                k, n = shape[0], shape[1] * 8
            elif family == "gptq":
                k, n = shape[0] * 8, shape[1]
            else:  # stored transposed: [N, K / 8]
                n, k = shape[0], shape[1] * 8
            spec = LinearSpec(module, family, {"qweight": key, "qzeros": zeros, "scales": scales}, k, n, k if group == -1 else group)
            if family == "gptq" and f"{module}.g_idx" in index:
                spec.keys["g_idx"] = f"{module}.g_idx"
            specs[module] = spec
            continue
        if len(index.meta(key)[1]) != 2:
            continue  # expert-stacked 3-D parameters are handled by load_experts
        # the NVFP4 trio first: its <key>_scale would otherwise be taken for an FP8 pair
        if fp4 and key + "_scale" in index and key + "_scale_2" in index and not is_skipped(key, list((qc or {}).get("ignore") or [])):
            if index.meta(key)[0] == "U8":
                n, half = index.meta(key)[1]
                module = key.rsplit(".", 1)[0]
                spec = LinearSpec(module, "nvfp4", {"weight": key, "weight_scale": key + "_scale", "weight_scale_2": key + "_scale_2"}, half * 2, n)
                if f"{module}.input_scale" in index:
                    spec.keys["input_scale"] = f"{module}.input_scale"
                specs[module] = spec
            continue
        if fp8 and index.meta(key)[0] == "F8_E4M3" and not is_skipped(key, patterns):
            scale_key = next((k for k in (key + "_scale", key + "_scale_inv") if k in index), None)  # both are multipliers
            if scale_key is not None:
                spec = _fp8_spec(index, key, scale_key)
                specs[spec.module] = spec
    return specs


# ---------------------------------------------------------------------------------------------- materialize


def _bits(t: torch.Tensor) -> torch.Tensor:
    return t.view(torch.uint8) if t.dtype != torch.uint8 else t


def load_linear(index: CheckpointIndex, spec: LinearSpec, device):
    """Reads the spec's tensors and returns the finalized module on `device` (CUDA)."""
    from . import linear as L

    dev = torch.device(device)
    get = lambda name: index.tensor(spec.keys[name]).to(dev)
    if spec.family in ("awq", "gptq", "ct"):
        qweight, qzeros, scales = get("qweight"), get("qzeros"), get("scales")
        fmt = spec.family
        if fmt == "ct":  # stored in torch's (out, in) orientation: transposing all three gives GPTQ's layout
            qweight, qzeros, scales = qweight.t().contiguous(), qzeros.t().contiguous(), scales.t().contiguous()
        if scales.dtype not in (torch.float16, torch.bfloat16):
            scales = scales.to(torch.float16)
        mod = L.W4A16Linear(spec.in_features, spec.out_features, spec.group_size, fmt=fmt, act_order="g_idx" in spec.keys, scale_dtype=scales.dtype)
        mod = mod.to(dev)
        mod.qweight, mod.qzeros, mod.scales = qweight.contiguous(), qzeros.contiguous(), scales.contiguous()
        if "g_idx" in spec.keys:
            mod.g_idx = get("g_idx").to(torch.int32).contiguous()
        return mod.finalize()
    if spec.family == "nvfp4":
        mod = L.NVFP4Linear(spec.in_features, spec.out_features).to(dev)
        mod.weight = _bits(get("weight")).contiguous()
        mod.weight_scale = _bits(get("weight_scale")).contiguous()
        mod.weight_scale_2 = get("weight_scale_2").float().reshape(1)
        if "input_scale" in spec.keys:
            mod.input_scale = get("input_scale").float().reshape(1)
        return mod.finalize()
    if spec.family == "fp8":
        mod = L.FP8Linear(spec.in_features, spec.out_features).to(dev)
        scale = get("weight_scale").float().reshape(-1)
        if scale.numel() == 1:
            scale = scale.expand(spec.out_features)
        mod.load_float8(_bits(get("weight")), scale.contiguous())
        if "input_scale" in spec.keys:
            mod.set_static_input_scale(get("input_scale").float().reshape(1))
        return mod
    if spec.family == "fp8_block":
        mod = L.FP8BlockLinear(spec.in_features, spec.out_features, spec.block).to(dev)
        return mod.load_float8(_bits(get("weight")), get("weight_scale").float().contiguous())
    raise ValueError(f"unknown family {spec.family!r}")


def load_quantized_linears(model_dir, device, only=None) -> dict:
    """module path -> module for every recognized linear (or those whose path `only(path)` accepts)."""
    index = CheckpointIndex(model_dir)
    return {name: load_linear(index, spec, device) for name, spec in scan(model_dir, index).items() if only is None or only(name)}


# ---------------------------------------------------------------------------------------------- routed experts


def deinterleave_gate_up(t: torch.Tensor) -> torch.Tensor:
    """A fused gate-up tensor whose LAST axis alternates gate / up columns -> [gate | up] halves (the layout the
    expert algebra's chunk(2) reads; emmy/compiler/trace/huggingface.py:1196-1205).  Applied alike to packed words,
    scales and zero points of a column-packed family, provided whole words stay whole: use `deinterleave_packed` for
    those."""
    return torch.cat([t[..., 0::2], t[..., 1::2]], dim=-1).contiguous()


def deinterleave_awq_gate_up(qweight, qzeros, scales, group: int):
    """De-interleaves a fused AWQ gate-up linear stored with gate / up on even / odd output columns.  The nibbles are
    unpacked on the device, permuted and packed again (eight columns share a word, so a column permutation cannot be
    done on words)."""
    from . import ops

    def repack(words):
        nib = ops.unpack_int4(words, "awq").to(torch.int32)          # [rows, N] logical order
        nib = deinterleave_gate_up(nib)
        r, n = nib.shape
        g = nib.reshape(r, n // 8, 8)
        out = torch.zeros((r, n // 8), dtype=torch.int32, device=words.device)
        for i, shift in enumerate((0, 16, 4, 20, 8, 24, 12, 28)):     # AWQ's slot order (0, 2, 4, 6, 1, 3, 5, 7)
            out |= g[:, :, i] << shift
        return out

    return repack(qweight), repack(qzeros), deinterleave_gate_up(scales)


def stack_experts(per_expert: dict[int, dict[str, tuple]]):
    """{expert index: {"gate": (qweight, qzeros, scales), "up": (...), "down": (...)}} (or "gate_up" already fused) ->
    (gate_up triple, down triple), each with a leading expert axis and gate columns before up columns: the E-leading
    program inputs of emmy/compiler/trace/huggingface.py:2110-2141.  The expert indices must be 0..E-1 without gaps."""
    order = sorted(per_expert)
    if order != list(range(len(order))):
        raise ValueError(f"experts {order[:4]}... are not 0..{len(order) - 1}")
    gate_up, down = [], []
    for e in order:
        entry = per_expert[e]
        if "gate_up" in entry:
            gate_up.append(entry["gate_up"])
        elif "gate" in entry and "up" in entry:
            gate_up.append(tuple(torch.cat([g, u], dim=-1) for g, u in zip(entry["gate"], entry["up"])))
        else:
            raise ValueError(f"expert {e} has a gate without an up projection (or the reverse)")
        down.append(entry["down"])
    pack = lambda triples: tuple(torch.stack([t[j] for t in triples]).contiguous() for j in range(3))
    return pack(gate_up), pack(down)


_EXPERT_RE = re.compile(r"^(?P<prefix>.*\.experts)\.(?P<e>\d+)\.(?P<proj>gate_proj|up_proj|down_proj|gate_up_proj)$")


def scan_experts(specs: dict[str, LinearSpec]) -> dict[str, dict[int, dict[str, LinearSpec]]]:
    """Groups the per-expert linears of `scan()` by their `...experts` prefix: {prefix: {expert: {"gate" | "up" | "down" |
    "gate_up": spec}}}."""
    out: dict = {}
    for name, spec in specs.items():
        m = _EXPERT_RE.match(name)
        if m:
            out.setdefault(m["prefix"], {}).setdefault(int(m["e"]), {})[m["proj"].replace("_proj", "")] = spec
    return out


def load_experts(index: CheckpointIndex, experts: dict[int, dict[str, LinearSpec]], device, top_k: int, interleaved_gate_up: bool = False):
    """One MoE layer's routed experts (AWQ int4) -> QuantMoE.  `interleaved_gate_up`: the fused gate_up_proj tensors hold
    gate and up on even / odd columns and are de-interleaved first."""
    from . import linear as L

    dev = torch.device(device)
    per: dict = {}
    group = None
    for e, projs in experts.items():
        entry = {}
        for role, spec in projs.items():
            if spec.family != "awq":
                raise ValueError(f"expert {e} {role}: the grouped expert kernels take AWQ int4 weights, got {spec.family}")
            group = spec.group_size
            triple = tuple(index.tensor(spec.keys[k]).to(dev) for k in ("qweight", "qzeros", "scales"))
            if role == "gate_up" and interleaved_gate_up:
                triple = deinterleave_awq_gate_up(*triple, group)
            entry[role] = triple
        per[e] = entry
    gate_up, down = stack_experts(per)
    return L.QuantMoE(top_k).to(dev).load_experts(gate_up, down, group, "awq")
