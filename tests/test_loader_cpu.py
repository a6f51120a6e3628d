"""The checkpoint-facing loader's recognition rules on synthetic checkpoints written into tmp_path (no GPU): the
reference's own pattern, tests/compiler/loader/test_quant.py:201-209."""

import json

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

from emmy_b200 import loader
from oracle import formats as fm
from oracle import synth


def write_checkpoint(path, tensors, quantization_config=None, shards=1):
    path.mkdir(parents=True, exist_ok=True)
    cfg = {"model_type": "llama"}
    if quantization_config is not None:
        cfg["quantization_config"] = quantization_config
    (path / "config.json").write_text(json.dumps(cfg))
    keys = sorted(tensors)
    if shards == 1:
        save_file({k: tensors[k].clone().contiguous() for k in keys}, str(path / "model.safetensors"))
        return
    weight_map = {}
    for i in range(shards):
        part = {k: tensors[k].clone().contiguous() for k in keys[i::shards]}
        name = f"model-{i + 1:05d}-of-{shards:05d}.safetensors"
        save_file(part, str(path / name))
        weight_map.update({k: name for k in part})
    (path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))


def awq_tensors(prefix, k, n, seed=0):
    qw, qz, sc = synth.awq_linear(k, n, seed=seed)
    return {f"{prefix}.qweight": torch.from_numpy(qw), f"{prefix}.qzeros": torch.from_numpy(qz), f"{prefix}.scales": torch.from_numpy(sc)}


def test_awq_and_gptq_recognition(tmp_path):
    t = awq_tensors("model.layers.0.mlp.down_proj", 256, 64)
    t["model.norm.weight"] = torch.ones(64)
    write_checkpoint(tmp_path / "awq", t, {"quant_method": "awq", "bits": 4, "group_size": 128, "zero_point": True, "version": "gemm"}, shards=2)
    specs = loader.scan(tmp_path / "awq")
    assert list(specs) == ["model.layers.0.mlp.down_proj"]
    s = specs["model.layers.0.mlp.down_proj"]
    assert (s.family, s.in_features, s.out_features, s.group_size) == ("awq", 256, 64, 128)

    qw, qz, sc, gi = synth.gptq_linear(256, 64, seed=1)
    g = {"m.qweight": torch.from_numpy(qw), "m.qzeros": torch.from_numpy(qz), "m.scales": torch.from_numpy(sc), "m.g_idx": torch.from_numpy(gi)}
    write_checkpoint(tmp_path / "gptq", g, {"quant_method": "gptq", "bits": 4, "group_size": 128, "sym": True, "desc_act": True})
    s = loader.scan(tmp_path / "gptq")["m"]
    assert (s.family, s.in_features, s.out_features) == ("gptq", 256, 64) and s.keys["g_idx"] == "m.g_idx"


@pytest.mark.parametrize("qc", [
    {"quant_method": "awq", "bits": 8, "group_size": 128},
    {"quant_method": "awq", "bits": 4, "version": "gemv"},
    {"quant_method": "awq", "bits": 4, "zero_point": False},
    {"quant_method": "gptq", "bits": 4, "sym": False},
    {"quant_method": "gptq", "bits": 8, "sym": True},
    {"quant_method": "gptq", "bits": 4, "sym": True, "checkpoint_format": "gptq_v2"},
    {"quant_method": "compressed-tensors", "format": "pack-quantized", "config_groups": {"g": {"weights": {"type": "int", "num_bits": 4, "group_size": 128, "symmetric": True}}}},
])
def test_unsupported_packed_variants_raise(qc):
    """A variant this decode does not implement must not load silently with every weight off by a scale unit
    (tests/compiler/loader/test_quant.py:1261-1268 pins the same refusals, act-order excepted)."""
    with pytest.raises(ValueError, match="unsupported"):
        loader.packed_int4_family(qc)


def test_missing_sibling_raises(tmp_path):
    t = awq_tensors("m", 128, 32)
    del t["m.scales"]
    write_checkpoint(tmp_path, t, {"quant_method": "awq", "bits": 4, "group_size": 128})
    with pytest.raises(ValueError, match="missing"):
        loader.scan(tmp_path)


def test_compressed_tensors_int4_is_gptq_transposed(tmp_path):
    """Stored transposed with zero points as they stand: transposing all three gives GPTQ's layout
    (emmy/compiler/loader/quant.py:119-133; tests/compiler/loader/test_quant.py:1113-1258)."""
    rng = np.random.default_rng(0)
    k, n, g = 256, 32, 128
    q = rng.integers(0, 16, (k, n), dtype=np.int32)
    z = rng.integers(0, 16, (k // g, n), dtype=np.int32)
    s = fm.round_bf16(rng.uniform(1e-3, 2e-2, (k // g, n)).astype(np.float32))
    packed = fm.pack_int4(q, "ct", along_rows=True)   # [K/8, N] in GPTQ orientation
    zeros = fm.pack_int4(z, "ct")                      # [K/G, N/8]
    t = {"m.weight_packed": torch.from_numpy(np.ascontiguousarray(packed.T)), "m.weight_zero_point": torch.from_numpy(np.ascontiguousarray(zeros.T)),
         "m.weight_scale": torch.from_numpy(np.ascontiguousarray(s.T)).bfloat16(), "m.weight_shape": torch.tensor([n, k])}
    qc = {"quant_method": "compressed-tensors", "format": "pack-quantized",
          "config_groups": {"g0": {"weights": {"type": "int", "num_bits": 4, "group_size": g, "symmetric": False}}}}
    write_checkpoint(tmp_path, t, qc)
    spec = loader.scan(tmp_path)["m"]
    assert (spec.family, spec.in_features, spec.out_features, spec.group_size) == ("ct", k, n, g)
    np.testing.assert_array_equal(fm.dequant_w4(packed, zeros, s, g, "ct"), (q - z.repeat(g, 0)).astype(np.float32) * s.repeat(g, 0))


def test_fp8_pairs_skip_rules_and_block_scales(tmp_path):
    f8 = lambda *shape: (torch.randn(*shape) * 0.1).to(torch.float8_e4m3fn)
    t = {
        "model.layers.0.self_attn.q_proj.weight": f8(256, 128), "model.layers.0.self_attn.q_proj.weight_scale": torch.rand(256, 1),
        "model.layers.0.mlp.down_proj.weight": f8(256, 256), "model.layers.0.mlp.down_proj.weight_scale_inv": torch.rand(2, 2),
        "model.layers.0.mlp.up_proj.weight": f8(128, 128), "model.layers.0.mlp.up_proj.weight_scale": torch.rand(1),
        "model.layers.0.mlp.up_proj.input_scale": torch.rand(1),
        "lm_head.weight": f8(128, 128), "lm_head.weight_scale": torch.rand(128, 1),
        "model.layers.1.mlp.gate.weight": f8(128, 128), "model.layers.1.mlp.gate.weight_scale": torch.rand(128, 1),
        "model.embed_tokens.weight": torch.randn(16, 128).bfloat16(),
    }
    qc = {"quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128], "modules_to_not_convert": ["lm_head", "re:.*mlp\\.gate$"]}
    write_checkpoint(tmp_path, t, qc)
    specs = loader.scan(tmp_path)
    assert sorted(specs) == ["model.layers.0.mlp.down_proj", "model.layers.0.mlp.up_proj", "model.layers.0.self_attn.q_proj"]
    assert specs["model.layers.0.self_attn.q_proj"].family == "fp8"
    blk = specs["model.layers.0.mlp.down_proj"]
    assert blk.family == "fp8_block" and blk.block == (128, 128) and blk.keys["weight_scale"].endswith("_scale_inv")
    assert specs["model.layers.0.mlp.up_proj"].keys["input_scale"] == "model.layers.0.mlp.up_proj.input_scale"
    # the skip spellings: exact, dotted suffix, parent module, regex
    assert loader.is_skipped("model.lm_head.weight", ["lm_head"]) and loader.is_skipped("a.b.c.weight", ["a.b"])
    assert loader.is_skipped("x.mlp.gate.weight", ["re:.*gate$"]) and not loader.is_skipped("x.mlp.gate_proj.weight", ["re:.*gate$"])


def test_nvfp4_trio_is_taken_before_the_fp8_pair(tmp_path):
    """A mixed-precision checkpoint answers both declarations; each leaf goes to the family whose stored siblings it has
    (emmy/compiler/loader/quant.py:1545-1557)."""
    w = (np.random.default_rng(0).standard_normal((64, 128)) * 0.02).astype(np.float32)
    packed, sbits, s2 = fm.quant_nvfp4(w)
    t = {
        "m.mlp.down_proj.weight": torch.from_numpy(packed), "m.mlp.down_proj.weight_scale": torch.from_numpy(sbits).view(torch.float8_e4m3fn),
        "m.mlp.down_proj.weight_scale_2": torch.from_numpy(s2), "m.mlp.down_proj.input_scale": torch.tensor([0.01]),
        "m.attn.q_proj.weight": (torch.randn(64, 128) * 0.1).to(torch.float8_e4m3fn), "m.attn.q_proj.weight_scale": torch.rand(64, 1),
    }
    qc = {"quant_method": "modelopt", "quant_algo": "MIXED_PRECISION",
          "config_groups": {"a": {"weights": {"type": "float", "num_bits": 4, "group_size": 16}}, "b": {"weights": {"type": "float", "num_bits": 8}}}}
    write_checkpoint(tmp_path, t, qc)
    specs = loader.scan(tmp_path)
    assert specs["m.mlp.down_proj"].family == "nvfp4" and specs["m.mlp.down_proj"].in_features == 128
    assert specs["m.mlp.down_proj"].keys["input_scale"] == "m.mlp.down_proj.input_scale"
    assert specs["m.attn.q_proj"].family == "fp8"
    assert loader.declares_nvfp4(qc) and loader.declares_fp8(qc)
    assert not loader.declares_nvfp4({"quant_method": "compressed-tensors", "config_groups": {"g": {"weights": {"type": "float", "num_bits": 4, "group_size": 32}}}})
    assert loader.declares_mxfp4({"quant_method": "mxfp4"}) and not loader.declares_mxfp4({"quant_method": "fp8"}) and not loader.declares_mxfp4(None)
    assert not loader.declares_fp8({"quant_method": "modelopt", "quant_algo": "NVFP4"})


def test_unquantized_checkpoint_has_no_quantized_linears(tmp_path):
    write_checkpoint(tmp_path, {"a.weight": torch.randn(8, 8)})
    assert loader.quantization_config(tmp_path) is None and loader.scan(tmp_path) == {}


def test_deinterleave_and_expert_stacking():
    """even/odd gate/up columns -> [gate | up] halves, then E-leading stacks with gate before up
    (emmy/compiler/trace/huggingface.py:1196-1205, 2110-2141)."""
    t = torch.arange(2 * 3 * 8).reshape(2, 3, 8)
    d = loader.deinterleave_gate_up(t)
    assert torch.equal(d[..., :4], t[..., 0::2]) and torch.equal(d[..., 4:], t[..., 1::2])
    mk = lambda v, n: (torch.full((4, n // 8), v, dtype=torch.int32), torch.full((1, n // 8), v, dtype=torch.int32), torch.full((1, n), float(v)).half())
    per = {e: {"gate": mk(10 + e, 16), "up": mk(20 + e, 16), "down": mk(30 + e, 8)} for e in range(3)}
    gate_up, down = loader.stack_experts(per)
    assert gate_up[0].shape == (3, 4, 4) and gate_up[2].shape == (3, 1, 32) and down[0].shape == (3, 4, 1)
    assert torch.equal(gate_up[2][1, 0, :16], torch.full((16,), 11.0).half()) and torch.equal(gate_up[2][1, 0, 16:], torch.full((16,), 21.0).half())
    with pytest.raises(ValueError, match="not 0"):
        loader.stack_experts({0: per[0], 2: per[2]})
    bad = {0: {"gate": mk(1, 16), "down": mk(3, 8)}}
    with pytest.raises(ValueError, match="gate without an up"):
        loader.stack_experts(bad)


def test_scan_experts_groups_by_layer(tmp_path):
    t = {}
    for e in range(2):
        for proj, (k, n) in (("gate_proj", (128, 32)), ("up_proj", (128, 32)), ("down_proj", (128, 128))):
            t.update(awq_tensors(f"model.layers.3.mlp.experts.{e}.{proj}", k, n, seed=e))
    write_checkpoint(tmp_path, t, {"quant_method": "awq", "bits": 4, "group_size": 128})
    groups = loader.scan_experts(loader.scan(tmp_path))
    assert list(groups) == ["model.layers.3.mlp.experts"]
    assert sorted(groups["model.layers.3.mlp.experts"]) == [0, 1] and sorted(groups["model.layers.3.mlp.experts"][1]) == ["down", "gate", "up"]
