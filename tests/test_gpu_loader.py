"""Synthetic checkpoints through the loader onto the GPU: every family's module against the oracle."""

import numpy as np
import pytest
import torch

from oracle import activations as oact
from oracle import formats as fm
from oracle import linear as ol
from oracle import moe as omoe
from oracle import synth
from tests.test_loader_cpu import awq_tensors, write_checkpoint

pytestmark = pytest.mark.gpu
TOL = 2e-2


def close(y, ref):
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= TOL * np.abs(ref).max()


def test_packed_int4_families_from_checkpoints(tmp_path):
    from emmy_b200 import loader

    k, n = 512, 256
    # AWQ
    qw, qz, sc = synth.awq_linear(k, n, seed=3)
    write_checkpoint(tmp_path / "awq", {"m.qweight": torch.from_numpy(qw), "m.qzeros": torch.from_numpy(qz), "m.scales": torch.from_numpy(sc)},
                     {"quant_method": "awq", "bits": 4, "group_size": 128})
    x = synth.activations(5, k, "f16", seed=1)
    mods = loader.load_quantized_linears(tmp_path / "awq", "cuda")
    close(mods["m"](torch.from_numpy(x).half().cuda()), ol.w4a16_linear(x, qw, qz, sc, 128, "awq", "f16"))
    # GPTQ with act-order (the reference refuses desc_act; this path implements the gather)
    qw, qz, sc, gi = synth.gptq_linear(k, n, seed=4)
    write_checkpoint(tmp_path / "gptq", {"m.qweight": torch.from_numpy(qw), "m.qzeros": torch.from_numpy(qz), "m.scales": torch.from_numpy(sc), "m.g_idx": torch.from_numpy(gi)},
                     {"quant_method": "gptq", "bits": 4, "group_size": 128, "sym": True, "desc_act": True})
    mods = loader.load_quantized_linears(tmp_path / "gptq", "cuda")
    close(mods["m"](torch.from_numpy(x).half().cuda()), ol.w4a16_linear(x, qw, qz, sc, 128, "gptq", "f16", gi))
    # compressed-tensors int4: transposed storage, bf16 scales, zero point as stored
    rng = np.random.default_rng(5)
    q = rng.integers(0, 16, (k, n), dtype=np.int32)
    z = rng.integers(0, 16, (k // 128, n), dtype=np.int32)
    s = fm.round_bf16(rng.uniform(1e-3, 2e-2, (k // 128, n)).astype(np.float32))
    packed, zeros = fm.pack_int4(q, "ct", along_rows=True), fm.pack_int4(z, "ct")
    write_checkpoint(tmp_path / "ct", {"m.weight_packed": torch.from_numpy(np.ascontiguousarray(packed.T)),
                                       "m.weight_zero_point": torch.from_numpy(np.ascontiguousarray(zeros.T)),
                                       "m.weight_scale": torch.from_numpy(np.ascontiguousarray(s.T)).bfloat16()},
                     {"quant_method": "compressed-tensors", "format": "pack-quantized",
                      "config_groups": {"g": {"weights": {"type": "int", "num_bits": 4, "group_size": 128, "symmetric": False}}}})
    xb = synth.activations(3, k, "bf16", seed=2)
    mods = loader.load_quantized_linears(tmp_path / "ct", "cuda")
    close(mods["m"](torch.from_numpy(xb).bfloat16().cuda()), ol.w4a16_linear(xb, packed, zeros, s, 128, "ct", "bf16"))
    # the dequantised-weight export of the third family is bit-exact too
    from emmy_b200 import ops

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    wd = ops.dequant_w4(dev(packed), dev(zeros), dev(s).bfloat16(), 128, "ct", out_dtype=torch.bfloat16)
    np.testing.assert_array_equal(wd.float().cpu().numpy(), fm.cast_weight(fm.dequant_w4(packed, zeros, s, 128, "ct"), "bf16"))


def test_fp8_and_nvfp4_from_a_mixed_checkpoint(tmp_path):
    from emmy_b200 import loader

    n, k = 256, 512
    bits, sw = synth.fp8_weight(n, k, seed=6)
    packed, sbits, s2 = synth.nvfp4_weight(n, k, seed=7)
    x = synth.activations(9, k, "bf16", seed=8)
    s2x = oact.nvfp4_global_scale(x)
    static = np.float32(np.abs(x).max() / 448.0)
    t = {
        "a.q_proj.weight": torch.from_numpy(bits).view(torch.float8_e4m3fn), "a.q_proj.weight_scale": torch.from_numpy(sw),
        "a.k_proj.weight": torch.from_numpy(bits).view(torch.float8_e4m3fn), "a.k_proj.weight_scale": torch.from_numpy(sw),
        "a.k_proj.input_scale": torch.tensor([static]),
        "b.down_proj.weight": torch.from_numpy(packed), "b.down_proj.weight_scale": torch.from_numpy(sbits).view(torch.float8_e4m3fn),
        "b.down_proj.weight_scale_2": torch.from_numpy(s2), "b.down_proj.input_scale": torch.tensor([s2x]),
    }
    qc = {"quant_method": "modelopt", "quant_algo": "MIXED_PRECISION",
          "config_groups": {"a": {"weights": {"type": "float", "num_bits": 4, "group_size": 16}}, "b": {"weights": {"type": "float", "num_bits": 8}}}}
    write_checkpoint(tmp_path, t, qc)
    mods = loader.load_quantized_linears(tmp_path, "cuda")
    xd = torch.from_numpy(x).bfloat16().cuda()
    close(mods["a.q_proj"](xd), ol.fp8_linear(x, bits, sw))
    close(mods["b.down_proj"](xd), ol.nvfp4_linear(x, packed, sbits, s2, s2x))
    # static activation scale: codes = e4m3(x / scale), the same scale for every token
    xh = fm.round_bf16(fm.e4m3_decode(fm.e4m3_encode((x / static).astype(np.float32))) * static)
    ref = xh @ fm.round_bf16(fm.dequant_fp8(bits, sw)).T
    close(mods["a.k_proj"](xd), ref)


@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (5, 384, 1536), (16, 256, 5120), (37, 384, 256), (300, 512, 1024)])
def test_block_scaled_fp8(m, n, k, tmp_path):
    from emmy_b200 import loader, ops

    rng = np.random.default_rng(m)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    # per 128 x 128 block: s = amax / 448, bits = e4m3(w / s) (emmy/compiler/loader/synthesize.py:95-103)
    blocks = w.reshape(n // 128, 128, k // 128, 128)
    s = (np.maximum(np.abs(blocks).max(axis=(1, 3)), 1e-12) / 448.0).astype(np.float32)
    bits = fm.e4m3_encode((blocks / s[:, None, :, None]).astype(np.float32).reshape(n, k))
    x = synth.activations(m, k, "bf16", seed=m + 1)
    # the per-group activation quantizer is bit-exact
    q, sx = ops.quant_fp8_per_group(torch.from_numpy(x).bfloat16().cuda())
    rq, rs = oact.fp8_dynamic_per_group(x)
    np.testing.assert_array_equal(sx.cpu().numpy(), rs)
    np.testing.assert_array_equal(q.cpu().numpy(), rq)
    write_checkpoint(tmp_path, {"m.weight": torch.from_numpy(bits).view(torch.float8_e4m3fn), "m.weight_scale_inv": torch.from_numpy(s)},
                     {"quant_method": "fp8", "activation_scheme": "dynamic", "weight_block_size": [128, 128]})
    mod = loader.load_quantized_linears(tmp_path, "cuda")["m"]
    close(mod(torch.from_numpy(x).bfloat16().cuda()), ol.fp8_block_linear(x, bits, s))


def test_experts_from_per_expert_modules_and_from_interleaved_fused_tensors(tmp_path):
    from emmy_b200 import loader

    e, h, inter, k = 4, 256, 128, 2
    gu = [synth.awq_linear(h, 2 * inter, seed=20 + i) for i in range(e)]  # logical [gate | up] columns
    dn = [synth.awq_linear(inter, h, seed=40 + i) for i in range(e)]
    ex = {"gate_up": tuple(np.stack([p[j] for p in gu]) for j in range(3)), "down": tuple(np.stack([p[j] for p in dn]) for j in range(3))}
    wgu, wdn = omoe.dequant_expert_weights(ex, torch.bfloat16)
    x = torch.from_numpy(synth.activations(6, h, "bf16", seed=9)).bfloat16()
    logits = torch.randn(6, e, generator=torch.Generator().manual_seed(2))
    ref = omoe.moe_layer(x, logits, wgu, wdn, k).float().numpy()

    def split(triple, lo, hi):  # columns [lo, hi) of an AWQ linear, in whole words
        qw, qz, sc = triple
        return torch.from_numpy(qw[:, lo // 8:hi // 8].copy()), torch.from_numpy(qz[:, lo // 8:hi // 8].copy()), torch.from_numpy(sc[:, lo:hi].copy())

    # (1) one module per expert and projection
    t = {}
    for i in range(e):
        for name, triple in (("gate_proj", split(gu[i], 0, inter)), ("up_proj", split(gu[i], inter, 2 * inter)), ("down_proj", tuple(torch.from_numpy(a) for a in dn[i]))):
            for leaf, tensor in zip(("qweight", "qzeros", "scales"), triple):
                t[f"model.layers.0.mlp.experts.{i}.{name}.{leaf}"] = tensor
    write_checkpoint(tmp_path / "split", t, {"quant_method": "awq", "bits": 4, "group_size": 128})
    index = loader.CheckpointIndex(tmp_path / "split")
    groups = loader.scan_experts(loader.scan(tmp_path / "split", index))
    moe = loader.load_experts(index, groups["model.layers.0.mlp.experts"], "cuda", top_k=k)
    close(moe(x.cuda(), logits.cuda()), ref)

    # (2) fused gate_up_proj with gate / up on even / odd columns: de-interleaved at load
    def interleave(triple):
        q = fm.unpack_int4(triple[0], "awq")
        z = fm.unpack_int4(triple[1], "awq")
        s = triple[2]
        mix = lambda a: np.stack([a[:, :inter], a[:, inter:]], axis=-1).reshape(a.shape[0], 2 * inter)
        return torch.from_numpy(fm.pack_int4(mix(q), "awq")), torch.from_numpy(fm.pack_int4(mix(z), "awq")), torch.from_numpy(mix(s))

    t = {}
    for i in range(e):
        for name, triple in (("gate_up_proj", interleave(gu[i])), ("down_proj", tuple(torch.from_numpy(a) for a in dn[i]))):
            for leaf, tensor in zip(("qweight", "qzeros", "scales"), triple):
                t[f"model.layers.0.mlp.experts.{i}.{name}.{leaf}"] = tensor
    write_checkpoint(tmp_path / "fused", t, {"quant_method": "awq", "bits": 4, "group_size": 128})
    index = loader.CheckpointIndex(tmp_path / "fused")
    groups = loader.scan_experts(loader.scan(tmp_path / "fused", index))
    moe = loader.load_experts(index, groups["model.layers.0.mlp.experts"], "cuda", top_k=k, interleaved_gate_up=True)
    close(moe(x.cuda(), logits.cuda()), ref)
