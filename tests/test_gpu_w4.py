"""W4 (AWQ / GPTQ) on the GPU against the CPU oracle, through the C ABI."""

import numpy as np
import pytest
import torch

from oracle import formats as fm
from oracle import linear as ol
from oracle import synth

pytestmark = pytest.mark.gpu

TOL = 2e-2  # max|err| <= TOL * max|ref|, f32 accumulation on both sides


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def act(x, dtype):
    t = torch.from_numpy(x).cuda()
    return t.half() if dtype == "f16" else t.bfloat16()


def check_close(y, ref):
    got = y.float().cpu().numpy()
    err = np.abs(got - ref).max()
    bound = TOL * np.abs(ref).max()
    assert np.isfinite(got).all()
    assert err <= bound, f"max err {err} > {bound}"
    return err / np.abs(ref).max()


@pytest.mark.parametrize("fmt,along", [("awq", False), ("gptq", True), ("gptq", False)])
def test_unpack_bit_exact(fmt, along):
    from emmy_b200 import ops

    words = np.random.default_rng(5).integers(-(2**31), 2**31, (40, 24), dtype=np.int64).astype(np.int32)
    got = ops.unpack_int4(dev(words), fmt, along_rows=along).cpu().numpy()
    np.testing.assert_array_equal(got, fm.unpack_int4(words, fmt, along_rows=along).astype(np.uint8))


def test_unpack_golden(golden):
    from emmy_b200 import ops

    for name in ("awq", "gptq"):
        rows = name == "gptq"
        got = ops.unpack_int4(dev(golden[f"{name}_qweight"]), name, along_rows=rows).cpu().numpy()
        np.testing.assert_array_equal(got, golden[f"{name}_unpacked"].astype(np.uint8))


@pytest.mark.parametrize("name", ["awq", "gptq", "awq_g32", "gptq_g32"])
@pytest.mark.parametrize("transpose", [False, True])
def test_dequant_golden_bit_exact(golden, name, transpose):
    from emmy_b200 import ops

    fmt = name.split("_")[0]
    out = ops.dequant_w4(
        dev(golden[f"{name}_qweight"]), dev(golden[f"{name}_qzeros"]), dev(golden[f"{name}_scales"]),
        int(golden[f"{name}_group"]), fmt, out_dtype=torch.float32, transpose=transpose,
    ).cpu().numpy()
    ref = golden[f"{name}_dequant"]
    np.testing.assert_array_equal(out, ref.T if transpose else ref)


@pytest.mark.parametrize("fmt", ["awq", "gptq"])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_dequant_rounds_once_bit_exact(fmt, dtype):
    """The dequantised weight in the model dtype equals the oracle's single rounding of the exact f32 product."""
    from emmy_b200 import ops

    k, n = 512, 384
    if fmt == "awq":
        qw, qz, sc = synth.awq_linear(k, n, seed=3)
        gi = None
    else:
        qw, qz, sc, gi = synth.gptq_linear(k, n, seed=3)
    tdt = torch.float16 if dtype == "f16" else torch.bfloat16
    out = ops.dequant_w4(dev(qw), dev(qz), dev(sc), 128, fmt, g_idx=None if gi is None else dev(gi), out_dtype=tdt, transpose=True)
    ref = fm.cast_weight(fm.dequant_w4(qw, qz, sc, 128, fmt, gi), dtype).T
    np.testing.assert_array_equal(out.float().cpu().numpy(), ref)


def test_dequant_scattered_g_idx_bit_exact():
    from emmy_b200 import ops

    k, n, g = 256, 64, 64
    qw, qz, sc, _ = synth.gptq_linear(k, n, group=g, seed=9)
    gi = np.random.default_rng(1).permutation(np.arange(k) // g).astype(np.int32)
    out = ops.dequant_w4(dev(qw), dev(qz), dev(sc), g, "gptq", g_idx=dev(gi), out_dtype=torch.float32).cpu().numpy()
    np.testing.assert_array_equal(out, fm.dequant_w4(qw, qz, sc, g, "gptq", gi))


def test_dequant_single_group():
    from emmy_b200 import ops

    qw, qz, sc = synth.awq_linear(128, 32, group=128, seed=2)
    out = ops.dequant_w4(dev(qw), dev(qz), dev(sc), -1, "awq", out_dtype=torch.float32).cpu().numpy()
    np.testing.assert_array_equal(out, fm.dequant_w4(qw, qz, sc, -1, "awq"))


@pytest.mark.parametrize("fmt", ["awq", "gptq"])
def test_repack_round_trip_bit_exact(fmt):
    """unpack(repack(w)) == unpack(w): the load-time re-tiling loses nothing."""
    from emmy_b200 import ops

    k, n = 512, 96
    if fmt == "awq":
        qw, qz, sc = synth.awq_linear(k, n, seed=4)
        w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, fmt)
    else:
        qw, qz, sc, gi = synth.gptq_linear(k, n, seed=4)
        w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, fmt, g_idx=dev(gi))
        assert w.perm is None  # block-constant g_idx needs no row permutation
    got = ops.w4_unpack_repacked(w).cpu().numpy()
    np.testing.assert_array_equal(got, fm.unpack_int4(qw, fmt, along_rows=(fmt == "gptq")).astype(np.uint8))


def test_repack_scattered_g_idx_sorts_rows():
    from emmy_b200 import ops

    k, n, g = 512, 32, 128
    qw, qz, sc, _ = synth.gptq_linear(k, n, group=g, seed=6)
    gi = np.random.default_rng(2).permutation(np.arange(k) // g).astype(np.int32)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), g, "gptq", g_idx=dev(gi))
    assert w.perm is not None
    perm = w.perm.cpu().numpy()[:k]
    np.testing.assert_array_equal(perm, np.argsort(gi, kind="stable"))
    got = ops.w4_unpack_repacked(w).cpu().numpy()
    np.testing.assert_array_equal(got, fm.unpack_int4(qw, "gptq", along_rows=True).astype(np.uint8)[perm])


def test_repack_rejects_unbalanced_groups():
    from emmy_b200 import ops
    from emmy_b200.lib import EmmyqError

    k, n, g = 256, 32, 128
    qw, qz, sc, _ = synth.gptq_linear(k, n, group=g, seed=6)
    gi = np.zeros(k, dtype=np.int32)
    gi[::3] = 1
    with pytest.raises(EmmyqError) as e:
        ops.w4_repack(dev(qw), dev(qz), dev(sc), g, "gptq", g_idx=dev(gi))
    assert e.value.status_name == "EQ_ERR_UNSUPPORTED"
    gi[0] = 99
    with pytest.raises(EmmyqError) as e:
        ops.w4_repack(dev(qw), dev(qz), dev(sc), g, "gptq", g_idx=dev(gi))
    assert e.value.status_name == "EQ_ERR_BAD_ARG"


@pytest.mark.parametrize("m", [1, 16])
def test_awq_linear_config1(m):
    """AWQ K=N=4096, group 128, fp16, M in {1, 16}."""
    from emmy_b200 import ops

    k = n = 4096
    qw, qz, sc = synth.awq_linear(k, n, seed=0)
    x = synth.activations(m, k, "f16", seed=1)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "awq")
    y = ops.w4a16_linear(act(x, "f16"), w)
    check_close(y, ol.w4a16_linear(x, qw, qz, sc, 128, "awq", "f16"))


@pytest.mark.parametrize("shape", [(4096, 14336), (14336, 4096)])
@pytest.mark.parametrize("m", [1, 4, 16, 20, 32])
def test_gptq_act_order_llama_mlp(shape, m):
    """GPTQ act-order, Llama-3.1-8B MLP shapes, decode-shaped M (17 to 24 rows: x staged in K slices; 32: the tensor path)."""
    from emmy_b200 import ops

    k, n = shape
    qw, qz, sc, gi = synth.gptq_linear(k, n, seed=0)
    x = synth.activations(m, k, "f16", seed=m)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "gptq", g_idx=dev(gi))
    y = ops.w4a16_linear(act(x, "f16"), w)
    check_close(y, ol.w4a16_linear(x, qw, qz, sc, 128, "gptq", "f16", gi))


@pytest.mark.parametrize("m", [64, 256])
def test_gptq_act_order_prefill_rows(m):
    from emmy_b200 import ops

    k, n = 4096, 2048
    qw, qz, sc, gi = synth.gptq_linear(k, n, seed=2)
    x = synth.activations(m, k, "f16", seed=3)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "gptq", g_idx=dev(gi))
    y = ops.w4a16_linear(act(x, "f16"), w)
    check_close(y, ol.w4a16_linear(x, qw, qz, sc, 128, "gptq", "f16", gi))


@pytest.mark.parametrize("m", [1, 2, 3, 7, 8, 9, 15, 17, 31, 33, 64, 65, 130])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_ragged_row_counts(m, dtype):
    from emmy_b200 import ops

    k, n = 768, 272  # 12 chunks, 17 column tiles: spans straddle tiles
    qw, qz, sc = synth.awq_linear(k, n, seed=m)
    x = synth.activations(m, k, dtype, seed=m + 1)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "awq")
    y = ops.w4a16_linear(act(x, dtype), w)
    check_close(y, ol.w4a16_linear(x, qw, qz, sc, 128, "awq", dtype))


def test_smallest_shape_and_empty_batch():
    from emmy_b200 import ops

    qw, qz, sc = synth.awq_linear(128, 16, group=128, seed=1)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "awq")
    x = synth.activations(2, 128, "f16")
    check_close(ops.w4a16_linear(act(x, "f16"), w), ol.w4a16_linear(x, qw, qz, sc, 128, "awq", "f16"))
    y = ops.w4a16_linear(torch.empty(0, 128, dtype=torch.float16, device="cuda"), w)
    assert y.shape == (0, 16)


def test_single_group_and_wide_groups():
    from emmy_b200 import ops

    for group in (-1, 256):
        qw, qz, sc = synth.awq_linear(512, 64, group=512 if group == -1 else group, seed=7)
        w = ops.w4_repack(dev(qw), dev(qz), dev(sc), group, "awq")
        x = synth.activations(3, 512, "f16")
        check_close(ops.w4a16_linear(act(x, "f16"), w), ol.w4a16_linear(x, qw, qz, sc, group, "awq", "f16"))


def test_group_64_is_refused_with_a_status():
    from emmy_b200 import ops
    from emmy_b200.lib import EmmyqError

    qw, qz, sc = synth.awq_linear(128, 16, group=64, seed=1)
    with pytest.raises(EmmyqError) as e:
        ops.w4_repack(dev(qw), dev(qz), dev(sc), 64, "awq")
    assert e.value.status_name == "EQ_ERR_UNSUPPORTED"


def test_scattered_act_order_linear():
    """A g_idx whose groups are scattered over K: rows are sorted at load time and x gathered at run time."""
    from emmy_b200 import ops

    k, n, g = 1024, 256, 128
    qw, qz, sc, _ = synth.gptq_linear(k, n, group=g, seed=8)
    gi = np.random.default_rng(3).permutation(np.arange(k) // g).astype(np.int32)
    for m in (1, 5):
        x = synth.activations(m, k, "f16", seed=m)
        w = ops.w4_repack(dev(qw), dev(qz), dev(sc), g, "gptq", g_idx=dev(gi))
        y = ops.w4a16_linear(act(x, "f16"), w)
        check_close(y, ol.w4a16_linear(x, qw, qz, sc, g, "gptq", "f16", gi))


def test_workspace_is_left_zero_and_calls_repeat():
    from emmy_b200 import ops

    k, n = 2048, 1024
    qw, qz, sc = synth.awq_linear(k, n, seed=0)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "awq")
    x = act(synth.activations(4, k, "f16"), "f16")
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    y1 = ops.w4a16_linear(x, w, workspace=ws)
    torch.cuda.synchronize()
    assert int(ws.count_nonzero()) == 0
    ops.w4a16_status(ws, 4, n)
    y2 = ops.w4a16_linear(x, w, workspace=ws)
    assert float((y1.float() - y2.float()).abs().max()) <= 1e-2 * float(y1.float().abs().max())
    assert int(ws.count_nonzero()) == 0


def test_linearity_at_full_size():
    """A size-independent property at the full down-projection size: W(a x1 + x2) == a W x1 + W x2 up to rounding."""
    from emmy_b200 import ops

    k, n = 14336, 4096
    qw, qz, sc, gi = synth.gptq_linear(k, n, seed=11)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "gptq", g_idx=dev(gi))
    x1 = act(synth.activations(1, k, "f16", seed=1), "f16")
    x2 = act(synth.activations(1, k, "f16", seed=2), "f16")
    y1, y2 = ops.w4a16_linear(x1, w).float(), ops.w4a16_linear(x2, w).float()
    y12 = ops.w4a16_linear((x1.float() * 0.5 + x2.float()).half(), w).float()
    ref = 0.5 * y1 + y2
    assert float((y12 - ref).abs().max()) <= TOL * float(ref.abs().max())


# ---------------------------------------------------------------------------------------------- tensor path (M > 16)
@pytest.mark.parametrize("m,n,k", [(200, 272, 768), (300, 1040, 256), (2560, 4096, 256), (2700, 4112, 128)])
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_prefill_tiles_and_tails(m, n, k, dtype):
    """Row counts and widths that leave ragged tiles in each of the tensor-path tilings."""
    from emmy_b200 import ops

    qw, qz, sc = synth.awq_linear(k, n, seed=m)
    x = synth.activations(m, k, dtype, seed=n)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "awq")
    ws = ops.w4a16_workspace(m, n, torch.device("cuda"), k)
    y = ops.w4a16_linear(act(x, dtype), w, workspace=ws)
    ops.w4a16_status(ws, m, n)
    check_close(y, ol.w4a16_linear(x, qw, qz, sc, 128, "awq", dtype))


def test_prefill_scattered_act_order():
    from emmy_b200 import ops

    k, n, g = 1024, 256, 128
    qw, qz, sc, _ = synth.gptq_linear(k, n, group=g, seed=8)
    gi = np.random.default_rng(3).permutation(np.arange(k) // g).astype(np.int32)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), g, "gptq", g_idx=dev(gi))
    for m in (40, 333):
        x = synth.activations(m, k, "bf16", seed=m)
        y = ops.w4a16_linear(act(x, "bf16"), w)
        check_close(y, ol.w4a16_linear(x, qw, qz, sc, g, "gptq", "bf16", gi))


@pytest.mark.parametrize("m", [64, 256, 4096])
def test_prefill_matches_dequantised_matmul_at_full_size(m):
    """Llama-3.1-8B gate/up shape: the tensor path against an f32 matmul on the bit-exact dequantised weight."""
    from emmy_b200 import ops

    k, n = 4096, 14336
    qw, qz, sc, gi = synth.gptq_linear(k, n, seed=0)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "gptq", g_idx=dev(gi))
    wd = ops.dequant_w4(dev(qw), dev(qz), dev(sc), 128, "gptq", out_dtype=torch.float16, g_idx=dev(gi))  # [K, N]
    x = act(synth.activations(m, k, "f16", seed=m), "f16")
    y = ops.w4a16_linear(x, w)
    ref = x.float() @ wd.float()
    err = float((y.float() - ref).abs().max())
    assert err <= 4e-3 * float(ref.abs().max())


@pytest.mark.parametrize("group", [-1, 256])
def test_prefill_wide_groups(group):
    """Groups wider than one 128-row item (their scale record repeats per item) on the tensor path."""
    from emmy_b200 import ops

    k, n = 512, 208
    qw, qz, sc = synth.awq_linear(k, n, group=k if group == -1 else group, seed=21)
    w = ops.w4_repack(dev(qw), dev(qz), dev(sc), group, "awq")
    for m in (40, 150):
        x = synth.activations(m, k, "f16", seed=m)
        check_close(ops.w4a16_linear(act(x, "f16"), w), ol.w4a16_linear(x, qw, qz, sc, group, "awq", "f16"))


def test_prefill_bf16_scales_with_f16_activations():
    """Scales stored in the other 16-bit type are converted once per item on the tensor path."""
    from emmy_b200 import ops

    k, n = 384, 160
    qw, qz, sc = synth.awq_linear(k, n, seed=5, scale_dtype=np.float32)  # bf16-rounded values held as f32
    sc_dev = torch.from_numpy(sc).cuda().bfloat16()
    w = ops.w4_repack(dev(qw), dev(qz), sc_dev, 128, "awq")
    for m in (3, 64):
        x = synth.activations(m, k, "f16", seed=m)
        check_close(ops.w4a16_linear(act(x, "f16"), w), ol.w4a16_linear(x, qw, qz, sc, 128, "awq", "f16"))


def test_concatenated_linears_share_one_launch():
    """[gate | up] as one linear: the outputs of the parts side by side, bit for bit (same kernel, same tiles)."""
    from emmy_b200 import ops

    k = 1024
    parts, refs = [], []
    x = synth.activations(1, k, "f16", seed=3)
    for i, n in enumerate((2400, 2384)):
        qw, qz, sc, gi = synth.gptq_linear(k, n, seed=30 + i)
        w = ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "gptq", g_idx=dev(gi))
        parts.append(w)
        refs.append(ol.w4a16_linear(x, qw, qz, sc, 128, "gptq", "f16", gi))
    both = ops.w4_concat(parts)
    assert both.n == 4784
    y = ops.w4a16_linear(act(x, "f16"), both)
    check_close(y, np.concatenate(refs, axis=1))
    for m in (5, 40):
        xm = synth.activations(m, k, "f16", seed=m)
        ym = ops.w4a16_linear(act(xm, "f16"), both)
        sep = torch.cat([ops.w4a16_linear(act(xm, "f16"), w) for w in parts], dim=1)
        assert float((ym.float() - sep.float()).abs().max()) <= 2e-3 * float(sep.float().abs().max())


def test_workspace_is_left_zero_by_every_path():
    """One workspace serves calls of different shapes in turn (prefill with scattered act-order groups, which keeps a
    gathered copy of x in it, then mid-M split-K, then the one-row GEMV, whose hand-over words must start out zero):
    every call leaves everything behind the header zero and every result matches the oracle."""
    from emmy_b200 import ops

    k, g = 1024, 128
    cases = []
    for n, seed in ((256, 8), (2048, 9)):
        qw, qz, sc, _ = synth.gptq_linear(k, n, group=g, seed=seed)
        gi = np.random.default_rng(seed).permutation(np.arange(k) // g).astype(np.int32)
        cases.append((n, qw, qz, sc, gi, ops.w4_repack(dev(qw), dev(qz), dev(sc), g, "gptq", g_idx=dev(gi))))
    lib = ops.L.load()
    size = max(lib.eq_w4a16_workspace_bytes(m, n, k) for m in (1, 8, 40, 333) for n in (256, 2048))
    ws = torch.zeros(size + 256, dtype=torch.uint8, device="cuda")
    for m in (333, 40, 1, 8, 333, 1):
        for n, qw, qz, sc, gi, w in cases:
            x = synth.activations(m, k, "f16", seed=m + n)
            y = ops.w4a16_linear(act(x, "f16"), w, workspace=ws)
            ops.w4a16_status(ws, m, n)
            assert int(ws[256:].count_nonzero()) == 0, f"M={m} N={n} left the workspace dirty"
            check_close(y, ol.w4a16_linear(x, qw, qz, sc, g, "gptq", "f16", gi))


@pytest.mark.parametrize("m", [1, 9, 40, 300, 513])
def test_gate_up_swiglu_in_one_call(m):
    """[gate | up] + SwiGLU: the elementwise form below 17 rows, the GEMM-epilogue form above (ragged last row block),
    against the oracle's eager roundings; twice on one workspace, which stays zero behind its header."""
    from emmy_b200 import ops

    k, inter = 1024, 1184  # 2 I = 2368: the last 128 + 128 column tile is partial
    parts = []
    raw = []
    for i in range(2):
        qw, qz, sc, gi = synth.gptq_linear(k, inter, seed=40 + i)
        raw.append((qw, qz, sc, gi))
        parts.append(ops.w4_repack(dev(qw), dev(qz), dev(sc), 128, "gptq", g_idx=dev(gi)))
    w = ops.w4_concat(parts)
    x = synth.activations(m, k, "bf16", seed=m)
    # the oracle on the concatenated checkpoint tensors (block-constant g_idx: each half gathers its own scale rows)
    gate = ol.w4a16_linear(x, *raw[0][:3], 128, "gptq", "bf16", raw[0][3])
    up = ol.w4a16_linear(x, *raw[1][:3], 128, "gptq", "bf16", raw[1][3])
    g, u = fm.round_bf16(gate), fm.round_bf16(up)
    ref = fm.round_bf16(fm.round_bf16(g / (np.float32(1) + np.exp(-g, dtype=np.float32))) * u)
    lib = ops.L.load()
    ws = torch.zeros(lib.eq_w4a16_gate_up_workspace_bytes(m, inter, k) + 256, dtype=torch.uint8, device="cuda")
    for _ in range(2):
        h = ops.w4a16_gate_up_swiglu(act(x, "bf16"), w, workspace=ws)
        ops.w4a16_status(ws, m, 2 * inter)
    check_close(h, ref)
    front = lib.eq_w4a16_workspace_bytes(m, 2 * inter, k)
    assert int(ws[256:front].count_nonzero()) == 0
    # an output that starts two bytes off a 16-byte boundary takes the elementwise form with scalar stores
    # (up to 16 rows; above, the epilogue form needs the alignment and the call says so)
    odd = torch.empty(m * inter + 1, dtype=torch.bfloat16, device="cuda")[1:].view(m, inter)
    assert odd.data_ptr() % 16 == 2
    if m <= 16:  # (not bit-equal to h: the warps of a CTA add their sums in arrival order)
        check_close(ops.w4a16_gate_up_swiglu(act(x, "bf16"), w, workspace=ws, out=odd), ref)
    else:
        with pytest.raises(ops.L.EmmyqError):
            ops.w4a16_gate_up_swiglu(act(x, "bf16"), w, workspace=ws, out=odd)
