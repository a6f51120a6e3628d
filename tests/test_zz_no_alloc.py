"""The allocation-free W4A16 entry point against the ordinary one.

For hosts that cannot give the library scratch memory (an engine that has handed all device memory to its own pool,
a decode loop where an allocation would stall the device), eq_w4a16_linear_noalloc keeps its scratch in an array
built into the library.  It must give what eq_w4a16_linear gives, on repeated calls (the array is shared and reused),
and must refuse sizes beyond the array.  What lives in the array: at one row, the sixteen-word hand-overs between
neighbouring CTAs of the GEMV (any weight of at least 148 column tiles); for shapes whose activations do not fit
shared memory, the partial sums and arrival counters of the split-K kernel.  Both are exercised below, twice in a
row, and both must leave the array zero.  This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""

import numpy as np
import pytest
import torch

from oracle import synth

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("m,k,n", [(1, 4096, 14336), (5, 14336, 4096), (16, 2048, 1536)])
def test_noalloc_matches_workspace_entry_point_twice(m, k, n):
    from emmy_b200 import ops

    qw, qz, sc, gi = synth.gptq_linear(k, n, seed=21)
    w = ops.w4_repack(_dev(qw), _dev(qz), _dev(sc), 128, "gptq", g_idx=_dev(gi))
    for call in range(2):  # two calls in a row: the second sees whatever the first left in the shared array
        x = _dev(synth.activations(m, k, "f16", seed=30 + call)).half()
        ref = ops.w4a16_linear(x, w).float()
        out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        ops.w4a16_linear_noalloc(x, w, out)
        got = out.float()
        assert torch.isfinite(got).all()
        # same kernel, same inputs: only the order of the f32 partial sums may differ
        assert float((got - ref).abs().max()) <= 2e-2 * float(ref.abs().max())
        assert float((got - ref).abs().max()) <= 2e-3 * float(ref.abs().max()) + 1e-3


@pytest.mark.parametrize("m,k,n", [(1, 131072, 32), (8, 53248, 64)])
def test_very_large_k_runs_through_both_entry_points(m, k, n):
    """K beyond what one CTA can stage in shared memory (one row) takes the split-K kernel, whose partial sums and
    counters live in the workspace / in the built-in array; a K of Llama-405B's down projection at a few rows takes
    the multi-row streaming kernel.  Both against the oracle, twice."""
    from emmy_b200 import lib as L
    from emmy_b200 import ops
    from oracle import linear as ol

    qw, qz, sc, gi = synth.gptq_linear(k, n, seed=5)
    w = ops.w4_repack(_dev(qw), _dev(qz), _dev(sc), 128, "gptq", g_idx=_dev(gi))
    for call in range(2):
        xs = synth.activations(m, k, "f16", seed=40 + call) * np.float32(0.125)
        x = _dev(xs).half()
        ref = ol.w4a16_linear(xs, qw, qz, sc, 128, "gptq", "f16", gi)
        ws = ops.w4a16_workspace(m, n, torch.device("cuda"), k)
        y = ops.w4a16_linear(x, w, workspace=ws).float().cpu().numpy()
        ops.w4a16_status(ws, m, n)
        out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
        ops.w4a16_linear_noalloc(x, w, out)
        L.check(L.load().eq_w4a16_noalloc_status(None))
        for got in (y, out.float().cpu().numpy()):
            assert np.isfinite(got).all()
            assert np.abs(got - ref).max() <= 2e-2 * np.abs(ref).max()
        assert int(ws.count_nonzero()) == 0  # every kernel leaves the words it used zero again


def test_noalloc_refuses_sizes_beyond_its_scratch():
    from emmy_b200 import ops
    from emmy_b200.lib import EmmyqError

    qw, qz, sc = synth.awq_linear(128, 32, seed=1)
    w = ops.w4_repack(_dev(qw), _dev(qz), _dev(sc), 128, "awq")
    x = torch.zeros(17, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(EmmyqError) as e:
        ops.w4a16_linear_noalloc(x, w, torch.empty(17, 32, dtype=torch.float16, device="cuda"))
    assert e.value.status_name == "EQ_ERR_UNSUPPORTED" and "at most 16 rows" in str(e.value)
