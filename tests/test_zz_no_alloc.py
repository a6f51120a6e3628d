"""The allocation-free W4A16 entry point against the ordinary one.

For hosts that cannot give the library scratch memory (an engine that has handed all device memory to its own pool,
a decode loop where an allocation would stall the device), eq_w4a16_linear_noalloc keeps its scratch in an array
built into the library.  It must give what eq_w4a16_linear gives, on repeated calls (the array is shared and reused),
and must refuse sizes beyond the array.  This file sorts last on purpose: a run that stops at the first failure has
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


def test_noalloc_refuses_sizes_beyond_its_scratch():
    from emmy_b200 import ops
    from emmy_b200.lib import EmmyqError

    qw, qz, sc = synth.awq_linear(128, 32, seed=1)
    w = ops.w4_repack(_dev(qw), _dev(qz), _dev(sc), 128, "awq")
    x = torch.zeros(17, 128, dtype=torch.float16, device="cuda")
    with pytest.raises(EmmyqError) as e:
        ops.w4a16_linear_noalloc(x, w, torch.empty(17, 32, dtype=torch.float16, device="cuda"))
    assert e.value.status_name == "EQ_ERR_UNSUPPORTED" and "at most 16 rows" in str(e.value)
