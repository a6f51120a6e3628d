"""Router, expert FFN and routed combine of one MoE layer on CPU torch (test infrastructure).

The reference's modules cannot be imported without its native extensions, so
these restate them from the cited lines.
"""

from __future__ import annotations

import numpy as np
import torch

from . import formats as fm


def route_softmax_topk(logits: torch.Tensor, k: int, renorm: bool = True):
    """logits [T, E] (any float dtype) -> (scores f32 [T,k], ids int64 [T,k]).

    Softmax in f32, top-k with ties going to the lowest expert id, picked
    probabilities renormalised to sum to one
    (emmy/serving/native/prepare.py:424-463; contract of the fused router in
    emmy/serving/gen_runner.py:3175-3197).  Slots are ordered by rank
    (largest first)."""
    lg = logits.float()
    probs = torch.softmax(lg, dim=-1)
    # stable descending sort keeps the lowest id first among equal logits
    order = torch.sort(lg, dim=-1, descending=True, stable=True).indices[:, :k]
    picked = probs.gather(1, order)
    if renorm:
        picked = picked / picked.sum(dim=1, keepdim=True)
    return picked, order


def expert_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """One expert on its rows: gate, up = linear(x, w_gate_up).chunk(2);
    linear(silu(gate) * up, w_down), all in the activation dtype with the
    library's f32 accumulation (emmy/compiler/trace/huggingface.py:1663-1669).
    w_gate_up is [2I, H] (gate rows then up rows), w_down [H, I]."""
    gate, up = torch.nn.functional.linear(x, w_gate_up).chunk(2, dim=-1)
    return torch.nn.functional.linear(torch.nn.functional.silu(gate) * up, w_down)


def combine_routed(x: torch.Tensor, scores: torch.Tensor, ids: torch.Tensor, run_expert) -> torch.Tensor:
    """out[t] = dtype( sum_j f32(score[t,j]) * f32(expert_{id[t,j]}(x[t])) ),
    the picks of each row added in ascending expert order, products and sum in
    f32, one final rounding (emmy/serving/gen_runner.py:235-287).  Scores are
    first cast to the activation dtype as the reference does (:263).
    `run_expert(e, rows)` returns expert e's output for x[rows]."""
    t, k = ids.shape
    sc = scores.to(x.dtype)
    ids_sorted, by_expert = ids.sort(dim=1, stable=True)
    sc = sc.gather(1, by_expert).float()
    acc = torch.zeros(t, x.shape[1], dtype=torch.float32)
    # slot-major accumulation keeps every row's additions in ascending expert order
    outs = {}
    for e in torch.unique(ids_sorted).tolist():
        rows = (ids_sorted == e).any(dim=1).nonzero().squeeze(1)
        outs[e] = (rows, run_expert(e, rows).float())
    pos = {e: {int(r): i for i, r in enumerate(rows.tolist())} for e, (rows, _) in outs.items()}
    for j in range(k):
        for r in range(t):
            e = int(ids_sorted[r, j])
            acc[r] += sc[r, j] * outs[e][1][pos[e][r]]
    return acc.to(x.dtype)


def dequant_expert_weights(experts: dict, dtype: torch.dtype):
    """AWQ expert stacks -> dense HF-orientation weights in `dtype`.

    experts: {"gate_up": (qweight [E,H,2I/8], qzeros [E,H/G,2I/8], scales
    [E,H/G,2I]), "down": (...)} as numpy arrays; group size from the shapes'
    ratio.  Returns (w_gate_up [E,2I,H], w_down [E,H,I])."""
    name = "bf16" if dtype == torch.bfloat16 else "f16"
    out = []
    for key in ("gate_up", "down"):
        qw, qz, sc = experts[key]
        mats = []
        for e in range(qw.shape[0]):
            g = qw.shape[1] // qz.shape[1]
            w = fm.cast_weight(fm.dequant_w4(qw[e], qz[e], sc[e], g, "awq"), name)
            mats.append(torch.from_numpy(np.ascontiguousarray(w.T)).to(dtype))
        out.append(torch.stack(mats))
    return out[0], out[1]


def moe_layer(x: torch.Tensor, logits: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, k: int):
    """Whole routed layer on dense expert weights."""
    scores, ids = route_softmax_topk(logits, k)
    return combine_routed(x, scores, ids, lambda e, rows: expert_ffn(x[rows], w_gate_up[e], w_down[e]))


def tp_expert_slice(name: str, tensor: torch.Tensor, rank: int, world: int, stacked: bool = False) -> torch.Tensor:
    """The reference's own sharding of ONE expert tensor, used here as a cross-check of expert parallelism: every rank
    keeps 1/world of the intermediate axis of every expert (emmy/compiler/trace/huggingface.py:1071-1089).  The
    intermediate axis is the rows of w_gate / w_up / w_gate_up and the columns of w_down (one further in for
    expert-stacked tensors); w_gate_up holds gate rows then up rows and keeps the same row range of both; a tensor
    whose intermediate extent is 1 (a broadcast scale) is returned as it is."""
    dim = int(stacked) + (1 if name.startswith("w_down") else 0)
    blocks = 2 if name.startswith("w_gate_up") else 1
    per_block = tensor.shape[dim] // blocks
    if per_block == 1:
        return tensor
    if per_block % world:
        raise ValueError(f"{name}: {per_block} intermediate entries do not split over {world} ranks")
    share = per_block // world
    index = torch.cat([torch.arange(b * per_block + rank * share, b * per_block + (rank + 1) * share) for b in range(blocks)])
    return tensor.index_select(dim, index)
