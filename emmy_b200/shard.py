"""Sharding of the quantized-linear path over the GPUs of one node (one process per GPU, torch.distributed).

Three partitions, as the path shards naturally:

* column-parallel linear: rank r keeps output columns [r N/W, (r+1) N/W) of every checkpoint tensor; x is replicated,
  activation quantization is the same on every rank, there is no collective (outputs stay column-sharded, or are
  all-gathered on request);
* row-parallel linear: rank r keeps input rows [r K/W, (r+1) K/W) on group boundaries, computes a full [M, N]
  partial from its slice of x, and the partials are summed in f32 over NVLink: decode-sized results by one kernel
  over peer memory (`PeerAllReduce`, eq_peer_allreduce), large ones by the process group's all-reduce;
* expert-parallel MoE: expert e lives on rank e // (E / W); picks are dispatched to their experts' ranks, run
  through the local grouped expert FFN, returned and combined at the source in ascending expert order in f32.
  Two exchanges exist: `ep_moe_forward` uses NCCL all-to-alls (and runs on gloo for the CPU tests); `EpMoe` lets the
  CUDA kernels do the exchange themselves over NVLink peer mappings (eq_ep_moe_w4a16): no host read, no NCCL call on
  the data path.

The reference shards differently -- every rank holds a 1/W slice of EVERY expert's intermediate axis and the
partials are all-reduced (emmy/compiler/trace/huggingface.py:1071-1124; emmy/serving/vllm_model_gen.py:986-991).
That slicing is restated with the test oracle, whose partial sums must equal the expert-parallel result up to f32
summation order: the tests use it as a cross-check.

The compute steps are passed in as callables, so the partition and exchange logic runs unchanged on CPU tensors
with the gloo backend (that is how it is tested without GPUs); on GPUs the callables are the C-ABI operators.
"""

from __future__ import annotations

from typing import Callable

import torch
import torch.distributed as dist

# ---------------------------------------------------------------------------------------------- slicing


def _cols(n: int, rank: int, world: int, unit: int) -> slice:
    if n % (world * unit):
        raise ValueError(f"{n} output columns do not split into {world} shards of whole {unit}-column units")
    w = n // world
    return slice(rank * w, (rank + 1) * w)


def column_slice_w4(fmt: str, qweight, qzeros, scales, g_idx, rank: int, world: int):
    """Output-column shard of an AWQ / GPTQ linear (checkpoint layouts).  16-column units keep the shard tileable."""
    n = scales.shape[1]
    c = _cols(n, rank, world, 16)
    c8 = slice(c.start // 8, c.stop // 8)
    qw = qweight[:, c8] if fmt == "awq" else qweight[:, c]
    return qw.contiguous(), qzeros[:, c8].contiguous(), scales[:, c].contiguous(), g_idx


def row_slice_w4(fmt: str, qweight, qzeros, scales, g_idx, group: int, rank: int, world: int):
    """Input-row shard of an AWQ / GPTQ linear on group boundaries.  With act-order information the shard keeps the
    scale / zero rows of the groups its rows name, renumbered from zero."""
    k = scales.shape[0] * group
    if k % (world * group):
        raise ValueError(f"{k} input rows do not split into {world} shards of whole groups of {group}")
    kw = k // world
    rows = slice(rank * kw, (rank + 1) * kw)
    qw = qweight[rows] if fmt == "awq" else qweight[rows.start // 8 : rows.stop // 8]
    if g_idx is None:
        groups = slice(rows.start // group, rows.stop // group)
        return qw.contiguous(), qzeros[groups].contiguous(), scales[groups].contiguous(), None, rows
    local = g_idx[rows]
    used, renumbered = torch.unique(local, sorted=True, return_inverse=True)
    if used.numel() * group != kw:
        raise ValueError("row shard does not hold whole act-order groups")
    return (qw.contiguous(), qzeros[used.long()].contiguous(), scales[used.long()].contiguous(), renumbered.to(g_idx.dtype), rows)


def column_slice_fp8(weight, weight_scale, rank: int, world: int):
    """Rows of the [N, K] e4m3 weight and of its per-channel scale."""
    c = _cols(weight.shape[0], rank, world, 16)
    return weight[c].contiguous(), weight_scale.reshape(-1)[c].contiguous()


def column_slice_nvfp4(weight, weight_scale, weight_scale_2, rank: int, world: int):
    """Rows of the packed [N, K/2] weight and of its [N, K/16] block scales; the global scale is shared."""
    c = _cols(weight.shape[0], rank, world, 8)
    return weight[c].contiguous(), weight_scale[c].contiguous(), weight_scale_2


def expert_owner(expert_ids: torch.Tensor, num_experts: int, world: int) -> torch.Tensor:
    """Rank that holds each expert: contiguous blocks of E / W experts."""
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not split over {world} ranks")
    return expert_ids // (num_experts // world)


# ---------------------------------------------------------------------------------------------- linears


class ColumnParallelLinear:
    """y_local[M, N/W] = linear_fn(x); `gather=True` all-gathers the column shards into [M, N]."""

    def __init__(self, linear_fn: Callable[[torch.Tensor], torch.Tensor], group=None):
        self.linear_fn, self.group = linear_fn, group

    def __call__(self, x: torch.Tensor, gather: bool = False) -> torch.Tensor:
        y = self.linear_fn(x)
        if not gather:
            return y
        world = dist.get_world_size(self.group)
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)


class RowParallelLinear:
    """y[M, N] = all_reduce_sum( linear_fn(x[:, rows]) ).  `rows` is this rank's input-feature slice.  The partials are
    summed in f32 and rounded once: by `reducer` (a `PeerAllReduce`: one kernel over NVLink peer memory) when one is given
    and the result fits it, else by the process group's all-reduce."""

    def __init__(self, linear_fn: Callable[[torch.Tensor], torch.Tensor], rows: slice, group=None, reduce_dtype=torch.float32, reducer=None):
        self.linear_fn, self.rows, self.group, self.reduce_dtype, self.reducer = linear_fn, rows, group, reduce_dtype, reducer

    def __call__(self, x: torch.Tensor, sliced: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
        """`sliced=True`: x already holds only this rank's input features (the output of a column-parallel linear)."""
        partial = self.linear_fn(x if sliced else x[:, self.rows].contiguous())
        if self.reducer is not None and self.reducer.fits(partial):
            return self.reducer(partial, out=out)
        acc = partial.to(self.reduce_dtype)
        dist.all_reduce(acc, op=dist.ReduceOp.SUM, group=self.group)
        if out is None:
            return acc.to(partial.dtype)
        out.copy_(acc)
        return out


# ---------------------------------------------------------------------------------------------- expert parallel


def ep_moe_forward(
    x: torch.Tensor,
    ids: torch.Tensor,
    scores: torch.Tensor,
    num_experts: int,
    experts_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
    combine_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
    group=None,
) -> torch.Tensor:
    """One routed MoE layer with the experts spread over the ranks of `group`.

    x [T, H]: this rank's tokens; ids int [T, k] / scores f32 [T, k]: their picks, ascending expert id per row.
    experts_fn(rows [R, H], local_expert_ids int32 [R]) -> [R, H]: the local grouped expert FFN.
    combine_fn(out_rows [T k, H], scores [T, k]) -> [T, H]: the f32 weighted sum in stored pick order.

    The counts exchange is the one host read of the layer (the reference has one too, emmy/serving/gen_runner.py:283);
    the token exchange is two all-to-alls of [picks, H] rows."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    t, k = ids.shape
    per_rank = num_experts // world
    flat = ids.reshape(-1).long()
    owner = expert_owner(flat, num_experts, world)
    order = torch.argsort(owner, stable=True)  # picks grouped by destination rank, token order kept inside
    send_counts = torch.bincount(owner, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    send_list, recv_list = send_counts.tolist(), recv_counts.tolist()

    send_rows = x[(order // k)].contiguous()
    send_eid = (flat[order] - owner[order] * per_rank).to(torch.int32).contiguous()
    recv_rows = x.new_empty((sum(recv_list), x.shape[1]))
    recv_eid = send_eid.new_empty(sum(recv_list))
    dist.all_to_all_single(recv_rows, send_rows, recv_list, send_list, group=group)
    dist.all_to_all_single(recv_eid, send_eid, recv_list, send_list, group=group)

    done = experts_fn(recv_rows, recv_eid) if recv_rows.shape[0] else recv_rows
    back = x.new_empty((t * k, x.shape[1]))
    dist.all_to_all_single(back, done.contiguous(), send_list, recv_list, group=group)

    out_rows = torch.empty_like(back)
    out_rows[order] = back  # undo the grouping by destination
    del rank
    return combine_fn(out_rows, scores)


# ---------------------------------------------------------------------------------------------- peer-memory exchange


class EpMoe:
    """Expert-parallel W4A16 MoE whose token exchange is done by the kernels over peer memory (eq_ep_moe_w4a16).

    Owns one symmetric buffer per rank (receive rows, their return addresses, the ranks' count tables, returned rows,
    epoch flags), mapped into every rank of `group` through torch symmetric memory, and a local workspace.  `t_max`
    bounds the tokens of a call on any rank.  A rank's receive buffer holds `world * cap` rows, shared by the sources and
    filled in expert order; the default cap, all of a rank's picks, can never overflow (even if every token of every rank
    picks this rank's experts).  A smaller cap saves receive memory (`default_cap` gives twice the balanced share plus
    slack) but is a bet on the routing: rows beyond the buffer are DROPPED, which only the status word reports.
    Results of a call are defined only if `status()` (or `forward(..., check=True)`) comes back clean: an overflow or a
    peer that did not arrive within the kernels' bounded wait leaves y undefined.  The call counter lives on the device,
    so `forward` has no host read and can be captured in a CUDA graph.  Construction is collective: it ends with a host
    barrier, so that no rank's first exchange waits on a peer that is still setting up."""

    @staticmethod
    def default_cap(t_max: int, topk: int, world: int) -> int:
        """The opt-in smaller receive capacity: twice the balanced share of a rank's picks plus 256 rows."""
        picks = t_max * topk
        return min(picks, 2 * picks // world + 256)


    def __init__(self, group, t_max: int, topk: int, hidden: int, inter: int, experts_local: int, dtype, device, cap: int | None = None):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings only, no NVLS binding
        import torch.distributed._symmetric_memory as symm_mem

        from . import lib as L

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > L.EQ_EP_MAX_RANKS:
            raise ValueError(f"at most {L.EQ_EP_MAX_RANKS} ranks")
        picks = t_max * topk
        if cap is None:
            cap = picks
        if not 0 < cap <= picks:
            raise ValueError(f"cap must be in 1..{picks}")
        self.cap, self.t_max, self.topk, self.hidden, self.inter, self.experts_local = cap, t_max, topk, hidden, inter, experts_local
        self.dtype, self.device = dtype, device
        esz = 2
        al = lambda v: (v + 255) // 256 * 256
        sizes = [al(self.world * cap * hidden * esz), al(self.world * cap * 8), al(self.world * self.world * experts_local * 4), al(picks * hidden * esz),
                 al(3 * self.world * 4)]
        offs = [0]
        for sz in sizes[:-1]:
            offs.append(offs[-1] + sz)
        self.buf = symm_mem.empty(offs[-1] + sizes[-1], dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        torch.cuda.synchronize(device)
        self.handle.barrier()
        peers = L.EpPeers()
        peers.world, peers.rank, peers.cap = self.world, self.rank, cap
        for r in range(self.world):
            base = int(self.handle.buffer_ptrs[r])
            peers.recv_x[r], peers.recv_meta[r], peers.recv_count[r] = base + offs[0], base + offs[1], base + offs[2]
            peers.back[r], peers.flags[r] = base + offs[3], base + offs[4]
        self.peers = peers
        self.lib = L
        need = L.load().eq_ep_moe_workspace_bytes(self.world, cap, experts_local, hidden, inter)
        self.workspace = torch.zeros(need, dtype=torch.uint8, device=device)  # holds the device-side call counter
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # every rank's buffers and flags exist before anybody's first exchange

    def forward(self, x: torch.Tensor, ids: torch.Tensor, scores: torch.Tensor, w, out: torch.Tensor | None = None,
                check: bool = False) -> torch.Tensor:
        """x [T, H] this rank's tokens; ids int32 [T, k] / scores f32 [T, k] over all experts; w: the local experts.
        check=True synchronizes the stream and raises if the call overflowed `cap` or timed out on a peer."""
        import ctypes as C

        from .ops import _DTYPE, _ptr, _stream

        t = x.shape[0]
        if t > self.t_max:
            raise ValueError(f"{t} tokens exceed the t_max={self.t_max} the buffers were sized for")
        y = out if out is not None else torch.empty((t, self.hidden), dtype=x.dtype, device=x.device)
        L = self.lib
        L.check(
            L.load().eq_ep_moe_w4a16(
                _ptr(w.gate_up), _ptr(w.down), _DTYPE[w.scale_dtype], self.experts_local, self.topk, self.hidden, self.inter, w.group,
                _ptr(x), _ptr(ids), _ptr(scores), t, _DTYPE[x.dtype], _ptr(y), C.byref(self.peers), 0, _ptr(self.workspace),
                self.workspace.numel(), _stream(),
            )
        )
        if check:
            self.status()
        return y

    def status(self) -> None:
        """Synchronizes the stream; raises if a peer wait ran out or rows overflowed the receive capacity."""
        from .ops import _ptr, _stream

        self.lib.check(self.lib.load().eq_ep_moe_status(_ptr(self.workspace), self.world, self.cap, self.experts_local, self.hidden, self.inter, _stream()))


class PeerAllReduce:
    """Sum of the ranks' f16 / bf16 partial results by one kernel over NVLink peer memory (eq_peer_allreduce): every
    rank pushes its partial into every peer's receive buffer, flags it, waits for the peers' pieces and adds the world's
    partials in rank order in f32 with one rounding, so all ranks hold bit-identical results.  One NVLink round and one
    launch instead of a library all-reduce's protocol latency; the traffic is (world - 1) x the result per rank, so it
    is meant for decode-sized results: `max_values` bounds what the symmetric buffers (two slots x world sources) can
    carry and `fits` tells a caller when to take the process group's all-reduce instead.  Collective: every rank calls
    it the same number of times with the same shape.  The call counter lives on the device, so calls replay from a
    captured CUDA graph.  Results are defined only if `status()` comes back clean (a peer that did not arrive within
    about a second sets the status word)."""

    def __init__(self, group, max_values: int, device):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings only, no NVLS binding
        import torch.distributed._symmetric_memory as symm_mem

        from . import lib as L

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self.world > L.EQ_EP_MAX_RANKS:
            raise ValueError(f"at most {L.EQ_EP_MAX_RANKS} ranks")
        self.cap = (max_values + 7) // 8 * 8
        lib = L.load()
        recv = (lib.eq_peer_allreduce_recv_bytes(self.world, self.cap) + 255) // 256 * 256
        flags = lib.eq_peer_allreduce_flag_bytes(self.world, self.cap)
        self.buf = symm_mem.empty(recv + flags, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        torch.cuda.synchronize(device)
        self.handle.barrier()
        peers = L.ArPeers()
        peers.world, peers.rank, peers.cap, peers.max_blocks = self.world, self.rank, self.cap, (self.cap + 2047) // 2048
        for r in range(self.world):
            base = int(self.handle.buffer_ptrs[r])
            peers.recv[r], peers.flags[r] = base, base + recv
        self.peers, self.lib = peers, L
        self.state = torch.zeros(lib.eq_peer_allreduce_state_bytes(), dtype=torch.uint8, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # every rank's buffers and flags exist before anybody's first push

    def fits(self, partial: torch.Tensor) -> bool:
        return partial.is_cuda and partial.dtype in (torch.float16, torch.bfloat16) and partial.numel() % 8 == 0 and partial.numel() <= self.cap

    def __call__(self, partial: torch.Tensor, out: torch.Tensor | None = None, check: bool = False) -> torch.Tensor:
        import ctypes as C

        from .ops import _DTYPE, _ptr, _stream

        partial = partial.contiguous()
        y = out if out is not None else torch.empty_like(partial)
        self.lib.check(self.lib.load().eq_peer_allreduce(C.byref(self.peers), _ptr(partial), partial.numel(), _DTYPE[partial.dtype], _ptr(y),
                                                         _ptr(self.state), _stream()))
        if check:
            self.status()
        return y

    def status(self) -> None:
        """Synchronizes the stream; raises if a peer's piece did not arrive in time."""
        from .ops import _ptr, _stream

        self.lib.check(self.lib.load().eq_peer_allreduce_status(_ptr(self.state), _stream()))


class EpMoePipelined:
    """`EpMoe` over `chunks` slices of the tokens, each slice a complete exchange of its own (own buffers, flags and
    workspace) on its own stream: while one slice's expert GEMMs run, the next slice's rows are crossing NVLink and the
    previous slice's results are on their way back, so the exchange hides behind the math instead of adding to it.
    The slices are row ranges of x, ids, scores and y; every rank must use the same `chunks`.  Streams are joined
    through events, so a call still captures into one CUDA graph.  Construction is collective."""

    def __init__(self, group, t_max: int, topk: int, hidden: int, inter: int, experts_local: int, dtype, device, chunks: int = 2,
                 cap: int | None = None):
        if chunks < 1:
            raise ValueError("chunks must be at least 1")
        self.chunks, self.t_max, self.hidden = chunks, t_max, hidden
        self.per = -(-t_max // chunks)
        self.parts = [EpMoe(group, self.per, topk, hidden, inter, experts_local, dtype, device, cap=cap) for _ in range(chunks)]
        self.streams = [None] + [torch.cuda.Stream(device=device) for _ in range(chunks - 1)]

    def forward(self, x: torch.Tensor, ids: torch.Tensor, scores: torch.Tensor, w, out: torch.Tensor | None = None,
                check: bool = False) -> torch.Tensor:
        t = x.shape[0]
        if t > self.t_max:
            raise ValueError(f"{t} tokens exceed the t_max={self.t_max} the buffers were sized for")
        y = out if out is not None else torch.empty((t, self.hidden), dtype=x.dtype, device=x.device)
        main = torch.cuda.current_stream(x.device)
        # every rank runs every slice (an empty one too): its flags are what the other ranks wait for
        bounds = [min(t, i * self.per) for i in range(self.chunks + 1)]
        for i, part in enumerate(self.parts):
            a, b = bounds[i], bounds[i + 1]
            side = self.streams[i]
            if side is None:
                part.forward(x[a:b], ids[a:b], scores[a:b], w, out=y[a:b])
            else:
                side.wait_stream(main)
                with torch.cuda.stream(side):
                    part.forward(x[a:b], ids[a:b], scores[a:b], w, out=y[a:b])
        for side in self.streams[1:]:
            main.wait_stream(side)
        if check:
            self.status()
        return y

    def status(self) -> None:
        for part in self.parts:
            part.status()

