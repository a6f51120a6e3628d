#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extra]
                    [--workload NAME [--rows ROWS]]

Headline (`gptq_llama8b_mlp_m1`): the W4A16 M=1 GEMV on GPTQ act-order weights with the Llama-3.1-8B MLP shapes
(gate/up K=4096 N=14336, down K=14336 N=4096, group 128) -- one step is one pass over a 32-layer stack of gate, up
and down projections (96 GEMVs, 2.9 GB of packed weights, far larger than L2, so every step streams its weights from
HBM).  Metric: algorithmic HBM bytes per second.

The same JSON line carries `extra`: one record per other call of the path at the benchmark shapes (AWQ and GPTQ at
their row counts, FP8 and NVFP4 linears, the MoE layer; with N > 1 also the sharded layers), each timed the same way:
one CUDA graph per step over weight copies that exceed L2, ten samples of the replay region, median / min / max, the
roofline floor that binds (the higher of bytes / HBM bandwidth and flops / tensor peak), and the end-to-end figure
with pinned host buffers.  `--workload NAME` runs one of them alone under the headline's contract (these are the
commands the profiles were made with).

Prints ONE JSON line on rank 0.  Launched by torchrun for N > 1 (one rank per GPU); every rank then owns its own
32-layer stack (weak scaling: independent layers, no data-path collective).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LAYERS = 32
SHAPES = {"gate": (4096, 14336), "up": (4096, 14336), "down": (14336, 4096)}
GROUP = 128
GEMM_K, GEMM_N = 5120, 17408
SAMPLES = 10  # repeats of the timed region behind median / min / max


def algorithmic_bytes(k: int, n: int, m: int = 1, g_idx: bool = True) -> int:
    """Bytes one W4A16 call must move, exactly as the checkpoint stores them: packed weight, packed zeros,
    16-bit scales, g_idx, x and y."""
    return k * n // 2 + (k // GROUP) * n // 2 + (k // GROUP) * n * 2 + (k * 4 if g_idx else 0) + m * k * 2 + m * n * 2


STEP_BYTES = LAYERS * sum(algorithmic_bytes(k, n) for k, n in SHAPES.values())

# dram bytes per launch of the GEMV kernel (dram__bytes_read.sum + dram__bytes_write.sum, mean of the captured launches of
# this workload) from the ncu capture summarised in profiles/w4a16_gemv1_kernel_gptq_m1.md
EP_CHUNKS = int(os.environ.get("EQ_BENCH_EP_CHUNKS", "1"))  # slices of the expert-parallel MoE record (1 = unsliced)
GEMV_KERNEL = "w4a16_gemv1_kernel<__half, true, DEPTH>"
TRAFFIC_PER_LAUNCH = 31242000


def peaks():
    """(HBM GB/s, bf16 burst TFLOP/s, bf16 sustained TFLOP/s, kind)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timed regions run; summary(t0, t1) covers a window."""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self, t0: float = 0.0, t1: float = float("inf")):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for stamp, r in self.rows:
            if not (t0 - 0.05 <= stamp <= t1 + 0.15):
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def stats(xs):
    return {"median": round(statistics.median(xs), 5), "min": round(min(xs), 5), "max": round(max(xs), 5), "samples": len(xs)}


class Timer:
    """One workload's step captured in a CUDA graph (or run eagerly) and timed with CUDA events on its stream."""

    def __init__(self, step, stream, device, world, capture=True, warmup=3):
        self.stream, self.device, self.world = stream, device, world
        with torch.cuda.stream(stream):
            for _ in range(max(warmup, 3)):
                step()
            stream.synchronize()
            self.run = step
            if capture:
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, stream=stream):
                    step()
                self.run = self.graph.replay
            for _ in range(2):
                self.run()
            stream.synchronize()

    def barrier(self):
        torch.cuda.synchronize()
        if self.world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def region(self, steps: int) -> float:
        """ms for `steps` steps, barrier + synchronize on both sides, max over ranks."""
        with torch.cuda.stream(self.stream):
            self.barrier()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(self.stream)
            for _ in range(steps):
                self.run()
            end.record(self.stream)
            end.synchronize()
            ms = start.elapsed_time(end)
            self.barrier()
        if self.world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=self.device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def e2e(self, steps: int, h2d, d2h) -> float:
        """ms per step with the step's inputs copied from pinned host memory and its result copied back, wall clock."""
        with torch.cuda.stream(self.stream):
            self.barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                for dst, src in h2d:
                    dst.copy_(src, non_blocking=True)
                self.run()
                for dst, src in d2h:
                    dst.copy_(src, non_blocking=True)
                self.stream.synchronize()
            ms = (time.perf_counter() - t0) * 1e3 / steps
            self.barrier()
        if self.world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=self.device)
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            ms = float(t.item())
        return ms


def roofline(alg_bytes, flops, peak_mult, seconds, kernel, traffic=None):
    """The floor that binds: the higher of bytes / HBM bandwidth and flops / tensor peak (the reference's rule for mid
    row counts, emmy/serving/roofline.py:137-148), against the measured time of one call."""
    hbm, burst, sustained, kind = peaks()
    t_hbm = (alg_bytes or 0) / (hbm * 1e9)
    t_tc = (flops or 0) / (sustained * peak_mult * 1e12) if peak_mult else 0.0
    if t_hbm >= t_tc:
        out = {"bound": "hbm", "achieved": round(alg_bytes / seconds / 1e9, 1), "peak": hbm, "unit": "GB/s"}
    else:
        out = {"bound": "tensor", "achieved": round(flops / seconds / 1e12, 1), "peak": round(sustained * peak_mult, 1), "unit": "TFLOP/s",
               "frac_of_burst": round(flops / seconds / 1e12 / (burst * peak_mult), 4)}
    out.update({"frac": round(max(t_hbm, t_tc) / seconds, 4), "peak_kind": kind, "traffic": traffic, "kernel": kernel,
                "floor_us": {"hbm": round(t_hbm * 1e6, 2), "tensor": round(t_tc * 1e6, 2)}})
    return out


# --------------------------------------------------------------------------------------------- synthetic weights


def gptq_weight(device, gen, k, n):
    from emmy_b200 import ops

    qweight = torch.randint(-(2**31), 2**31 - 1, (k // 8, n), dtype=torch.int32, device=device, generator=gen)
    qzeros = torch.full((k // GROUP, n // 8), 0x77777777, dtype=torch.int32, device=device)  # stored 7 = zero 8
    scales = (torch.rand((k // GROUP, n), device=device, generator=gen) * (2e-2 - 1e-3) + 1e-3).half()
    perm = torch.randperm(k // GROUP, device=device, generator=gen)
    g_idx = perm[torch.arange(k, device=device) // GROUP].int()
    return ops.w4_repack(qweight, qzeros, scales, GROUP, "gptq", g_idx=g_idx)


def awq_weight(device, gen, k, n):
    from emmy_b200 import ops

    qweight = torch.randint(-(2**31), 2**31 - 1, (k, n // 8), dtype=torch.int32, device=device, generator=gen)
    qzeros = torch.randint(-(2**31), 2**31 - 1, (k // GROUP, n // 8), dtype=torch.int32, device=device, generator=gen)
    scales = (torch.rand((k // GROUP, n), device=device, generator=gen) * (2e-2 - 1e-3) + 1e-3).half()
    return ops.w4_repack(qweight, qzeros, scales, GROUP, "awq")


def fp8_weight(device, gen, n, k):
    """W ~ N(0, 0.02) quantized per output channel (the dynamic rule applied to the weight's rows)."""
    from emmy_b200 import ops

    w = torch.randn(n, k, device=device, generator=gen) * 0.02
    bits, scale = ops.quant_fp8_per_token(w)
    return bits, scale.reshape(-1).contiguous()


def nvfp4_weight(device, gen, n, k):
    """W ~ N(0, 0.02) through the reference's weight quantizer (on the device), scales tiled for the tensor path."""
    from emmy_b200 import ops_nvfp4 as o4

    w = torch.randn(n, k, device=device, generator=gen) * 0.02
    packed, sf, s2 = o4.quant_nvfp4_weight(w)
    return packed, o4.nvfp4_tile_weight_scales(sf, k), s2


# --------------------------------------------------------------------------------------------- workloads
#
# Each returns a dict: step (callable), calls per step, algorithmic bytes and flops PER CALL, the tensor peak multiple
# of the operand type, host/device buffers of one step for the end-to-end leg, a status check, and labels.


def wl_gemv_stack(device, rank):
    from emmy_b200 import ops

    gen = torch.Generator(device=device).manual_seed(1234 + rank)
    stack = [{name: gptq_weight(device, gen, k, n) for name, (k, n) in SHAPES.items()} for _ in range(LAYERS)]
    hg = torch.Generator().manual_seed(7 + rank)
    x_host = torch.randn(1, 4096, generator=hg).half().pin_memory()
    h_host = torch.randn(1, 14336, generator=hg).half().pin_memory()
    x, h = x_host.to(device), h_host.to(device)
    ys = {name: torch.empty(1, n, dtype=torch.float16, device=device) for name, (_, n) in SHAPES.items()}
    out_host = {name: torch.empty(1, n, dtype=torch.float16).pin_memory() for name, (_, n) in SHAPES.items()}
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device=device)

    def step():
        for layer in stack:
            ops.w4a16_linear(x, layer["gate"], workspace=ws, out=ys["gate"])
            ops.w4a16_linear(x, layer["up"], workspace=ws, out=ys["up"])
            ops.w4a16_linear(h, layer["down"], workspace=ws, out=ys["down"])

    def hot_step():  # one layer's three weights over and over: 92 MB, resident in L2
        for _ in range(LAYERS):
            ops.w4a16_linear(x, stack[0]["gate"], workspace=ws, out=ys["gate"])
            ops.w4a16_linear(x, stack[0]["up"], workspace=ws, out=ys["up"])
            ops.w4a16_linear(h, stack[0]["down"], workspace=ws, out=ys["down"])

    return dict(step=step, hot_step=hot_step, calls=3 * LAYERS, kernels_per_call=1, alg_bytes=STEP_BYTES / (3 * LAYERS), flops=0.0, peak_mult=0.0,
                h2d=[(x, x_host), (h, h_host)], d2h=[(out_host[n_], ys[n_]) for n_ in ys], status=lambda: ops.w4a16_status(ws, 1, 4096),
                kernel=GEMV_KERNEL, traffic=TRAFFIC_PER_LAUNCH)


def wl_w4(device, rank, fmt, k, n, m):
    from emmy_b200 import ops

    gen = torch.Generator(device=device).manual_seed(300 + rank)
    copies = max(3, int(2.2 * 126e6 // (k * n // 2)) + 1)
    ws = [(gptq_weight if fmt == "gptq" else awq_weight)(device, gen, k, n) for _ in range(copies)]
    x_host = torch.randn(m, k, generator=torch.Generator().manual_seed(rank)).half().pin_memory()
    y_host = torch.empty(m, n, dtype=torch.float16).pin_memory()
    x = x_host.to(device)
    y = torch.empty(m, n, dtype=torch.float16, device=device)
    wsp = torch.zeros(ops.L.load().eq_w4a16_workspace_bytes(m, n, k) + 256, dtype=torch.uint8, device=device)

    def step():
        for w in ws:
            ops.w4a16_linear(x, w, workspace=wsp, out=y)

    kernel = GEMV_KERNEL if m == 1 else ("w4a16_stream_kernel" if m <= 24 else "w4a16_gemm_tc_kernel<__half>")
    return dict(step=step, calls=copies, kernels_per_call=1, alg_bytes=algorithmic_bytes(k, n, m, fmt == "gptq"), flops=2.0 * m * k * n, peak_mult=1.0,
                h2d=[(x, x_host)], d2h=[(y_host, y)], status=lambda: ops.w4a16_status(wsp, m, n), kernel=kernel,
                dtype="int4 weights, f16 activations, f32 accumulate")


def wl_gate_up_fused(device, rank):
    """gate and up of the Llama MLP as ONE linear ([gate | up] concatenated along N, as the reference stores expert
    weights): one launch streams both projections behind one prologue."""
    from emmy_b200 import ops

    gen = torch.Generator(device=device).manual_seed(350 + rank)
    k, n = SHAPES["gate"]
    copies = 5
    ws = [ops.w4_concat([gptq_weight(device, gen, k, n), gptq_weight(device, gen, k, n)]) for _ in range(copies)]
    x_host = torch.randn(1, k, generator=torch.Generator().manual_seed(rank)).half().pin_memory()
    y_host = torch.empty(1, 2 * n, dtype=torch.float16).pin_memory()
    x = x_host.to(device)
    y = torch.empty(1, 2 * n, dtype=torch.float16, device=device)
    wsp = torch.zeros(ops.L.load().eq_w4a16_workspace_bytes(1, 2 * n, k) + 256, dtype=torch.uint8, device=device)

    def step():
        for w in ws:
            ops.w4a16_linear(x, w, workspace=wsp, out=y)

    return dict(step=step, calls=copies, kernels_per_call=1, alg_bytes=2 * algorithmic_bytes(k, n) - 2 * k, flops=4.0 * k * n, peak_mult=1.0,
                h2d=[(x, x_host)], d2h=[(y_host, y)], status=lambda: ops.w4a16_status(wsp, 1, 2 * n), kernel=GEMV_KERNEL,
                dtype="int4 weights, f16 activations, f32 accumulate")


def wl_fp8_block(device, rank, m, n=GEMM_N, k=GEMM_K):
    """The official block-scaled FP8 form: 128 x 128 weight blocks, activations per token and per 128 elements of K."""
    from emmy_b200 import ops

    gen = torch.Generator(device=device).manual_seed(150 + rank)
    copies = 2
    ws = []
    for _ in range(copies):
        w = torch.randn(n, k, device=device, generator=gen) * 0.02
        blocks = w.reshape(n // 128, 128, k // 128, 128)
        s = (blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12) / 448.0).float()
        bits = (blocks / s[:, None, :, None]).reshape(n, k).to(torch.float8_e4m3fn).view(torch.uint8)
        ws.append((bits.contiguous(), s.contiguous()))
    x_host = torch.randn(m, k, generator=torch.Generator().manual_seed(rank)).bfloat16().pin_memory()
    y_host = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
    x = x_host.to(device)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=device)
    wsp = torch.empty(ops.L.load().eq_fp8_block_workspace_bytes(m, k) + 256, dtype=torch.uint8, device=device)

    def step():
        for w, s in ws:
            ops.fp8_block_linear(x, w, s, workspace=wsp, out=y)

    return dict(step=step, calls=copies, kernels_per_call=2, alg_bytes=n * k + (n // 128) * (k // 128) * 4 + m * k * 2 + m * n * 2, flops=2.0 * m * k * n,
                peak_mult=2.0, h2d=[(x, x_host)], d2h=[(y_host, y)], status=lambda: ops.fp8_block_status(wsp, m, k),
                kernel="fp8_block_decode_tc_kernel<__nv_bfloat16>" if m <= 16 else "fp8_block_tc_kernel<__nv_bfloat16, BN>",
                dtype="e4m3 weights (128 x 128 block scales) and activations (per token, per 128 of K), f32 accumulate, bf16 out")


def wl_fp8(device, rank, m, n=GEMM_N, k=GEMM_K):
    from emmy_b200 import ops

    gen = torch.Generator(device=device).manual_seed(100 + rank)
    copies = max(2, int(2.2 * 126e6 // (n * k)) + 1)
    ws = [fp8_weight(device, gen, n, k) for _ in range(copies)]
    x_host = torch.randn(m, k, generator=torch.Generator().manual_seed(rank)).bfloat16().pin_memory()
    y_host = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
    x = x_host.to(device)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=device)
    wsp = ops.fp8_workspace(m, k, device)

    def step():
        for w, s in ws:
            ops.fp8_linear(x, w, s, workspace=wsp, out=y)

    return dict(step=step, calls=copies, kernels_per_call=2, alg_bytes=n * k + n * 4 + m * k * 2 + m * n * 2, flops=2.0 * m * k * n, peak_mult=2.0,
                h2d=[(x, x_host)], d2h=[(y_host, y)], status=lambda: ops.fp8_status(wsp, m, k),
                kernel="fp8_gemm_tc_kernel<__nv_bfloat16>" if m > 16 else "fp8_decode_tc_kernel<__nv_bfloat16>",
                dtype="e4m3 weights and activations, f32 accumulate, bf16 out")


def wl_nvfp4(device, rank, m, n=GEMM_N, k=GEMM_K):
    from emmy_b200 import ops_nvfp4 as o4

    gen = torch.Generator(device=device).manual_seed(200 + rank)
    copies = 3
    ws = [nvfp4_weight(device, gen, n, k) for _ in range(copies)]
    x_host = torch.randn(m, k, generator=torch.Generator().manual_seed(rank)).bfloat16().pin_memory()
    y_host = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
    x = x_host.to(device)
    s2 = o4.nvfp4_global_scale(x)  # input_scale calibrated on the sample (emmy/compiler/loader/synthesize.py:181-183)
    y = torch.empty(m, n, dtype=torch.bfloat16, device=device)
    wsp = o4.nvfp4_workspace(m, k, device)

    def step():
        for w, sf, g in ws:
            o4.nvfp4_linear(x, w, sf, g, s2, workspace=wsp, out=y)

    return dict(step=step, calls=copies, kernels_per_call=2, alg_bytes=n * k // 2 + n * k // 16 + 4 + m * k * 2 + m * n * 2, flops=2.0 * m * k * n,
                peak_mult=4.0, h2d=[(x, x_host)], d2h=[(y_host, y)], status=lambda: o4.nvfp4_status(wsp, m, k),
                kernel="nvfp4_gemm_tc_kernel<__nv_bfloat16>", dtype="e2m1 weights and activations with e4m3 block scales, f32 accumulate, bf16 out")


MOE = dict(e=128, topk=8, hidden=2048, inter=768)
MOE_EXPERT_BYTES = 2_451_456  # one expert's packed gate_up + down, zeros and scales (AWQ group 128)


def moe_experts_weights(device, seed, first, count):
    """`count` experts starting at expert `first` of the 128 (seeded per expert, so that every rank draws the same)."""
    from emmy_b200 import ops_moe as om

    h, i = MOE["hidden"], MOE["inter"]

    def stack(k, n, salt):
        qw, qz, sc = [], [], []
        for e in range(first, first + count):
            gen = torch.Generator(device=device).manual_seed(seed + 7919 * e + salt)
            qw.append(torch.randint(-(2**31), 2**31 - 1, (k, n // 8), dtype=torch.int32, device=device, generator=gen))
            qz.append(torch.randint(-(2**31), 2**31 - 1, (k // GROUP, n // 8), dtype=torch.int32, device=device, generator=gen))
            sc.append((torch.rand((k // GROUP, n), device=device, generator=gen) * (2e-2 - 1e-3) + 1e-3).half())
        return torch.stack(qw), torch.stack(qz), torch.stack(sc)

    return om.moe_repack(stack(h, 2 * i, 0), stack(i, h, 1))


def wl_moe(device, rank, world, t, exchange="peer"):
    """Qwen3-30B-A3B expert shapes; with N > 1 ranks the experts are sharded E/N per rank and the tokens travel."""
    from emmy_b200 import ops_moe as om
    from emmy_b200 import shard

    e, topk, hidden, inter = MOE["e"], MOE["topk"], MOE["hidden"], MOE["inter"]
    local_e = e // world
    # decode-sized steps run several layers (distinct weights) per graph, as a decode step does; the figures are per layer
    layers = 4 if (world == 1 and t <= 64) else 1
    ws = [moe_experts_weights(device, 400 + 31 * layer, rank * local_e, local_e) for layer in range(layers)]
    w = ws[0]
    hg = torch.Generator().manual_seed(rank)
    x_host = torch.randn(t, hidden, generator=hg).bfloat16().pin_memory()
    y_host = torch.empty(t, hidden, dtype=torch.bfloat16).pin_memory()
    logits = torch.randn(t, e, generator=hg).to(device)
    x = x_host.to(device)
    y = torch.empty(t, hidden, dtype=torch.bfloat16, device=device)
    if world == 1:
        wsp = om.moe_workspace(t, w, topk, device)

        def step():
            for wl_ in ws:
                om.moe_forward(x, logits, wl_, topk, workspace=wsp, out=y)

        status = lambda: om.moe_status(wsp, t, w, topk)
        capture = True
    elif exchange == "nccl":
        def step():
            ids, scores = om.moe_route(logits, topk)
            out = shard.ep_moe_forward(x, ids, scores, e, lambda rows, eid: om.moe_experts(rows, eid, w),
                                       lambda rows, sc: om.moe_combine(rows, sc, topk))
            y.copy_(out)

        status = lambda: None
        capture = False
    else:
        # EQ_BENCH_EP_CHUNKS > 1 runs the token-sliced form (measured slower at two GPUs: 0.82 ms in two slices, 0.69 ms in one)
        ep = (shard.EpMoePipelined(None, t, topk, hidden, inter, local_e, torch.bfloat16, device, chunks=EP_CHUNKS) if t >= 2048 and EP_CHUNKS > 1
              else shard.EpMoe(None, t, topk, hidden, inter, local_e, torch.bfloat16, device))

        def step():
            ids, scores = om.moe_route(logits, topk)
            ep.forward(x, ids, scores, w, out=y)

        status = ep.status
        capture = True

    def parity():
        """Sampled rows of this rank's output against the single-GPU layer on all 128 experts."""
        rows = torch.from_numpy(np.sort(np.random.default_rng(rank).choice(t, size=min(t, 48), replace=False))).to(device)
        full = w if world == 1 else moe_experts_weights(device, 400, 0, e)
        ref = om.moe_forward(x[rows].contiguous(), logits[rows].contiguous(), full, topk).float()
        return float((y[rows].float() - ref).abs().max() / ref.abs().max())

    if world == 1:
        hit = int(torch.unique(om.moe_route(logits, topk)[0]).numel())  # distinct experts this batch touches
    else:
        hit = local_e  # every local expert is hit by the ranks' tokens at these sizes
    tier = "moe_decode_kernel (two phases)" if (world == 1 and t <= 16) else "moe_stream_kernel (grouped)" if t * topk <= 8 * e else "w4a16_gemm_tc_kernel (grouped)"
    return dict(step=step, calls=layers, kernels_per_call=2 if t <= 16 else 6 if t * topk <= 8 * e else 8, alg_bytes=hit * MOE_EXPERT_BYTES + t * (2 * hidden * 2 + e * 4),
                flops=float(t) * topk * (2.0 * hidden * 2 * inter + 2.0 * inter * hidden), peak_mult=1.0,
                h2d=[(x, x_host)], d2h=[(y_host, y)], status=status, capture=capture, parity=parity if world > 1 else None,
                kernel=tier,
                dtype="int4 expert weights, bf16 activations, f32 accumulate and combine")


def wl_tp_mlp(device, rank, world, m):
    """A Llama-3.1-8B MLP split over the ranks: gate and up column-parallel (no collective), down row-parallel with one
    f32 all-reduce; GPTQ act-order weights, every rank draws the same full weights and keeps its shard."""
    from emmy_b200 import ops, shard

    h, inter = 4096, 14336
    gen = torch.Generator().manual_seed(500)

    def raw(k, n):
        qw = torch.randint(-(2**31), 2**31 - 1, (k // 8, n), dtype=torch.int32, generator=gen)
        qz = torch.full((k // GROUP, n // 8), 0x77777777, dtype=torch.int32)
        sc = (torch.rand((k // GROUP, n), generator=gen) * (2e-2 - 1e-3) + 1e-3).half()
        perm = torch.randperm(k // GROUP, generator=gen)
        return qw, qz, sc, perm[torch.arange(k) // GROUP].int()

    full, local = {}, {}
    for name, (k, n) in (("gate", (h, inter)), ("up", (h, inter)), ("down", (inter, h))):
        t4 = raw(k, n)
        full[name] = ops.w4_repack(*(a.to(device) for a in t4[:3]), GROUP, "gptq", g_idx=t4[3].to(device))
        if name == "down":
            a, b, c, g, rows = shard.row_slice_w4("gptq", *t4, GROUP, rank, world)
        else:
            a, b, c, g = shard.column_slice_w4("gptq", *t4, rank, world)
        local[name] = ops.w4_repack(a.to(device), b.to(device), c.to(device), GROUP, "gptq", g_idx=g.to(device))
    x_host = (torch.randn(m, h, generator=torch.Generator().manual_seed(9)) * 0.25).half().pin_memory()  # the same tokens on every rank
    y_host = torch.empty(m, h, dtype=torch.float16).pin_memory()
    x = x_host.to(device)
    y = torch.empty(m, h, dtype=torch.float16, device=device)
    # decode-sized results are summed by one kernel over NVLink peer memory, larger ones by NCCL
    reducer = shard.PeerAllReduce(None, 64 * h, device) if world > 1 else None
    down = shard.RowParallelLinear(lambda v: ops.w4a16_linear(v, local["down"]), slice(0, inter // world), reducer=reducer)
    peer_sum = reducer is not None and m * h <= reducer.cap

    def mlp(weights, xx):
        return torch.nn.functional.silu(ops.w4a16_linear(xx, weights["gate"])) * ops.w4a16_linear(xx, weights["up"])

    # this rank's gate and up columns as ONE linear ([gate | up], as the reference stores them): one launch for both
    local_gu = ops.w4_concat([local["gate"], local["up"]])
    def step():
        hidden = ops.w4a16_gate_up_swiglu(x, local_gu)  # [M, inter / world]: this rank's columns, SwiGLU in the GEMM's epilogue
        if world > 1:
            down(hidden, sliced=True, out=y)
        else:
            ops.w4a16_linear(hidden, local["down"], out=y)

    def parity():
        rows = torch.arange(0, m, max(1, m // 32), device=device)
        ref = ops.w4a16_linear(mlp(full, x[rows].contiguous()), full["down"]).float()
        return float((y[rows].float() - ref).abs().max() / ref.abs().max())

    return dict(step=step, calls=1, kernels_per_call=5, alg_bytes=sum(algorithmic_bytes(k, n, m) for k, n in SHAPES.values()) // world,
                flops=2.0 * m * 3 * h * inter / world, peak_mult=1.0, h2d=[(x, x_host)], d2h=[(y_host, y)],
                status=(reducer.status if peer_sum else (lambda: None)), capture=True, parity=parity,
                kernel="w4a16 linears + " + ("peer_allreduce_kernel (peer memory)" if peer_sum else "NCCL all-reduce"),
                dtype="int4 weights, f16 activations, f32 accumulate and all-reduce")


# --------------------------------------------------------------------------------------------- records


def measure(wl, device, world, steps, clocks, name, metric, unit, workload):
    """Times one workload and returns its `extra` record."""
    stream = torch.cuda.Stream(device)
    timer = Timer(wl["step"], stream, device, world, capture=wl.get("capture", True))
    with torch.cuda.stream(stream):
        wl["status"]()
    t0 = time.time()
    per_step = [timer.region(steps) / steps for _ in range(SAMPLES)]
    t1 = time.time()
    with torch.cuda.stream(stream):
        wl["status"]()  # after the timed replays too
        e2e_ms = timer.e2e(max(1, min(steps, 5)), wl["h2d"], wl["d2h"])
        parity = wl["parity"]() if wl.get("parity") else None
    med = statistics.median(per_step)
    call_s = med * 1e-3 / wl["calls"]
    units = wl["alg_bytes"] if unit == "GB/s" else wl["flops"]
    scale = 1e9 if unit == "GB/s" else 1e12
    rec = {
        "name": name, "metric": metric, "unit": unit, "value": round(units * world / call_s / scale, 1), "n_gpus": world,
        "ms_per_step": stats(per_step), "us_per_call": round(call_s * 1e6, 2), "calls_per_step": wl["calls"], "steps_per_sample": steps,
        "config": {"workload": workload, "l2": "weights rotate over copies that exceed L2", "launch": "one CUDA graph per step" if wl.get("capture", True) else "eager calls"},
        "dtype": wl["dtype"], "roofline": roofline(wl["alg_bytes"], wl["flops"], wl["peak_mult"], call_s, wl["kernel"]),
        "e2e": {"value": round(units * world / (e2e_ms * 1e-3 / wl["calls"]) / scale, 2), "unit": unit,
                "h2d_bytes_per_step": int(sum(s.numel() * s.element_size() for _, s in wl["h2d"])),
                "d2h_bytes_per_step": int(sum(d.numel() * d.element_size() for d, _ in wl["d2h"]))},
        "clocks": clocks.summary(t0, t1),
    }
    if parity is not None:
        rec["parity_max_rel_err"] = round(parity, 6)
    return rec


def extra_records(device, rank, world, clocks, quick_steps=3):
    """The other calls of the path at the benchmark shapes.  N = 1: every rank-local call.  N > 1: the sharded layers."""
    recs = []

    def add(builder, *a, **kw):
        try:
            wl = builder()
            recs.append(measure(wl, device, world, *a, **kw))
            del wl
        except Exception as exc:  # one record must not take the headline down
            recs.append({"name": kw.get("name") or a[1], "error": f"{type(exc).__name__}: {exc}"[:300]})
        torch.cuda.empty_cache()

    if world == 1:
        for m in (1, 16):
            add(lambda: wl_w4(device, rank, "awq", 4096, 4096, m), quick_steps, clocks, f"awq_4096_m{m}", "w4a16_gemv_hbm_gbs", "GB/s",
                f"AWQ W4A16, K=N=4096, group 128, M={m}")
        for proj, (k, n) in (("gate_up", SHAPES["gate"]), ("down", SHAPES["down"])):
            for m in (4, 16, 24, 64, 256, 8192):
                unit = "GB/s" if m <= 24 else "TFLOP/s"
                add(lambda: wl_w4(device, rank, "gptq", k, n, m), quick_steps, clocks, f"gptq_{proj}_m{m}",
                    "w4a16_gemv_hbm_gbs" if m <= 24 else "w4a16_gemm_tflops", unit, f"GPTQ act-order W4A16, Llama-3.1-8B {proj} K={k} N={n}, M={m}")
        add(lambda: wl_gate_up_fused(device, rank), quick_steps, clocks, "gptq_gate_up_fused_m1", "w4a16_gemv_hbm_gbs", "GB/s",
            "GPTQ act-order W4A16, Llama-3.1-8B gate and up as one [gate | up] linear K=4096 N=28672, M=1: one launch for both projections")
        for m in (1, 16, 2048):
            add(lambda: wl_fp8_block(device, rank, m), quick_steps, clocks, f"fp8_block_m{m}", "fp8_block_hbm_gbs" if m <= 16 else "fp8_block_gemm_tflops",
                "GB/s" if m <= 16 else "TFLOP/s", f"block-scaled FP8 W8A8 (128 x 128 weight blocks, per-token per-128 activation scales, quantize timed), K={GEMM_K} N={GEMM_N} M={m}")
        for m in (1, 32, 512, 8192):
            unit = "GB/s" if m <= 32 else "TFLOP/s"
            add(lambda: wl_fp8(device, rank, m), quick_steps, clocks, f"fp8_m{m}", "fp8_w8a8_hbm_gbs" if m <= 32 else "fp8_w8a8_gemm_tflops", unit,
                f"FP8-E4M3 W8A8, per-channel weight scale, dynamic per-token activation scale (quantize timed), K={GEMM_K} N={GEMM_N} M={m}")
        for m in (1, 128, 4096):
            unit = "GB/s" if m == 1 else "TFLOP/s"
            add(lambda: wl_nvfp4(device, rank, m), quick_steps, clocks, f"nvfp4_m{m}", "nvfp4_hbm_gbs" if m == 1 else "nvfp4_gemm_tflops", unit,
                f"NVFP4 W4A4, weights N(0,0.02) through the two-level weight quantizer, static activation scale (quantize timed), K={GEMM_K} N={GEMM_N} M={m}")
        for t in (1, 64, 4096):
            unit = "GB/s" if t <= 64 else "TFLOP/s"
            add(lambda: wl_moe(device, rank, 1, t), quick_steps, clocks, f"moe_t{t}", "moe_hbm_gbs" if t <= 64 else "moe_w4a16_tflops", unit,
                f"routed W4A16 MoE layer, Qwen3-30B-A3B shapes (128 experts, top-8, hidden 2048, intermediate 768, AWQ group 128), T={t}")
    else:
        add(lambda: wl_moe(device, rank, world, 4096, "peer"), quick_steps, clocks, "moe_ep_t4096", "moe_w4a16_tflops", "TFLOP/s",
            f"expert-parallel MoE, {128 // world} experts per rank, T=4096 tokens per rank, rows stored into the owner's receive buffer and results "
            "stored back from the second GEMM's epilogue over NVLink peer memory")
        for m in (16, 2048):
            add(lambda: wl_tp_mlp(device, rank, world, m), quick_steps, clocks, f"tp_mlp_m{m}", "w4a16_mlp_tflops", "TFLOP/s",
                f"tensor-parallel Llama-3.1-8B MLP over {world} ranks: gate/up column-parallel, down row-parallel + f32 sum of the partials "
                f"({'one kernel over NVLink peer memory' if m * 4096 <= 64 * 4096 else 'NCCL all-reduce'}), M={m}")
    return recs


# --------------------------------------------------------------------------------------------- our arm


def run_ours(args, rank, world, local_rank):
    from emmy_b200.build import build

    if not (ROOT / "emmy_b200" / "libemmyq.so").exists():
        build()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    warmup = max(args.warmup, 3)
    with ClockSampler(local_rank) as clocks:
        wl = wl_gemv_stack(device, rank)
        stream = torch.cuda.Stream(device)
        timer = Timer(wl["step"], stream, device, world, warmup=warmup)
        # ---- the timed region of the contract: K steps, weights resident, device time, max over ranks
        t0 = time.time()
        dev_ms = timer.region(args.steps)
        t1 = time.time()
        if dev_ms < 400:  # keep the clock sampler fed on short runs
            end = time.time() + 0.4
            while time.time() < end:
                timer.run()
            stream.synchronize()
            t1 = time.time()
        samples = [timer.region(args.steps) / args.steps for _ in range(SAMPLES)]
        e2e_ms = timer.e2e(args.steps, wl["h2d"], wl["d2h"]) * args.steps
        eager = Timer(wl["step"], stream, device, world, capture=False)
        eager_ms = eager.e2e(max(1, min(args.steps, 5)), wl["h2d"], wl["d2h"])
        hot = Timer(wl["hot_step"], stream, device, world)
        hot_ms = statistics.median(hot.region(args.steps) / args.steps for _ in range(3))
        with torch.cuda.stream(stream):
            wl["status"]()
        headline_clocks = clocks.summary(t0, t1)
        del timer, eager, hot, wl
        torch.cuda.empty_cache()
        extras = [] if args.no_extra else extra_records(device, rank, world, clocks)
    if rank != 0:
        return
    hbm, _, _, peak_kind = peaks()
    total_bytes = STEP_BYTES * world
    value = total_bytes * args.steps / (dev_ms * 1e-3) / 1e9
    launches = 3 * LAYERS
    per_launch_us = dev_ms * 1e3 / (args.steps * launches)
    achieved = (STEP_BYTES / launches) / (per_launch_us * 1e-6) / 1e9
    line = {
        "metric": "w4a16_m1_gemv_hbm_gbs",
        "value": round(value, 1),
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": round(dev_ms / args.steps, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "int4 weights, f16 activations, f32 accumulate",
        "data": "synthetic",
        "config": {
            "workload": "gptq_llama8b_mlp_m1: GPTQ-Int4 act-order W4A16 GEMV, Llama-3.1-8B MLP shapes (gate/up 4096x14336, down 14336x4096, group 128), M=1, 32-layer stack per GPU",
            "algorithmic_bytes_per_step": STEP_BYTES,
            "l2": "inputs larger than L2: 2.9 GB of weights streamed per step",
            "launch": "one CUDA graph of 96 GEMV launches per step",
        },
        "e2e": {
            "value": round(total_bytes * args.steps / (e2e_ms * 1e-3) / 1e9, 1),
            "unit": "GB/s",
            "h2d_bytes_per_step": 2 * (4096 + 14336),
            "d2h_bytes_per_step": 2 * (14336 + 14336 + 4096),
            "eager_calls_value": round(total_bytes / (eager_ms * 1e-3) / 1e9, 1),
        },
        "gpu_launches": launches * args.steps,
        "roofline": {
            "bound": "hbm",
            "achieved": round(achieved, 1),
            "peak": hbm,
            "unit": "GB/s",
            "frac": round(achieved / hbm, 4),
            "peak_kind": peak_kind,
            "traffic": TRAFFIC_PER_LAUNCH,
            "kernel": GEMV_KERNEL,
            "avg_launch_us": round(per_launch_us, 3),
        },
        "samples": {"ms_per_step": stats(samples), "gbs_median": round(total_bytes / (statistics.median(samples) * 1e-3) / 1e9, 1),
                    "hot_l2_gbs": round(total_bytes / (hot_ms * 1e-3) / 1e9, 1),
                    "note": f"{SAMPLES} repeats of the {args.steps}-step region after the contract's region; hot_l2: one layer's weights (92 MB) replayed, resident in L2"},
        "clocks": headline_clocks,
        "cpu_baseline": cpu_baseline(sample_layers=1),
        "extra": extras,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------- one workload alone


def cpu_sample(name, m):
    """The oracle port on a bounded sample of a secondary workload's rows; (units, seconds, description)."""
    from oracle import linear as ol
    from oracle import moe as omoe
    from oracle import synth

    if name == "fp8_gemm":
        rows = min(m, 16)
        wb, wsc = synth.fp8_weight(GEMM_N, GEMM_K, seed=0)
        x = synth.activations(rows, GEMM_K, "bf16")
        t0 = time.perf_counter()
        ol.fp8_linear(x, wb, wsc)
        return 2.0 * rows * GEMM_K * GEMM_N, time.perf_counter() - t0, f"{rows} of {m} rows: numpy dequantize, per-token round trip, f32 matmul"
    if name == "nvfp4_gemm":
        rows = min(m, 16)
        packed, sb, s2 = synth.nvfp4_weight(2048, GEMM_K, seed=0)
        x = synth.activations(rows, GEMM_K, "bf16")
        from oracle import activations as oa

        t0 = time.perf_counter()
        ol.nvfp4_linear(x, packed, sb, s2, oa.nvfp4_global_scale(x))
        return 2.0 * rows * GEMM_K * 2048, time.perf_counter() - t0, f"{rows} of {m} rows, 2048 of {GEMM_N} output channels: numpy dequantize, static activation round trip, f32 matmul"
    if name == "w4a16_prefill":
        rows = min(m, 16)
        k, n = SHAPES["gate"]
        qw, qz, sc, gi = synth.gptq_linear(k, n, seed=0)
        x = synth.activations(rows, k, "f16")
        t0 = time.perf_counter()
        ol.w4a16_linear(x, qw, qz, sc, GROUP, "gptq", "f16", gi)
        return 2.0 * rows * k * n, time.perf_counter() - t0, f"{rows} of {m} rows: numpy dequantize (g_idx gather) + f32 matmul"
    # moe: one token's eight experts, dense dequantised
    hidden, inter = 2048, 768
    gu = [synth.awq_linear(hidden, 2 * inter, seed=2 * i) for i in range(8)]
    dn = [synth.awq_linear(inter, hidden, seed=2 * i + 1) for i in range(8)]
    ex = {"gate_up": tuple(np.stack([p[j] for p in gu]) for j in range(3)), "down": tuple(np.stack([p[j] for p in dn]) for j in range(3))}
    x = torch.from_numpy(synth.activations(1, hidden, "bf16")).bfloat16()
    logits = torch.randn(1, 8, generator=torch.Generator().manual_seed(0))
    t0 = time.perf_counter()
    wgu, wdn = omoe.dequant_expert_weights(ex, torch.bfloat16)
    omoe.moe_layer(x, logits, wgu, wdn, 8)
    return 8 * (2.0 * hidden * 2 * inter + 2.0 * inter * hidden), time.perf_counter() - t0, "1 token, its 8 experts: numpy dequantize + bf16 torch CPU expert FFN + f32 combine"


def run_other(args, rank, world, local_rank):
    from emmy_b200.build import build

    if not (ROOT / "emmy_b200" / "libemmyq.so").exists():
        build()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    name = args.workload
    m = args.rows or {"fp8_gemm": 8192, "fp8_block_gemm": 2048, "nvfp4_gemm": 4096, "w4a16_prefill": 2048, "moe": 4096}[name]
    if name == "moe":
        wl, metric = wl_moe(device, rank, world, m, args.exchange), "moe_w4a16_tflops"
    elif name == "fp8_gemm":
        wl, metric = wl_fp8(device, rank, m), "fp8_w8a8_gemm_tflops"
    elif name == "fp8_block_gemm":
        wl, metric = wl_fp8_block(device, rank, m), "fp8_block_gemm_tflops"
    elif name == "nvfp4_gemm":
        wl, metric = wl_nvfp4(device, rank, m), "nvfp4_gemm_tflops"
    else:
        wl, metric = wl_w4(device, rank, "gptq", *SHAPES["gate"], m), "w4a16_gemm_tflops"
    stream = torch.cuda.Stream(device)
    warmup = max(args.warmup, 3)
    timer = Timer(wl["step"], stream, device, world, capture=wl.get("capture", True), warmup=warmup)
    with torch.cuda.stream(stream):
        wl["status"]()
    with ClockSampler(local_rank) as clocks:
        dev_ms = timer.region(args.steps)
        if dev_ms < 400:
            for _ in range(min(5000, int(400.0 / max(dev_ms / args.steps, 1e-3)) + 1)):
                timer.run()
            stream.synchronize()
    with torch.cuda.stream(stream):
        wl["status"]()
    e2e_ms = timer.e2e(max(1, min(args.steps, 5)), wl["h2d"], wl["d2h"])
    if rank != 0:
        return
    step_ms = dev_ms / args.steps
    call_s = step_ms * 1e-3 / wl["calls"]
    units, secs, what = cpu_sample(name, m)
    line = {
        "metric": metric, "value": round(wl["flops"] * wl["calls"] * world / (step_ms * 1e-3) / 1e12, 1), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": round(step_ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": f"{name} rows={m}", "flops_per_call": wl["flops"], "calls_per_step": wl["calls"],
                   "algorithmic_bytes_per_call": wl["alg_bytes"], "l2": "weights rotate over distinct copies that exceed L2",
                   "launch": "one CUDA graph per step" if wl.get("capture", True) else "eager calls"},
        "e2e": {"value": round(wl["flops"] * wl["calls"] * world / (e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": int(sum(s.numel() * s.element_size() for _, s in wl["h2d"])),
                "d2h_bytes_per_step": int(sum(d.numel() * d.element_size() for d, _ in wl["d2h"]))},
        "gpu_launches": wl["calls"] * wl["kernels_per_call"] * args.steps,
        "roofline": roofline(wl["alg_bytes"], wl["flops"], wl["peak_mult"], call_s, wl["kernel"]),
        "clocks": clocks.summary(),
        "cpu_baseline": {"value": round(units / secs / 1e12, 6), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": f"{what}, {secs:.1f} s"},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------- CPU arm


def cpu_threads() -> int:
    return max(1, min(os.cpu_count() or 1, 64))


def cpu_layer_inputs(seed: int = 0):
    """One layer's three GPTQ projections and their activations (synthetic; generated outside any timed region)."""
    from oracle import synth

    out = []
    for k, n in SHAPES.values():
        qw, qz, sc, gi = synth.gptq_linear(k, n, seed=seed)
        x = torch.from_numpy(synth.activations(1, k, "f16", seed=seed + 1)).half()
        out.append((k, n, qw, qz, sc, gi, x))
    return out


def cpu_layer_seconds(inputs):
    """The reference's CPU path for one layer's three projections at M=1: numpy dequantize (with the g_idx gather;
    column chunks on all host threads), one rounding to fp16, torch CPU linear.  Returns (seconds, algorithmic bytes)."""
    from concurrent.futures import ThreadPoolExecutor

    from oracle import formats as fm

    threads = cpu_threads()
    torch.set_num_threads(threads)
    total_s, total_b = 0.0, 0
    with ThreadPoolExecutor(max_workers=threads) as pool:
        for k, n, qw, qz, sc, gi, x in inputs:
            step = max(8, (n // threads + 7) // 8 * 8)
            chunks = [(c, min(c + step, n)) for c in range(0, n, step)]
            t0 = time.perf_counter()
            parts = list(pool.map(lambda ab: fm.dequant_w4(qw[:, ab[0]:ab[1]], qz[:, ab[0] // 8:ab[1] // 8], sc[:, ab[0]:ab[1]], GROUP, "gptq", gi), chunks))
            w = np.concatenate(parts, axis=1)
            wt = torch.from_numpy(np.ascontiguousarray(w.T)).half()
            torch.nn.functional.linear(x, wt)
            total_s += time.perf_counter() - t0
            total_b += algorithmic_bytes(k, n)
    return total_s, total_b


def cpu_baseline(sample_layers: int = 1):
    secs, nbytes = 0.0, 0
    for i in range(sample_layers):
        s, b = cpu_layer_seconds(cpu_layer_inputs(seed=i))
        secs += s
        nbytes += b
    return {
        "value": round(nbytes / secs / 1e9, 4),
        "unit": "GB/s",
        "cores": cpu_threads(),
        "kind": "port",
        "sample": f"{sample_layers} of 32 layers (gate, up, down at M=1): numpy dequantize in column chunks on all host threads + fp16 torch CPU linear, {secs:.1f} s",
    }


def run_reference(args, rank):
    """The reference's CPU implementation of the path (the oracle port: the reference itself is Python plus a Rust runtime
    that does not build here), one layer of the stack per step, inputs generated outside the timed region."""
    if rank != 0:
        return
    warmup = max(args.warmup, 0)
    inputs = [cpu_layer_inputs(seed=i) for i in range(min(args.steps, 4))]  # steps cycle over a few distinct layers
    for i in range(warmup):
        cpu_layer_seconds(inputs[i % len(inputs)])
    secs, nbytes = 0.0, 0
    for i in range(args.steps):
        s, b = cpu_layer_seconds(inputs[i % len(inputs)])
        secs += s
        nbytes += b
    value = nbytes / secs / 1e9
    line = {
        "impl": "reference",
        "metric": "w4a16_m1_gemv_hbm_gbs",
        "value": round(value, 4),
        "unit": "GB/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": round(secs * 1e3 / args.steps, 2),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "int4 weights, f16 activations, f32 accumulate",
        "data": "synthetic",
        "config": {
            "workload": "gptq_llama8b_mlp_m1: GPTQ-Int4 act-order W4A16 GEMV, Llama-3.1-8B MLP shapes (gate/up 4096x14336, down 14336x4096, group 128), M=1, 32-layer stack per GPU",
            "sample": "each step is ONE layer (gate, up, down) of the 32-layer stack on the host cores; inputs are generated before the timed region",
        },
        "cpu_baseline": {
            "value": round(value, 4),
            "unit": "GB/s",
            "cores": cpu_threads(),
            "kind": "port",
            "sample": "1 of 32 layers per step: numpy dequantize (g_idx gather) in column chunks on all host threads + fp16 torch CPU linear",
        },
        "e2e": {"value": round(value, 4), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gptq_llama8b_mlp_m1",
                    choices=["gptq_llama8b_mlp_m1", "w4a16_prefill", "fp8_gemm", "fp8_block_gemm", "nvfp4_gemm", "moe"])
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="moe workload at N > 1: who moves the tokens")
    ap.add_argument("--rows", type=int, default=0, help="rows (tokens) of the secondary workloads; 0 = the workload's default")
    ap.add_argument("--no-extra", action="store_true", help="headline only: skip the extra records")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "gptq_llama8b_mlp_m1":
            run_ours(args, rank, world, local_rank)
        else:
            run_other(args, rank, world, local_rank)
    finally:
        if world > 1:
            torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
