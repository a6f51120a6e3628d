#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME [--rows ROWS]]

Default workload (`gptq_llama8b_mlp_m1`): the W4A16 M=1 GEMV on GPTQ act-order weights with the
Llama-3.1-8B MLP shapes (gate/up K=4096 N=14336, down K=14336 N=4096, group 128) -- one step is one pass
over a 32-layer stack of gate, up and down projections (96 GEMVs, 2.9 GB of packed weights, far larger
than L2, so every step streams its weights from HBM).  Metric: algorithmic HBM bytes per second.

Prints ONE JSON line on rank 0.  Launched by torchrun for N > 1 (one rank per GPU); every rank then owns its
own 32-layer stack (weak scaling: independent layers, no data-path collective).
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


def algorithmic_bytes(k: int, n: int, m: int = 1) -> int:
    """Bytes one GEMV must move, exactly as the checkpoint stores them: packed weight, packed zeros,
    fp16 scales, g_idx, x and y."""
    return k * n // 2 + (k // GROUP) * n // 2 + (k // GROUP) * n * 2 + k * 4 + m * k * 2 + m * n * 2


STEP_BYTES = LAYERS * sum(algorithmic_bytes(k, n) for k, n in SHAPES.values())


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def tensor_peaks():
    """(burst, sustained) dense bf16 TFLOP/s; FP8 runs at twice and NVFP4 at four times these."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

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
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
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


# --------------------------------------------------------------------------------------------- our arm


def build_stack(device, seed: int):
    """32 layers of GPTQ act-order weights, generated on the device and repacked at load time."""
    from emmy_b200 import ops

    gen = torch.Generator(device=device).manual_seed(seed)
    stack = []
    for _ in range(LAYERS):
        layer = {}
        for name, (k, n) in SHAPES.items():
            qweight = torch.randint(-(2**31), 2**31 - 1, (k // 8, n), dtype=torch.int32, device=device, generator=gen)
            qzeros = torch.full((k // GROUP, n // 8), 0x77777777, dtype=torch.int32, device=device)  # stored 7 = zero 8
            scales = (torch.rand((k // GROUP, n), device=device, generator=gen) * (2e-2 - 1e-3) + 1e-3).half()
            perm = torch.randperm(k // GROUP, device=device, generator=gen)
            g_idx = perm[torch.arange(k, device=device) // GROUP].int()
            layer[name] = ops.w4_repack(qweight, qzeros, scales, GROUP, "gptq", g_idx=g_idx)
        stack.append(layer)
    torch.cuda.synchronize()
    return stack


def run_ours(args, rank, world, local_rank):
    from emmy_b200 import ops
    from emmy_b200.build import build

    if not (ROOT / "emmy_b200" / "libemmyq.so").exists():
        build()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    stack = build_stack(device, seed=1234 + rank)
    gen = torch.Generator().manual_seed(7 + rank)
    x_host = torch.randn(1, 4096, generator=gen).half().pin_memory()
    h_host = torch.randn(1, 14336, generator=gen).half().pin_memory()
    x, h = x_host.to(device), h_host.to(device)
    ys = {name: torch.empty(1, n, dtype=torch.float16, device=device) for name, (_, n) in SHAPES.items()}
    ws = torch.zeros(1 << 20, dtype=torch.uint8, device=device)
    out_host = {name: torch.empty(1, n, dtype=torch.float16).pin_memory() for name, (_, n) in SHAPES.items()}

    def step():
        for layer in stack:
            ops.w4a16_linear(x, layer["gate"], workspace=ws, out=ys["gate"])
            ops.w4a16_linear(x, layer["up"], workspace=ws, out=ys["up"])
            ops.w4a16_linear(h, layer["down"], workspace=ws, out=ys["down"])

    stream = torch.cuda.Stream(device)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        for _ in range(2):
            graph.replay()
        stream.synchronize()

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                torch.distributed.barrier()
            torch.cuda.synchronize()

        # ---- device-timed region: weights resident, K steps
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            start.record(stream)
            for _ in range(args.steps):
                graph.replay()
            end.record(stream)
            end.synchronize()
            dev_ms = start.elapsed_time(end)
            # keep the sampler fed for short runs
            if dev_ms < 400:
                t_end = time.time() + 0.4
                while time.time() < t_end:
                    graph.replay()
                stream.synchronize()
        barrier()

        # ---- end to end through the operator API with host buffers
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            x.copy_(x_host, non_blocking=True)
            h.copy_(h_host, non_blocking=True)
            graph.replay()
            for name in ys:
                out_host[name].copy_(ys[name], non_blocking=True)
            stream.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        barrier()
        # the same with one operator call per projection instead of the captured graph (reported, not the headline)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            x.copy_(x_host, non_blocking=True)
            h.copy_(h_host, non_blocking=True)
            step()
            for name in ys:
                out_host[name].copy_(ys[name], non_blocking=True)
            stream.synchronize()
        eager_ms = (time.perf_counter() - t0) * 1e3
        barrier()

    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    dev_ms, e2e_ms = times.tolist()
    if rank != 0:
        return
    peak, peak_kind = peaks()
    total_bytes = STEP_BYTES * world
    value = total_bytes * args.steps / (dev_ms * 1e-3) / 1e9
    e2e_value = total_bytes * args.steps / (e2e_ms * 1e-3) / 1e9
    launches = 3 * LAYERS
    per_launch_us = dev_ms * 1e3 / (args.steps * launches)
    achieved = (STEP_BYTES / launches) / (per_launch_us * 1e-6) / 1e9
    line = {
        "metric": "w4a16_m1_gemv_hbm_gbs",
        "value": round(value, 1),
        "unit": "GB/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
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
            "value": round(e2e_value, 1),
            "unit": "GB/s",
            "h2d_bytes_per_step": int(x_host.numel() * 2 + h_host.numel() * 2),
            "d2h_bytes_per_step": int(sum(t.numel() * 2 for t in out_host.values())),
            "eager_calls_value": round(STEP_BYTES * args.steps / (eager_ms * 1e-3) / 1e9, 1),
        },
        "gpu_launches": launches * args.steps,
        "roofline": {
            "bound": "hbm",
            "achieved": round(achieved, 1),
            "peak": peak,
            "unit": "GB/s",
            "frac": round(achieved / peak, 4),
            "peak_kind": peak_kind,
            "traffic": TRAFFIC_PER_LAUNCH,
            "kernel": "w4a16_stream_kernel<__half,1,true>",
            "avg_launch_us": round(per_launch_us, 3),
        },
        "clocks": clocks.summary(),
        "cpu_baseline": cpu_baseline(sample_layers=1),
    }
    print(json.dumps(line), flush=True)


# dram bytes per launch of the GEMV kernel (dram__bytes_read.sum + dram__bytes_write.sum, mean of three launches of this
# workload) from the ncu capture summarised in profiles/w4a16_stream_kernel_gptq_m1.md
TRAFFIC_PER_LAUNCH = 31224000


# --------------------------------------------------------------------------------------------- other workloads
#
# The same contract for the other calls of the path; `--workload NAME [--rows ROWS]`.  One step = `copies` calls on distinct
# weight copies (so that weights come from HBM, not L2), captured in one CUDA graph where the call has no host read.

GEMM_K, GEMM_N = 5120, 17408


def _wl_fp8(device, rank, m):
    from emmy_b200 import ops

    gen = torch.Generator(device=device).manual_seed(100 + rank)
    copies = 2
    ws = []
    for _ in range(copies):
        w = (torch.randn(GEMM_N, GEMM_K, device=device, generator=gen) * 0.02)
        s = w.abs().amax(dim=1).clamp_min(1e-12) / 448.0
        ws.append(((w / s[:, None]).to(torch.float8_e4m3fn).view(torch.uint8), s.float().contiguous()))
    x_host = torch.randn(m, GEMM_K, generator=torch.Generator().manual_seed(rank)).bfloat16().pin_memory()
    x = x_host.to(device)
    y = torch.empty(m, GEMM_N, dtype=torch.bfloat16, device=device)
    wsp = ops.fp8_workspace(m, GEMM_K, device)

    def step():
        for w, s in ws:
            ops.fp8_linear(x, w, s, workspace=wsp, out=y)

    return dict(
        step=step, flops=2.0 * m * GEMM_K * GEMM_N * copies, calls=copies, kernels_per_call=2, x=x, x_host=x_host, y=y, graph=True,
        metric="fp8_w8a8_gemm_tflops", dtype="e4m3 weights and activations, f32 accumulate, bf16 out", peak_mult=2.0,
        kernel="fp8_gemm_tc_kernel<__nv_bfloat16>" if m > 64 else "fp8_smallm_kernel",
        status=lambda: ops.fp8_status(wsp, m, GEMM_K),
        workload=f"fp8_gemm: FP8-E4M3 W8A8, per-channel weight scale, dynamic per-token activation scale (quantize timed), K={GEMM_K} N={GEMM_N} M={m}, bf16 out",
        alg_bytes=GEMM_N * GEMM_K + GEMM_N * 4 + m * GEMM_K * 2 + m * GEMM_N * 2,
    )


def _wl_nvfp4(device, rank, m):
    from emmy_b200 import ops_nvfp4 as o4

    gen = torch.Generator(device=device).manual_seed(200 + rank)
    copies = 3
    ws = []
    for _ in range(copies):
        w = torch.randint(0, 256, (GEMM_N, GEMM_K // 2), dtype=torch.uint8, device=device, generator=gen)
        sf = torch.randint(0x28, 0x40, (GEMM_N, GEMM_K // 16), dtype=torch.uint8, device=device, generator=gen)
        ws.append((w, o4.nvfp4_tile_weight_scales(sf, GEMM_K), torch.tensor([2.0e-5], device=device)))
    x_host = torch.randn(m, GEMM_K, generator=torch.Generator().manual_seed(rank)).bfloat16().pin_memory()
    x = x_host.to(device)
    s2 = o4.nvfp4_global_scale(x)
    y = torch.empty(m, GEMM_N, dtype=torch.bfloat16, device=device)
    wsp = o4.nvfp4_workspace(m, GEMM_K, device)

    def step():
        for w, sf, g in ws:
            o4.nvfp4_linear(x, w, sf, g, s2, workspace=wsp, out=y)

    return dict(
        step=step, flops=2.0 * m * GEMM_K * GEMM_N * copies, calls=copies, kernels_per_call=2, x=x, x_host=x_host, y=y, graph=True,
        metric="nvfp4_gemm_tflops", dtype="e2m1 weights and activations with e4m3 block scales, f32 accumulate, bf16 out", peak_mult=4.0,
        kernel="nvfp4_gemm_tc_kernel<__nv_bfloat16>", status=lambda: o4.nvfp4_status(wsp, m, GEMM_K),
        workload=f"nvfp4_gemm: NVFP4 block-scaled W4A4 (codes uniform, block scales uniform 0x28..0x3F: synthetic codes stand in for quantized N(0,0.02) weights), static activation scale (quantize timed), K={GEMM_K} N={GEMM_N} M={m}, bf16 out",
        alg_bytes=GEMM_N * GEMM_K // 2 + GEMM_N * GEMM_K // 16 + 4 + m * GEMM_K * 2 + m * GEMM_N * 2,
    )


def _wl_w4_prefill(device, rank, m):
    from emmy_b200 import ops

    gen = torch.Generator(device=device).manual_seed(300 + rank)
    k, n = SHAPES["gate"]
    copies = 4
    ws = []
    for _ in range(copies):
        qweight = torch.randint(-(2**31), 2**31 - 1, (k // 8, n), dtype=torch.int32, device=device, generator=gen)
        qzeros = torch.full((k // GROUP, n // 8), 0x77777777, dtype=torch.int32, device=device)
        scales = (torch.rand((k // GROUP, n), device=device, generator=gen) * (2e-2 - 1e-3) + 1e-3).half()
        perm = torch.randperm(k // GROUP, device=device, generator=gen)
        g_idx = perm[torch.arange(k, device=device) // GROUP].int()
        ws.append(ops.w4_repack(qweight, qzeros, scales, GROUP, "gptq", g_idx=g_idx))
    x_host = torch.randn(m, k, generator=torch.Generator().manual_seed(rank)).half().pin_memory()
    x = x_host.to(device)
    y = torch.empty(m, n, dtype=torch.float16, device=device)
    wsp = torch.zeros(ops.L.load().eq_w4a16_workspace_bytes(m, n, k) + 256, dtype=torch.uint8, device=device)

    def step():
        for w in ws:
            ops.w4a16_linear(x, w, workspace=wsp, out=y)

    return dict(
        step=step, flops=2.0 * m * k * n * copies, calls=copies, kernels_per_call=1, x=x, x_host=x_host, y=y, graph=True,
        metric="w4a16_gemm_tflops", dtype="int4 weights dequantised to f16 in shared memory, f16 activations, f32 accumulate", peak_mult=1.0,
        kernel="w4a16_gemm_tc_kernel<__half>", status=lambda: ops.w4a16_status(wsp, m, n),
        workload=f"w4a16_prefill: GPTQ-Int4 act-order W4A16, Llama-3.1-8B gate/up shape K={k} N={n} group 128, M={m}",
        alg_bytes=algorithmic_bytes(k, n, m),
    )


def _wl_moe(device, rank, world, t, exchange="peer"):
    """Qwen3-30B-A3B expert shapes; with N > 1 ranks the experts are sharded E/N per rank and tokens travel by all-to-all."""
    from emmy_b200 import ops_moe as om
    from emmy_b200 import shard

    e, topk, hidden, inter = 128, 8, 2048, 768
    local_e = e // world
    gen = torch.Generator(device=device).manual_seed(400 + rank)

    def stack(k, n):
        qw = torch.randint(-(2**31), 2**31 - 1, (local_e, k, n // 8), dtype=torch.int32, device=device, generator=gen)
        qz = torch.randint(-(2**31), 2**31 - 1, (local_e, k // GROUP, n // 8), dtype=torch.int32, device=device, generator=gen)
        sc = (torch.rand((local_e, k // GROUP, n), device=device, generator=gen) * (2e-2 - 1e-3) + 1e-3).half()
        return qw, qz, sc

    w = om.moe_repack(stack(hidden, 2 * inter), stack(inter, hidden))
    hg = torch.Generator().manual_seed(rank)
    x_host = torch.randn(t, hidden, generator=hg).bfloat16().pin_memory()
    logits = torch.randn(t, e, generator=hg).to(device)
    x = x_host.to(device)
    y = torch.empty(t, hidden, dtype=torch.bfloat16, device=device)
    if world == 1:
        wsp = om.moe_workspace(t, w, topk, device)

        def step():
            om.moe_forward(x, logits, w, topk, workspace=wsp, out=y)

        status = lambda: om.moe_status(wsp, t, w, topk)
    elif exchange == "nccl":
        def step():
            ids, scores = om.moe_route(logits, topk)
            out = shard.ep_moe_forward(x, ids, scores, e, lambda rows, eid: om.moe_experts(rows, eid, w),
                                       lambda rows, sc: om.moe_combine(rows, sc, topk))
            y.copy_(out)

        status = lambda: None
    else:
        ep = shard.EpMoe(None, t, topk, hidden, inter, local_e, torch.bfloat16, device)

        def step():
            ids, scores = om.moe_route(logits, topk)
            ep.forward(x, ids, scores, w, out=y)

        status = ep.status
    return dict(
        step=step, flops=float(t) * topk * (2.0 * hidden * 2 * inter + 2.0 * inter * hidden), calls=1, kernels_per_call=8, x=x, x_host=x_host,
        y=y, graph=world == 1 or exchange == "peer", metric="moe_w4a16_tflops", dtype="int4 expert weights, bf16 activations, f32 accumulate and combine",
        peak_mult=1.0, kernel="moe_expert_gemm_kernel", status=status,
        workload=f"moe: routed W4A16 expert layer, Qwen3-30B-A3B shapes (128 experts, top-8, hidden 2048, intermediate 768, AWQ group 128), T={t} tokens per rank"
        + (f", experts sharded {local_e} per rank, " + ("all-to-all dispatch and return over NCCL" if exchange == "nccl" else
            "rows stored into the owner's receive buffer and results stored back from the second GEMM's epilogue over NVLink peer memory")
           if world > 1 else ""),
        alg_bytes=None,
    )


def cpu_sample(name, m):
    """The oracle port on a bounded sample of the workload's rows; (units, seconds, description)."""
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
    default_m = {"fp8_gemm": 8192, "nvfp4_gemm": 4096, "w4a16_prefill": 2048, "moe": 4096}[name]
    m = args.rows or default_m
    wl = _wl_moe(device, rank, world, m, args.exchange) if name == "moe" else {"fp8_gemm": _wl_fp8, "nvfp4_gemm": _wl_nvfp4, "w4a16_prefill": _wl_w4_prefill}[name](device, rank, m)
    step = wl["step"]
    stream = torch.cuda.Stream(device)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        stream.synchronize()
        wl["status"]()
        run = step
        if wl["graph"]:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step()
            graph.replay()
            stream.synchronize()
            run = graph.replay
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            start.record(stream)
            for _ in range(args.steps):
                run()
            end.record(stream)
            end.synchronize()
            dev_ms = start.elapsed_time(end)
            # keep the clock sampler fed on short runs: the same number of extra steps on every rank (the steps may be collective)
            feed = torch.tensor([dev_ms / args.steps], dtype=torch.float64, device=device)
            if world > 1:
                torch.distributed.all_reduce(feed, op=torch.distributed.ReduceOp.MAX)
            if dev_ms < 400:
                for _ in range(min(5000, int(400.0 / max(feed.item(), 1e-3)) + 1)):
                    run()
                stream.synchronize()
        barrier()
        # end to end: the step's activations come from pinned host memory, its result goes back
        y_host = torch.empty(wl["y"].shape, dtype=wl["y"].dtype).pin_memory()
        e2e_steps = max(1, min(args.steps, 5))
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            wl["x"].copy_(wl["x_host"], non_blocking=True)
            run()
            y_host.copy_(wl["y"], non_blocking=True)
            stream.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        barrier()
    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(times, op=torch.distributed.ReduceOp.MAX)
    dev_ms, e2e_ms = times.tolist()
    if rank != 0:
        return
    burst, sustained, kind = tensor_peaks()
    step_ms = dev_ms / args.steps
    value = wl["flops"] * world / (step_ms * 1e-3) / 1e12
    per_call_us = step_ms * 1e3 / wl["calls"]
    achieved = wl["flops"] / wl["calls"] / (per_call_us * 1e-6) / 1e12
    peak = sustained * wl["peak_mult"]
    units, secs, what = cpu_sample(name, m)
    line = {
        "metric": wl["metric"], "value": round(value, 1), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(step_ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": wl["workload"], "flops_per_step": wl["flops"], "calls_per_step": wl["calls"],
                   "l2": "weights rotate over distinct copies and activations plus outputs exceed L2",
                   "launch": "one CUDA graph per step" if wl["graph"] else "eager calls"},
        "e2e": {"value": round(wl["flops"] * world / (e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                "h2d_bytes_per_step": int(wl["x_host"].numel() * wl["x_host"].element_size()),
                "d2h_bytes_per_step": int(y_host.numel() * y_host.element_size())},
        "gpu_launches": wl["calls"] * wl["kernels_per_call"] * args.steps,
        "roofline": {"bound": "tensor", "achieved": round(achieved, 1), "peak": round(peak, 1), "unit": "TFLOP/s",
                     "frac": round(achieved / peak, 4), "peak_kind": f"{kind}: {wl['peak_mult']:g} x sustained bf16 {sustained} (burst {burst})",
                     "frac_of_burst": round(achieved / (burst * wl["peak_mult"]), 4), "traffic": None, "kernel": wl["kernel"],
                     "avg_call_us": round(per_call_us, 2), "includes": "activation quantize and the GEMM of each call"},
        "clocks": clocks.summary(),
        "cpu_baseline": {"value": round(units / secs / 1e12, 6), "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": f"{what}, {secs:.1f} s"},
    }
    if wl["alg_bytes"]:
        line["config"]["algorithmic_bytes_per_call"] = wl["alg_bytes"]
        line["roofline"]["hbm_gbs"] = round(wl["alg_bytes"] / (per_call_us * 1e-6) / 1e9, 1)
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------- CPU arm


def cpu_threads() -> int:
    return max(1, min(os.cpu_count() or 1, 64))


def cpu_layer_seconds(seed: int = 0):
    """The reference's CPU path for one layer's three projections at M=1: numpy dequantize (with the g_idx
    gather; column chunks on all host threads), one rounding to fp16, torch CPU linear.  Returns (seconds,
    algorithmic bytes)."""
    from concurrent.futures import ThreadPoolExecutor

    from oracle import formats as fm
    from oracle import synth

    threads = cpu_threads()
    torch.set_num_threads(threads)
    total_s, total_b = 0.0, 0
    with ThreadPoolExecutor(max_workers=threads) as pool:
        for k, n in SHAPES.values():
            qw, qz, sc, gi = synth.gptq_linear(k, n, seed=seed)
            x = torch.from_numpy(synth.activations(1, k, "f16", seed=seed + 1)).half()
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
        s, b = cpu_layer_seconds(seed=i)
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
    if rank != 0:
        return
    for _ in range(min(args.warmup, 1)):
        cpu_layer_seconds(seed=99)
    t0 = time.perf_counter()
    nbytes = 0
    for i in range(args.steps):
        _, b = cpu_layer_seconds(seed=i)
        nbytes += b
    secs = time.perf_counter() - t0
    value = nbytes / secs / 1e9
    line = {
        "impl": "reference",
        "metric": "w4a16_m1_gemv_hbm_gbs",
        "value": round(value, 4),
        "unit": "GB/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": min(args.warmup, 1),
        "ms_per_step": round(secs * 1e3 / args.steps, 2),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "int4 weights, f16 activations, f32 accumulate",
        "data": "synthetic",
        "config": {
            "workload": "gptq_llama8b_mlp_m1: GPTQ-Int4 act-order W4A16 GEMV, Llama-3.1-8B MLP shapes, M=1; each step is ONE layer (gate, up, down) of the 32-layer stack on the host cores",
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
                    choices=["gptq_llama8b_mlp_m1", "w4a16_prefill", "fp8_gemm", "nvfp4_gemm", "moe"])
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"], help="moe workload at N > 1: who moves the tokens")
    ap.add_argument("--rows", type=int, default=0, help="rows (tokens) of the secondary workloads; 0 = the workload's default")
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
