#!/usr/bin/env python
"""Benchmark of the codebook-linear decode path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

Workload (N = 1): the Qwen2.5-7B-shaped decode GEMV set at batch 1 - 28 layers x {q 3584x3584,
k/v 512x3584, o 3584x3584, gate/up 18944x3584, down 3584x18944} = 196 matrices, each with its own
4096 x 8 fp16 codebook, 12-bit packed tags and fp16 row scales; synthetic random tags/books (seeded),
x ~ N(0,1) bf16. One step = y = W x for all 196 matrices (1.24 GB of packed weights, far larger
than L2, so every step streams from HBM). The metric is achieved HBM GB/s on the algorithmic bytes
(packed tags + codebooks + row scales + activations in/out).

With N > 1 every matrix is tensor-parallel sharded (q/k/v/gate/up by rows, o/down by columns with
an NCCL all-reduce of the partial outputs) and the same total set is processed by the N ranks
("strong" scaling).

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Qwen2.5-7B block linears: (name, R, C, kind) kind: "col" = split rows under TP, "row" = split columns
SHAPES_7B = [("q", 3584, 3584, "col"), ("k", 512, 3584, "col"), ("v", 512, 3584, "col"), ("o", 3584, 3584, "row"),
             ("gate", 18944, 3584, "col"), ("up", 18944, 3584, "col"), ("down", 3584, 18944, "row")]
LAYERS_7B = 28
METRIC = "codebook_gemv_hbm_gbs_batch1"
FALLBACK_HBM_GBS = 6650.0

# DRAM bytes per launch of the batch-1 kernel on the 18944 x 3584 shape from one ncu capture
# (profiles/gemv_l8_gate_7b.md: dram__bytes_read.sum + dram__bytes_write.sum), and the algorithmic
# bytes of that launch; traffic of other launches is scaled by their algorithmic bytes.
NCU_TRAFFIC_GATE = (12_902_912 + 0, 12_833_792 + 3584 * 2 + 18944 * 2)


def measured_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes(R: int, C: int, B: int = 1) -> int:
    W = (C // 8 * 12 + 31) // 32
    return R * W * 4 + 4096 * 8 * 2 + R * 2 + B * C * 2 + B * R * 2


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._stop_evt = index, [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown, "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown, "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.02)

    def stop(self) -> dict:
        self._stop_evt.set()
        self.join(timeout=2)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


# ----------------------------------------------------------------------------------------- reference arm
def run_reference(args, rank: int, world: int) -> None:
    """The reference's CPU execution of the path (unpack + decode + fp32 matmul in CPU torch, all host
    threads), on a bounded sample of the same workload: one matrix per distinct shape per step, scaled
    to the full set by the shape counts."""
    if rank != 0:
        return
    from oracle import cbl_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    g = torch.Generator().manual_seed(0)
    sample = []
    for name, R, C, _ in SHAPES_7B:
        if name in ("v", "o", "up"):
            continue                      # same shapes as k, q, gate
        Rs = min(R, 2048)                 # bounded sample: at most 2048 rows of each shape
        W = (C // 8 * 12 + 31) // 32
        words = torch.randint(-2**31, 2**31 - 1, (Rs, W), dtype=torch.int32, generator=g)
        table = torch.randn(4096, 8, generator=g).half()
        rs = (torch.rand(Rs, generator=g) * 0.02 + 0.01).half()
        x = torch.randn(1, C, generator=g).bfloat16()
        count = {"q": 2, "k": 2, "gate": 2, "down": 1}[name] * LAYERS_7B
        sample.append((words, table, rs, x, R, C, Rs, count))

    def step() -> float:
        """Seconds the full 196-matrix set would take, extrapolated from the sampled rows."""
        total = 0.0
        for words, table, rs, x, R, C, Rs, count in sample:
            t0 = time.perf_counter()
            orc.cpu_linear_torch(words, table, rs, x, 12, 8)
            total += (time.perf_counter() - t0) * (R / Rs) * count
        return total

    for _ in range(args.warmup):
        step()
    ts = [step() for _ in range(args.steps)]
    t = sum(ts) / len(ts)
    total_bytes = sum(algorithmic_bytes(R, C) for _, R, C, _ in SHAPES_7B) * LAYERS_7B
    val = total_bytes / t / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": "qwen2.5-7b decode GEMV set (196 codebook matrices), batch 1", "timing": "host wall clock"},
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port",
                             "sample": "<=2048 rows of one matrix per distinct shape (q, k, gate, down) per step, scaled by rows and counts"},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------- our arm
def build_set(dev, rank: int, world: int, batch: int):
    """The rank's share of the 196 matrices as PackedLinear objects (random tags generated on the device)."""
    from quantexperiments_b200.linear import PackedLinear
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    lins, kinds, total_bytes = [], [], 0
    for layer in range(LAYERS_7B):
        for name, R, C, kind in SHAPES_7B:
            r, c = R, C
            if world > 1:
                if kind == "col":
                    r = max(R // world, 1) if R % world == 0 else R       # k/v at TP 8: 512 / 8 = 64 rows
                else:
                    c = C // world
            W = (c // 8 * 12 + 31) // 32
            words = torch.randint(-2**31, 2**31 - 1, (r, W), dtype=torch.int32, device=dev, generator=g)
            table = torch.randn(4096, 8, device=dev, generator=g).half()
            rs = (torch.rand(r, device=dev, generator=g) * 0.02 + 0.01).half()
            perms = torch.arange(c, device=dev)[None]
            lin = PackedLinear(words, table, rs, None, None, perms, 4096, 8)
            lin.l8 if (batch == 1 and lin.use_l8()) else lin.small_batch(batch).xp_buffer(batch)
            lins.append(lin)
            kinds.append(kind)
            total_bytes += algorithmic_bytes(r, c, batch)
    return lins, kinds, total_bytes


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch.distributed as dist
    from quantexperiments_b200 import kernels  # noqa: F401  (fails loudly if libcbl.so is missing)
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    B = args.batch
    lins, kinds, rank_bytes = build_set(dev, rank, world, B)
    g = torch.Generator(device=dev).manual_seed(7)
    xs = {c: torch.randn(B, c, device=dev, generator=g).bfloat16() for c in {l.C for l in lins}}
    ys = {r: torch.empty(B, r, device=dev, dtype=torch.bfloat16) for r in {l.R for l in lins}}

    def launch(lin, x, y):
        if B == 1:
            lin.gemv(x[0], y[0])
        else:
            lin.small_batch(B).run(x, y, B)

    # batch 1: q|k|v and gate|up share their input and run as one grouped launch each, as the reference merges
    # them (7 matrices per layer -> 4 launches + 4 finish kernels)
    from quantexperiments_b200.kernels import L8Group
    per_layer = len(SHAPES_7B)
    groups = []
    arena = None
    if B == 1 and world > 1:
        # row-parallel products sum their partial outputs through peer memory inside the finish kernel
        from quantexperiments_b200.tp import PeerArena, PeerReduceGemv
        arena = PeerArena(8 << 20)
    # every product reads its own slice of one input arena and writes its own slice of one output arena, so that the
    # end-to-end leg moves a step's inputs and results with ONE copy each way
    n_in = sum(B * l.C for i, l in enumerate(lins) if i % per_layer in (0, 3, 4, 6))
    xarena = torch.randn(n_in, device=dev, generator=g).bfloat16()
    yarena = torch.empty(sum(B * l.R for l in lins), device=dev, dtype=torch.bfloat16)
    xoff = yoff = 0
    items = []                     # batch > 1: (lin, x [B, C], y [B, R], kind)
    for l0 in range(0, len(lins), per_layer):
        q, k, v, o, gate, up, down = lins[l0:l0 + per_layer]
        for members, kind in (((q, k, v), "col"), ((o,), "row"), ((gate, up), "col"), ((down,), "row")):
            C = members[0].C
            x = xarena[xoff:xoff + B * C].view(B, C)
            xoff += B * C
            outs = []
            for m in members:
                outs.append(yarena[yoff:yoff + B * m.R].view(B, m.R))
                yoff += B * m.R
                items.append((m, x, outs[-1], kind))
            if B == 1:
                if arena is not None and kind == "row":
                    groups.append((PeerReduceGemv(members[0].l8, arena), x[0], [outs[0][0]], "fused"))
                else:
                    groups.append((L8Group([m.l8 for m in members]), x[0], [o_[0] for o_ in outs], kind))

    def step_kernels():
        if B == 1:
            for grp, x, outs, kind in groups:
                if kind == "fused":
                    grp.run(x, outs[0])
                else:
                    grp.run(x, outs)
            return
        staged = (None, None)             # matrices that share their input share one staging pass of it
        for lin, x, y, kind in items:
            if staged[0] is not x:
                staged = (x, lin.small_batch(B).prep(x, B))
            lin.small_batch(B).run_prepped(staged[1], y, B)
            if world > 1 and kind == "row":
                dist.all_reduce(y)

    launches_per_step = 2 * len(groups) if B == 1 else len(lins) + 4 * (len(lins) // per_layer)
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        step_kernels()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()         # NCCL all-reduces are captured with the kernels
        with torch.cuda.graph(graph, stream=stream):
            step_kernels()
        run = graph.replay

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)

        for _ in range(max(args.warmup, 3)):
            run()
        barrier()
        sampler = ClockSampler(physical_gpu_index(local_rank))
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        torch.cuda.cudart().cudaProfilerStart()        # lets a profiler restrict itself to the timed region
        e0.record(stream)
        for _ in range(args.steps):
            run()
        e1.record(stream)
        barrier()
        torch.cuda.cudart().cudaProfilerStop()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop()

        # dominant kernel alone: the batch-1 table-lookup kernel over its matrices, timed with events
        roof = None
        if world == 1 and B == 1:
            big = [lin for lin in lins if lin.use_l8()]
            gk = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gk, stream=stream):
                for lin in big:
                    lin.l8.run(xs[lin.C][0], ys[lin.R][0])
            for _ in range(3):
                gk.replay()
            torch.cuda.synchronize(dev)
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record(stream)
            for _ in range(args.steps):
                gk.replay()
            k1.record(stream)
            torch.cuda.synchronize(dev)
            per_launch_s = k0.elapsed_time(k1) * 1e-3 / (args.steps * len(big))
            alg = sum(algorithmic_bytes(lin.R, lin.C) for lin in big) / len(big)
            peak, src = measured_peak()
            achieved = alg / per_launch_s / 1e9
            roof = {"bound": "hbm", "kernel": "k_gemv_l8", "achieved": achieved, "peak": peak, "peak_source": src, "unit": "GB/s",
                    "frac": achieved / peak, "frac_of_nominal_8000": achieved / 8000.0,
                    "traffic": alg * NCU_TRAFFIC_GATE[0] / NCU_TRAFFIC_GATE[1], "algorithmic_bytes_per_launch": alg,
                    "us_per_launch": per_launch_s * 1e6, "launches_timed": args.steps * len(big)}

        # end to end with HOST buffers: the step's inputs come from pinned host memory (one copy into the input arena),
        # the products run, the step's results go back to pinned host memory (one copy of the output arena); copies and
        # kernels of a step form one CUDA graph and the host waits for every step's results
        hx = torch.randn(xarena.numel()).bfloat16().pin_memory()
        hy = torch.empty(yarena.numel(), dtype=torch.bfloat16).pin_memory()
        h2d, d2h = xarena.numel() * 2, yarena.numel() * 2

        def e2e_body():
            xarena.copy_(hx, non_blocking=True)
            step_kernels()
            hy.copy_(yarena, non_blocking=True)

        e2e_body()
        stream.synchronize()
        ge = torch.cuda.CUDAGraph()
        with torch.cuda.graph(ge, stream=stream):
            e2e_body()

        def step_e2e():
            ge.replay()
            stream.synchronize()

        for _ in range(2):
            step_e2e()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(args.steps):
            step_e2e()
        t1.record(stream)
        barrier()
        ms_e2e = t0.elapsed_time(t1)

    # max over ranks, whole-job bytes
    tv = torch.tensor([ms, ms_e2e, float(rank_bytes)], device=dev, dtype=torch.float64)
    if world > 1:
        tmax = tv.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        tsum = tv.clone()
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms, ms_e2e, total_bytes = float(tmax[0]), float(tmax[1]), float(tsum[2])
    else:
        total_bytes = float(rank_bytes)
    if rank != 0:
        return
    value = total_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e = total_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    line = {"metric": METRIC if B == 1 else f"codebook_gemv_hbm_gbs_batch{B}", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"qwen2.5-7b decode GEMV set (196 codebook matrices, d=8, K=4096, 12-bit tags), batch {B}",
                       "parallelism": f"tp{world}" if world > 1 else "single", "l2": "inputs larger than L2 (1.24 GB of packed weights per step)",
                       "accumulate": "fp32", "activations": "bf16", "launch": "one CUDA graph per step (q|k|v and gate|up grouped)" + ("" if world == 1 else "; o/down summed over ranks through peer memory in the finish kernel"),
                       "e2e": "a step's inputs from pinned host memory and its results back to pinned host memory (one copy each way), copies and kernels in one CUDA graph, host synchronises every step"},
            "clocks": clocks, "gpu_launches": launches_per_step * args.steps * world,
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                    "ms_per_step": ms_e2e / args.steps}}
    if roof is not None:
        line["roofline"] = roof
    if world == 1:
        line["cpu_baseline"] = cpu_baseline_sample()
    print(json.dumps(line), flush=True)


def run_prefill(args, rank: int, world: int, local_rank: int) -> None:
    """Prefill product of the same 196-matrix set: Y = X W^T for --tokens tokens per matrix on the tcgen05
    kernel; metric TFLOPS = 2 * tokens * R * C summed over the matrices / time."""
    import torch.distributed as dist
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    T = args.tokens
    from quantexperiments_b200.kernels import DenseStack
    from quantexperiments_b200.linear import DENSE_MIN_TOKENS
    lins, kinds, _ = build_set(dev, rank, world, 64)
    g = torch.Generator(device=dev).manual_seed(7)
    xs = {c: torch.randn(T, c, device=dev, generator=g).bfloat16() for c in {l.C for l in lins}}
    flops = sum(2.0 * T * l.R * l.C for l in lins)
    # q|k|v and gate|up share their activations: one stacked product each, as the reference's gemm(x, [pieces]) does.
    # From DENSE_MIN_TOKENS tokens on the stack is decoded once into a 16-bit scratch and multiplied by the TMA-fed
    # tcgen05 GEMM; below, every piece runs the kernel that decodes weight tiles on the fly.
    dense = T >= (args.dense_min if args.dense_min is not None else DENSE_MIN_TOKENS)
    groups, launches = [], 0
    for l0 in range(0, len(lins), len(SHAPES_7B)):
        q, k, v, o, gate, up, down = lins[l0:l0 + len(SHAPES_7B)]
        for members, kind in (((q, k, v), "col"), ((o,), "row"), ((gate, up), "col"), ((down,), "row")):
            y = torch.empty(T, sum(m.R for m in members), device=dev, dtype=torch.bfloat16)
            groups.append((DenseStack([m.dm for m in members]) if dense else None, members, xs[members[0].C], y, kind))
            launches += (len(members) + 2) if dense else 2 * len(members)

    def run_group(stack, members, x, y, kind):
        if stack is not None:
            stack.gemm(x, y)
        else:
            off = 0
            for m in members:
                m.l8.gemm(x, y[:, off:off + m.R])
                off += m.R
        if world > 1 and kind == "row":
            dist.all_reduce(y)

    def step():
        for grp in groups:
            run_group(*grp)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step()
        barrier()
        sampler = ClockSampler(physical_gpu_index(local_rank))
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        # end to end: the layer inputs come from pinned host memory, the last token's outputs go back
        hx = {c: torch.randn(T, c).bfloat16().pin_memory() for c in xs}
        hyo = [torch.empty(grp[3].shape[1], dtype=torch.bfloat16).pin_memory() for grp in groups[:4]]

        def step_e2e():
            for gi, grp in enumerate(groups):
                grp[2].copy_(hx[grp[2].shape[1]], non_blocking=True)      # every stack's activations come from the host
                run_group(*grp)
                hyo[gi % 4].copy_(grp[3][T - 1], non_blocking=True)
            stream.synchronize()

        step_e2e()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record(stream)
        for _ in range(max(args.steps // 4, 1)):
            step_e2e()
        t1.record(stream)
        barrier()
        ms_e2e = t0.elapsed_time(t1) / max(args.steps // 4, 1)
    tv = torch.tensor([ms, ms_e2e, flops], device=dev, dtype=torch.float64)
    if world > 1:
        tmax, tsum = tv.clone(), tv.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        ms, ms_e2e, flops = float(tmax[0]), float(tmax[1]), float(tsum[2])
    if rank != 0:
        return
    peaks = {}
    try:
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    except Exception:
        pass
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    value = flops * args.steps / (ms * 1e-3) / 1e12
    line = {"metric": "prefill_dequant_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"qwen2.5-7b prefill dequant-GEMM set (196 codebook matrices), {T} tokens", "accumulate": "fp32",
                       "path": "decode once into a 16-bit scratch + TMA-fed tcgen05 GEMM (q|k|v and gate|up stacked)" if dense
                               else "weight tiles decoded on the fly inside the tcgen05 GEMM",
                       "activations": "bf16 in, fp16 on the tensor cores with a power-of-two scale per token", "output": "bf16",
                       "parallelism": f"tp{world}" if world > 1 else "single", "l2": "inputs larger than L2 per step"},
            "clocks": clocks, "gpu_launches": launches * args.steps * world,
            "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": sum(T * grp[2].shape[1] * 2 for grp in groups) * world,
                    "d2h_bytes_per_step": sum(grp[3].shape[1] * 2 for grp in groups) * world, "ms_per_step": ms_e2e},
            "roofline": {"bound": "tensor", "kernel": "k_gemm_dense_2sm" if dense else "k_gemm_l8", "achieved": value / world, "peak": peak,
                         "peak_source": "measured (sustained)" if peaks else "fallback", "unit": "TFLOP/s", "frac": value / world / peak,
                         "frac_of_burst": value / world / float(peaks.get("bf16_tflops", 1590.0)), "traffic": None}}
    print(json.dumps(line), flush=True)


def run_decode(args, rank: int, world: int, local_rank: int) -> None:
    """End-to-end decode of a random-init Qwen2.5-7B architecture with every block linear in the packed format:
    prompt of --tokens random ids (batched prefill), then --steps generated tokens per sequence by CUDA-graph replay
    of the decode step, --batch sequences at once. Metric: generated tokens/s. N > 1: independent replicas (the
    engine is a single-GPU program), value = sum over ranks."""
    import torch.distributed as dist
    from quantexperiments_b200.engine import Cfg, Qwen2BatchEngine, generate, random_engine
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    B, T, K = args.batch, args.tokens, args.steps
    cfg = Cfg(max_len=(T + 2 * K + 64 + 31) // 32 * 32)
    eng = random_engine(cfg, seed=rank, dev=dev, head=args.head, embed=args.embed)
    run_eng = eng if B == 1 else Qwen2BatchEngine(eng, B)
    gcpu = torch.Generator().manual_seed(5 + rank)
    prompts = [torch.randint(0, cfg.vocab, (T,), generator=gcpu) for _ in range(B)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    run_eng.capture()
    run_eng.reset(0)
    for b in range(B):
        run_eng.prefill(prompts[b].to(dev), b)
    for _ in range(max(args.warmup, 3)):
        run_eng.graph.replay()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(K):
        run_eng.graph.replay()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    run_eng.check()
    # end to end through generate(): host prompt in, every token read back by the host (batch 1 engine)
    t0 = time.perf_counter()
    out = generate(eng, prompts[0].tolist(), K, graph=True)
    torch.cuda.synchronize(dev)
    s_e2e = time.perf_counter() - t0
    assert len(out) == K
    tv = torch.tensor([ms, s_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tv, op=dist.ReduceOp.MAX)
    ms, s_e2e = float(tv[0]), float(tv[1])
    if rank != 0:
        return
    peak, src = measured_peak()
    kv_bytes = 2 * cfg.layers * cfg.n_kv * cfg.head_dim * 2 * (T + K // 2) * B
    step_bytes = eng.weight_bytes() + kv_bytes
    achieved = step_bytes / (ms / K * 1e-3) / 1e9
    launches = (10 * cfg.layers + 4) if B == 1 else (22 * cfg.layers + 5)
    line = {"metric": "decode_tok_s", "value": B * K * world / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"qwen2.5-7b architecture, random init, every block linear packed (d=8, K=4096, 12-bit tags); prompt {T}, "
                                   f"generate {K}, batch {B}; "
                                   + ("bf16" if args.embed == "16" else "4-bit block-32") + " embedding, " + ("bf16" if args.head == "16" else "8-bit block-32")
                                   + " head, bf16 KV cache",
                       "parallelism": "replicas" if world > 1 else "single", "launch": "one CUDA graph per decode step",
                       "l2": "inputs larger than L2 (2.3 GB of weights per step)"},
            "clocks": clocks, "gpu_launches": launches * K * world,
            "e2e": {"value": K * world / s_e2e, "unit": "tok/s", "h2d_bytes_per_step": T * 8 // K, "d2h_bytes_per_step": 8,
                    "note": f"generate() at batch 1: prompt upload + prefill of {T} tokens + {K} steps with a host read per token"},
            "roofline": {"bound": "hbm", "kernel": "decode step (all kernels)", "achieved": achieved, "peak": peak, "peak_source": src,
                         "unit": "GB/s", "frac": achieved / peak, "traffic": None, "algorithmic_bytes_per_step": step_bytes}}
    print(json.dumps(line), flush=True)


def run_snap(args, rank: int, world: int, local_rank: int) -> None:
    """Encoder side: snap one 18944 x 3584 matrix (8,486,912 chunks, the 7B gate shape) against a 4096-word book and pack
    the 12-bit tags. A step = assign + pack_bits of the whole matrix. Metric: million chunks per second. The kernel is
    bound by fp32 FMAs (16 flop per chunk and codeword), so the roofline is the fp32 rate, not HBM. N > 1: replicas."""
    import torch.distributed as dist
    from quantexperiments_b200 import codebook as cb
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    R, C, K = 18944, 3584, 4096
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    x = torch.randn(R * C // 8, 8, device=dev, generator=g)
    book = torch.randn(K, 8, device=dev, generator=g).half()
    n = x.shape[0]

    def step():
        idx, err = cb.assign(x, book)
        return cb.pack_bits(idx.view(R, C // 8), 12), err

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        words, err = step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop()
    # end to end: fp32 chunks from pinned host memory in, packed tags out to the host
    hx = x.cpu().pin_memory()
    hw = torch.empty(words.shape, dtype=torch.int32).pin_memory()
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    for _ in range(3):
        x.copy_(hx, non_blocking=True)
        words, err = step()
        hw.copy_(words, non_blocking=True)
        torch.cuda.synchronize(dev)
    s_e2e = (time.perf_counter() - t0) / 3
    tv = torch.tensor([ms, s_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tv, op=dist.ReduceOp.MAX)
    ms, s_e2e = float(tv[0]), float(tv[1])
    if rank != 0:
        return
    # the reference's CPU path (torch addmm + min in batches of 65,536, shapequant/codebook.py:58-71) on a bounded sample
    from oracle import cbl_oracle as orc
    ns = 1 << 20
    xs, bk = x[:ns].cpu().numpy(), book.cpu().numpy()
    t0 = time.perf_counter()
    for s0 in range(0, ns, 65536):
        orc.assign(xs[s0:s0 + 65536], bk)
    cpu_s = time.perf_counter() - t0
    flops = n * K * 16.0
    sm_clock = (clocks.get("sm_mhz") or 1900) * 1e6
    peak = 148 * 128 * 2 * sm_clock / 1e12
    line = {"metric": "snap_mchunks_s", "value": n * world / (ms * 1e-3) / 1e6, "unit": "Mchunks/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": f"snap of one {R} x {C} matrix: {n} chunks of 8 against a {K}-word fp16 book (exact fp32 argmin) + 12-bit packing",
                       "parallelism": "replicas" if world > 1 else "single", "l2": "inputs larger than L2 (272 MB of chunks per step)"},
            "clocks": clocks, "gpu_launches": 2 * args.steps * world,
            "e2e": {"value": n * world / s_e2e / 1e6, "unit": "Mchunks/s", "h2d_bytes_per_step": n * 32, "d2h_bytes_per_step": int(hw.numel()) * 4},
            "roofline": {"bound": "fp32", "kernel": "k_assign<8,false>", "achieved": flops / (ms * 1e-3) / 1e12, "peak": peak,
                         "peak_source": "148 SMs x 128 FMA x 2 x the SM clock sampled during the run", "unit": "TFLOP/s",
                         "frac": flops / (ms * 1e-3) / 1e12 / peak, "traffic": None},
            "cpu_baseline": {"value": ns / cpu_s / 1e6, "unit": "Mchunks/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": f"{ns} chunks through the oracle's assign (torch addmm + min, batches of 65,536)"}}
    print(json.dumps(line), flush=True)


def run_load(args, rank: int, world: int, local_rank: int) -> None:
    """Packed file -> device: writes a synthetic packed file of --tokens/512 7B layers (default 4 layers = 28 matrices,
    177 MB) to a temporary directory, then times load_linears (streamed copies + in-place kernel layouts, l8 and x16).
    A step = one full load. Metric: file GB per second. N > 1: every rank loads its own shard (tensor parallel kinds)."""
    import tempfile
    import torch.distributed as dist
    from quantexperiments_b200 import loader, packed
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    layers = max(1, args.tokens // 512)
    kinds = {}
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, f"m{rank}.safetensors")
        g = torch.Generator().manual_seed(1)
        mats = {}
        for li in range(layers):
            for name, r, c, kind in SHAPES_7B:
                W = (c // 8 * 12 + 31) // 32
                t = {"tags": torch.randint(-2**31, 2**31 - 1, (r, W), dtype=torch.int32, generator=g), "table": torch.randn(4096, 8, generator=g).half(),
                     "row_scale": (torch.rand(r, generator=g) * 0.02 + 0.01).half()}
                crc = packed.perm_crc(packed.seeded_perms(c, 1, torch.Generator(device="cpu").manual_seed(0)))
                meta = {"R": r, "C": c, "d": 8, "K": 4096, "G": 1, "M": 1, "seed": 0, "perm_crc": crc, "bits": r * W * 32}
                mats[f"l{li}.{name}"] = (t, meta)
                kinds[f"l{li}.{name}"] = kind
        packed.save(path, mats, base_model="synthetic/7b-shapes")
        del mats
        nbytes = os.path.getsize(path)

        def step():
            lins = loader.load_linears(path, device=dev, layouts=("l8", "x16"), rank=rank, world=world, kinds=kinds)
            return lins.stats

        for _ in range(2):
            step()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            stats = step()
        torch.cuda.synchronize(dev)
        s = (time.perf_counter() - t0) / args.steps
        # the reference's way: one tensor at a time (PackedLinear.from_packed), layouts built after each copy
        from quantexperiments_b200.linear import PackedLinear
        pf = packed.PackedFile(path)
        t0 = time.perf_counter()
        for name in list(pf.meta)[:7]:
            lin = PackedLinear.from_packed(pf, name, device=dev)
            lin.l8, lin.x16
        torch.cuda.synchronize(dev)
        s_one = (time.perf_counter() - t0) * len(pf.meta) / 7
    tv = torch.tensor([s], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tv, op=dist.ReduceOp.MAX)
    s = float(tv[0])
    if rank != 0:
        return
    line = {"metric": "packed_load_gbs", "value": nbytes / s / 1e9, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": 2,
            "ms_per_step": s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": f"load of a packed file with {layers} layers of Qwen2.5-7B shapes ({nbytes} bytes, page cache warm) into one arena "
                                   f"with the l8 and x16 kernel layouts", "parallelism": f"tp{world}" if world > 1 else "single",
                       "timing": "host wall clock around load_linears (the path is host-driven: file read, pinned copy, H2D, repack kernels)"},
            "gpu_launches": 3 * len(kinds) * args.steps, "arena_bytes": stats["arena_bytes"], "h2d_bytes_per_step": stats["h2d_bytes"],
            "tensor_by_tensor_ms": s_one * 1e3}
    print(json.dumps(line), flush=True)


def cpu_baseline_sample() -> dict:
    """The reference's CPU path (oracle port) timed on this host's cores on a bounded sample."""
    from oracle import cbl_oracle as orc
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(0)
    t_total = 0.0
    for name, R, C, count in (("q", 3584, 3584, 2), ("k", 512, 3584, 2), ("gate", 18944, 3584, 2), ("down", 3584, 18944, 1)):
        Rs = min(R, 1024)
        W = (C // 8 * 12 + 31) // 32
        words = torch.randint(-2**31, 2**31 - 1, (Rs, W), dtype=torch.int32, generator=g)
        table = torch.randn(4096, 8, generator=g).half()
        rs = (torch.rand(Rs, generator=g) * 0.02 + 0.01).half()
        x = torch.randn(1, C, generator=g).bfloat16()
        orc.cpu_linear_torch(words[:64], table, rs[:64], x, 12, 8)
        t0 = time.perf_counter()
        orc.cpu_linear_torch(words, table, rs, x, 12, 8)
        t_total += (time.perf_counter() - t0) * (R / Rs) * count * LAYERS_7B
    total_bytes = sum(algorithmic_bytes(R, C) for _, R, C, _ in SHAPES_7B) * LAYERS_7B
    return {"value": total_bytes / t_total / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "1024 rows of one matrix per distinct shape (q, k, gate, down), scaled by rows and counts to the 196-matrix set"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--workload", default="gemv", choices=["gemv", "prefill", "decode", "snap", "load"],
                    help="gemv: decode products (the headline metric); prefill: the same 196 matrices against --tokens tokens; "
                         "decode: end-to-end generation (prompt --tokens, --steps generated tokens, --batch sequences)")
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--head", default="16", choices=["16", "q8"], help="decode workload: output head in bf16 (the named config) or the reference's 8-bit block-32 format")
    ap.add_argument("--embed", default="16", choices=["16", "q4"], help="decode workload: embedding in bf16 or the reference's 4-bit block-32 format")
    ap.add_argument("--dense-min", type=int, default=None, help="prefill: token count from which the two-phase path runs (default: the library's)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        if args.workload == "prefill":
            run_prefill(args, rank, world, local_rank)
        elif args.workload == "decode":
            run_decode(args, rank, world, local_rank)
        elif args.workload == "snap":
            run_snap(args, rank, world, local_rank)
        elif args.workload == "load":
            run_load(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
