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

# block linears: (name, R, C, kind) kind: "col" = split rows under TP, "row" = split columns
SHAPES_7B = [("q", 3584, 3584, "col"), ("k", 512, 3584, "col"), ("v", 512, 3584, "col"), ("o", 3584, 3584, "row"),
             ("gate", 18944, 3584, "col"), ("up", 18944, 3584, "col"), ("down", 3584, 18944, "row")]
SHAPES_32B = [("q", 5120, 5120, "col"), ("k", 1024, 5120, "col"), ("v", 1024, 5120, "col"), ("o", 5120, 5120, "row"),
              ("gate", 27648, 5120, "col"), ("up", 27648, 5120, "col"), ("down", 5120, 27648, "row")]
# "7b": BASELINE configs[1] (one book, one column order); "32b": configs[4] (two summed books, 16 seeded column orders)
MODELS = {"7b": {"shapes": SHAPES_7B, "layers": 28, "books": 1, "M": 1, "label": "qwen2.5-7b"},
          "32b": {"shapes": SHAPES_32B, "layers": 64, "books": 2, "M": 16, "label": "qwen2.5-32b"}}
LAYERS_7B = 28
METRIC = "codebook_gemv_hbm_gbs_batch1"
FALLBACK_HBM_GBS = 6650.0

# DRAM bytes per launch of the batch-1 kernel on the 18944 x 3584 gate|up pair from one ncu capture
# (profiles/gemv_l8_gateup_7b.md: dram__bytes_read.sum + dram__bytes_write.sum), and the algorithmic
# bytes of that launch; traffic of other launches is scaled by their algorithmic bytes.
NCU_TRAFFIC_GATEUP = (25_732_608 + 0, 2 * (12_833_792 + 18944 * 2) + 3584 * 2)


def measured_peak() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def algorithmic_bytes(R: int, C: int, B: int = 1, books: int = 1, M: int = 1) -> int:
    """Packed tags + books + row scales (+ the rows' column-order ids) + activations in and out."""
    W = (C // 8 * 12 + 31) // 32
    return books * (R * W * 4 + 4096 * 8 * 2) + R * 2 + (R if M > 1 else 0) + B * C * 2 + B * R * 2


def set_bytes(model: str, B: int = 1) -> int:
    m = MODELS[model]
    return sum(algorithmic_bytes(R, C, B, m["books"], m["M"]) for _, R, C, _ in m["shapes"]) * m["layers"]


def workload_name(model: str, B: int) -> str:
    m = MODELS[model]
    n = len(m["shapes"]) * m["layers"]
    extra = "" if m["books"] == 1 else f", {m['books']} summed books, {m['M']} seeded column orders"
    return f"{m['label']} decode GEMV set ({n} codebook matrices, d=8, K=4096, 12-bit tags{extra}), batch {B}"


def make_matrix(model: str, layer: int, name: str, R: int, C: int, device="cpu"):
    """One synthetic matrix of the set in the file layout, seeded by (model, layer, name): uniform random tags, an
    N(0,1) fp16 book, row scales distributed like the RMS of N(0, 0.02) rows.  Generated on the CPU it is the same
    tensor in both arms of the bench (the GPU arm copies it to the device); returns (tensors, meta, perms)."""
    import zlib
    from quantexperiments_b200 import packed
    m = MODELS[model]
    seed = zlib.crc32(f"{model}/{layer}/{name}".encode())
    g = torch.Generator(device=device).manual_seed(seed)
    W = (C // 8 * 12 + 31) // 32
    t = {"tags": torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device=device, generator=g),
         "table": torch.randn(4096, 8, device=device, generator=g).half(),
         "row_scale": (0.02 * (1.0 + torch.randn(R, device=device, generator=g) / (2.0 * C) ** 0.5)).half()}
    if m["books"] == 2:
        t["tags2"] = torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device=device, generator=g)
        t["table2"] = torch.randn(4096, 8, device=device, generator=g).half()
    perms = None
    if m["M"] > 1:
        t["row_mask"] = torch.randint(0, m["M"], (R,), device=device, generator=g).to(torch.uint8)
        perms = packed.seeded_perms(C, m["M"], torch.Generator(device="cpu").manual_seed(seed & 0x7FFFFFFF))
    meta = {"R": R, "C": C, "d": 8, "K": 4096, "G": 1, "M": m["M"]}
    return t, meta, perms


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
def reference_cpu_linear():
    """(fn, kind): the reference's CPU execution of one product - unpack_bits + decode_tensors + fp32 matmul.
    The reference's own modules when they have been staged under oracle/_ref (kind "reference"), else the oracle's
    restatement of them (kind "port")."""
    try:
        from oracle import make_ref
        if make_ref.load() is not None:
            import shapequant.packed as rp

            def fn(words, table, row_scale, x):
                nch = x.shape[-1] // 8
                tags = rp.unpack_bits(words, 12, nch)
                perms = torch.arange(x.shape[-1])[None]
                w = rp.decode_tensors(tags, table, row_scale, torch.zeros(words.shape[0], dtype=torch.int64), None, perms, 4096)
                return x.float() @ w.t()
            return fn, "reference"
    except Exception:
        pass
    from oracle import cbl_oracle as orc
    return (lambda words, table, row_scale, x: orc.cpu_linear_torch(words, table, row_scale, x, 12, 8)), "port"


def reference_sample(model: str = "7b"):
    """The bounded sample of the set that the CPU legs time: layer 0's q and k whole (v, o have their shapes), the
    first 2048 rows of its gate (= up) and of its down - the very tensors the GPU arm multiplies."""
    out = []
    counts = {"q": 2, "k": 2, "gate": 2, "down": 1}
    for name, R, C, _ in MODELS[model]["shapes"]:
        if name not in counts:
            continue
        t, _, _ = make_matrix(model, 0, name, R, C)
        Rs = min(R, 2048)
        x = torch.randn(1, C, generator=torch.Generator().manual_seed(C)).bfloat16()
        out.append((t["tags"][:Rs], t["table"], t["row_scale"][:Rs], x, R, Rs, counts[name] * MODELS[model]["layers"]))
    return out


def time_reference_step(fn, sample) -> float:
    """Seconds the whole set would take on this host: the sample's products timed, scaled by rows and shape counts."""
    total = 0.0
    for words, table, rs, x, R, Rs, count in sample:
        t0 = time.perf_counter()
        fn(words, table, rs, x)
        total += (time.perf_counter() - t0) * (R / Rs) * count
    return total


SAMPLE_TEXT = "layer 0's q and k matrices whole and 2048 rows each of its gate and down matrices (the tensors the GPU arm uses), scaled by rows and shape counts to the 196-matrix set"


def run_reference(args, rank: int, world: int) -> None:
    """The reference's CPU execution of the path (unpack + decode + fp32 matmul in CPU torch, all host threads), on a
    bounded sample of the same workload and the same tensors as the GPU arm."""
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    fn, kind = reference_cpu_linear()
    sample = reference_sample("7b")
    for _ in range(max(args.warmup, 1)):
        time_reference_step(fn, sample)
    ts = [time_reference_step(fn, sample) for _ in range(args.steps)]
    t = sum(ts) / len(ts)
    val = set_bytes("7b") / t / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name("7b", 1), "timing": "host wall clock; ms_per_step is the full set's time extrapolated from the sample"},
            "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": kind, "sample": SAMPLE_TEXT},
            "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def cpu_baseline_sample() -> dict:
    """The reference's CPU path timed on this host's cores on the bounded sample (one pass after a warm-up pass)."""
    torch.set_num_threads(os.cpu_count() or 1)
    fn, kind = reference_cpu_linear()
    sample = reference_sample("7b")
    time_reference_step(fn, [(w[:64], t, r[:64], x, R, Rs, c) for w, t, r, x, R, Rs, c in sample])
    t = time_reference_step(fn, sample)
    return {"value": set_bytes("7b") / t / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": kind, "sample": SAMPLE_TEXT}


def gpu_reference(dev, stream, lins_shapes, steps: int) -> dict:
    """The reference's own GPU kernel for this format - the Triton PackedLinear.gemv of shapequant/kernels/gemv.py -
    over the same 196 matrices on the same device (the GPU-versus-GPU comparison).  Needs the staged reference and Triton."""
    try:
        from oracle import make_ref
        if make_ref.load() is None:
            return {"unavailable": "oracle/_ref has not been staged (python oracle/make_ref.py)"}
        import shapequant.kernels.gemv as rg
    except Exception as e:                                    # Triton missing or not importable on this box
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    try:
        mods, xs, ys = [], {}, {}
        for (t, meta, perms) in lins_shapes:
            C = meta["C"]
            p = torch.arange(C, device=dev)[None]
            mods.append(rg.PackedLinear(t["tags"], t["table"], t["row_scale"], None, None, p, 4096, 8))
            xs.setdefault(C, torch.randn(C, device=dev).bfloat16())
            ys.setdefault(meta["R"], torch.empty(meta["R"], device=dev, dtype=torch.bfloat16))
        with torch.cuda.stream(stream):
            for m in mods[:7]:
                m.gemv(xs[m.C], ys[m.R])                        # compiles the kernel
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for m in mods:
                    m.gemv(xs[m.C], ys[m.R])
            for _ in range(3):
                g.replay()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                g.replay()
            e1.record(stream)
            stream.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"kernel": "shapequant.kernels.gemv._gemv_kernel (Triton, unmodified)", "ms_per_step": ms,
                "value": set_bytes("7b") / (ms * 1e-3) / 1e9, "unit": "GB/s", "launches_per_step": len(mods)}
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {e}"[:300]}


# ----------------------------------------------------------------------------------------- our arm
def build_set(dev, rank: int, world: int, batch: int, model: str = "7b", layers: int | None = None, keep_file_layout: bool = False):
    """The rank's tensor-parallel share of the model's matrices as PackedLinear objects: every rank derives its shard
    from the same seeded full matrix (rows for q/k/v/gate/up, chunk ranges of the input for o/down; with column
    orders the o/down shards keep global column indices and read the full activation vector)."""
    from quantexperiments_b200 import tp
    from quantexperiments_b200.linear import PackedLinear
    m = MODELS[model]
    gen_dev = "cpu" if model == "7b" else dev            # the 7B set is shared with the CPU arm; 12 GB of 32B tags are drawn on the GPU
    lins, kinds, raw = [], [], []
    for layer in range(m["layers"] if layers is None else layers):
        for name, R, C, kind in m["shapes"]:
            t, meta, perms = make_matrix(model, layer, name, R, C, gen_dev)
            if world > 1:
                if kind == "col":
                    r0, r1 = tp.row_range(R, rank, world)
                    t, meta = tp.shard_rows(t, meta, r0, r1)
                else:
                    c0, c1 = tp.col_range(C, 8, rank, world)
                    t, meta, perms = tp.shard_cols(t, meta, c0, c1, perms)
            t = {k: v.to(dev) for k, v in t.items()}
            p = perms.to(dev) if perms is not None else torch.arange(meta["C"], device=dev)[None]
            wide = world > 1 and kind == "row" and m["M"] > 1         # the shard's column orders name positions of the full vector
            lin = PackedLinear(t["tags"], t["table"], t["row_scale"], None, t.get("row_mask"), p, 4096, 8,
                               words2=t.get("tags2"), table2=t.get("table2"), x_cols=C if wide else None)
            lin.kind = kind
            if batch == 1 and (lin.dm.M == 1 or lin.use_l8()):
                lin.l8
            else:
                lin.small_batch(batch).xp_buffer(batch)
            lins.append(lin)
            kinds.append(kind)
            if keep_file_layout:
                raw.append((t, meta, perms))
    return lins, kinds, raw


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import torch.distributed as dist
    from quantexperiments_b200 import kernels  # noqa: F401  (fails loudly if libcbl.so is missing)
    from quantexperiments_b200.kernels import L8Group
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    B, model = args.batch, args.model
    mdl = MODELS[model]
    shapes = mdl["shapes"]
    want_gpu_ref = world == 1 and B == 1 and model == "7b" and not args.no_extras
    lins, kinds, raw = build_set(dev, rank, world, B, model, keep_file_layout=want_gpu_ref)
    g = torch.Generator(device=dev).manual_seed(7)
    per_layer = len(shapes)
    C_full = {name: C for name, _, C, _ in shapes}
    groups = []
    arena = None
    if B == 1 and world > 1:
        # row-parallel products sum their partial outputs through peer memory inside the finish kernel
        from quantexperiments_b200.tp import PeerArena, PeerReduceGemv
        need = sum(kernels.lib.cbl_gemv_l8_ar_workspace_bytes(l.R) + 512 for l in lins if l.kind == "row")
        arena = PeerArena(need + (1 << 20))
    # every product reads its own slice of one input arena and writes its own slice of one output arena, so that the
    # end-to-end leg moves a step's inputs and results with ONE copy each way
    def in_cols(lin, name):
        return C_full[name] if lin.wide else lin.C
    n_in = sum(B * in_cols(l, shapes[i % per_layer][0]) for i, l in enumerate(lins) if i % per_layer in (0, 3, 4, 6))
    xarena = torch.randn(n_in, device=dev, generator=g).bfloat16()
    yarena = torch.empty(sum(B * l.R for l in lins), device=dev, dtype=torch.bfloat16)
    xoff = yoff = 0
    items = []                     # batch > 1: (lin, x [B, C], y [B, R], kind)
    for l0 in range(0, len(lins), per_layer):
        q, k, v, o, gate, up, down = lins[l0:l0 + per_layer]
        for members, kind, nm in (((q, k, v), "col", "q"), ((o,), "row", "o"), ((gate, up), "col", "gate"), ((down,), "row", "down")):
            C = in_cols(members[0], nm)
            x = xarena[xoff:xoff + B * C].view(B, C)
            xoff += B * C
            outs = []
            for mm in members:
                outs.append(yarena[yoff:yoff + B * mm.R].view(B, mm.R))
                yoff += B * mm.R
                items.append((mm, x, outs[-1], kind))
            if B == 1:
                # one token: the table-lookup kernel, unless the matrices have so many column orders for their rows that
                # per-order tables do not pay (PackedLinear.use_l8); those run on the row-tile kernel
                tables = all(mm.dm.M == 1 or mm.use_l8() for mm in members)
                if arena is not None and kind == "row" and tables:
                    groups.append((PeerReduceGemv(members[0].l8, arena), x[0], [outs[0][0]], "fused", members))
                elif tables:
                    groups.append((L8Group([mm.l8 for mm in members]), x[0], [o_[0] for o_ in outs], kind, members))
                else:
                    groups.append((None, x, outs, "t16", members))

    def step_kernels():
        if B == 1:
            for grp, x, outs, kind, members in groups:
                if kind == "fused":
                    grp.run(x, outs[0])
                elif kind == "t16":
                    for mm, y in zip(members, outs):
                        mm.t16.run(x, y, 1, wide=mm.wide)
                        if world > 1 and mm.kind == "row":
                            dist.all_reduce(y)
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

    launches_per_step = (sum(2 * len(grp[4]) if grp[3] == "t16" else (2 if grp[3] == "fused" else 1) for grp in groups) if B == 1
                         else len(lins) + 4 * (len(lins) // per_layer))
    stream = torch.cuda.Stream(device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    with torch.cuda.stream(stream):
        barrier()                              # every rank's shards and peer work spaces exist before the first launch
        step_kernels()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()         # NCCL all-reduces are captured with the kernels
        with torch.cuda.graph(graph, stream=stream):
            step_kernels()
        run = graph.replay

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

        # tensor-parallel runs: every fused peer sum reported no expired wait, every rank holds the same output, and
        # that output equals the sum of the ranks' separately computed partial products
        tp_check = None
        if world > 1 and B == 1:
            status_ok, worst, same = True, 0.0, True
            for grp, x, outs, kind, members in groups:
                if kind == "fused":
                    status_ok = status_ok and grp.status()
            for grp, x, outs, kind, members in groups[:4]:            # layer 0: the o and the down product
                if kind != "fused":
                    continue
                lin = members[0]
                part = lin.l8.run(x, torch.empty(lin.R, device=dev, dtype=torch.float32), wide=lin.wide)
                parts = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(parts, part)
                ref = parts[0].clone()
                for p in parts[1:]:
                    ref += p
                fused = outs[0].float()
                worst = max(worst, float((fused - ref).abs().max() / ref.abs().max()))
                ys_all = [torch.empty_like(outs[0]) for _ in range(world)]
                dist.all_gather(ys_all, outs[0].contiguous())
                same = same and all(torch.equal(ys_all[0], t) for t in ys_all[1:])
            flags = torch.tensor([float(status_ok), float(same), worst], device=dev, dtype=torch.float64)
            mn, mx = flags.clone(), flags.clone()
            dist.all_reduce(mn, op=dist.ReduceOp.MIN)
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            tp_check = {"status_ok": bool(mn[0] > 0), "ranks_bit_identical": bool(mn[1] > 0), "max_rel_err": float(mx[2]),
                        "tolerance": 2.0 ** -7, "checked": "layer 0's o and down products: fused peer sum vs the rank-ordered sum of all ranks' partial products"}
            tp_check["ok"] = tp_check["status_ok"] and tp_check["ranks_bit_identical"] and tp_check["max_rel_err"] < tp_check["tolerance"]

        # dominant kernel alone: the batch-1 table-lookup kernel over the set's grouped launches, timed with events
        roof = None
        if world == 1 and B == 1:
            k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k0.record(stream)
            for _ in range(args.steps):
                run()
            k1.record(stream)
            torch.cuda.synchronize(dev)
            per_launch_s = k0.elapsed_time(k1) * 1e-3 / (args.steps * len(groups))
            alg = set_bytes(model) / len(groups)
            peak, src = measured_peak()
            achieved = alg / per_launch_s / 1e9
            roof = {"bound": "hbm", "kernel": "k_gemv_l8" if all(grp[3] != "t16" for grp in groups) else "k_gemv_l8 / k_gemv_t16 (per shape)", "achieved": achieved, "peak": peak, "peak_source": src, "unit": "GB/s",
                    "frac": achieved / peak, "frac_of_nominal_8000": achieved / 8000.0,
                    "traffic": alg * NCU_TRAFFIC_GATEUP[0] / NCU_TRAFFIC_GATEUP[1], "algorithmic_bytes_per_launch": alg,
                    "us_per_launch": per_launch_s * 1e6, "launches_timed": args.steps * len(groups),
                    "note": "the step is nothing but launches of this kernel (q|k|v, o, gate|up, down per layer): average over them"}

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
        gref = gpu_reference(dev, stream, raw, max(args.steps // 4, 2)) if want_gpu_ref else None

    # max over ranks; the value counts the model's fixed byte set once, however many ranks share it
    tv = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tv, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(tv[0]), float(tv[1])
    if rank != 0:
        return
    total_bytes = float(set_bytes(model, B))
    value = total_bytes * args.steps / (ms * 1e-3) / 1e9
    e2e = total_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
    line = {"metric": METRIC if B == 1 else f"codebook_gemv_hbm_gbs_batch{B}", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(model, B),
                       "parallelism": f"tp{world}" if world > 1 else "single", "l2": f"inputs larger than L2 ({total_bytes / 1e9:.2f} GB of packed weights per step)",
                       "accumulate": "fp32", "activations": "bf16", "launch": "one CUDA graph per step (q|k|v and gate|up grouped)" + ("" if world == 1 else "; o/down summed over ranks through peer memory in the finish kernel"),
                       "e2e": "a step's inputs from pinned host memory and its results back to pinned host memory (one copy each way), copies and kernels in one CUDA graph, host synchronises every step"},
            "clocks": clocks, "gpu_launches": launches_per_step * args.steps * world,
            "e2e": {"value": e2e, "unit": "GB/s", "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                    "ms_per_step": ms_e2e / args.steps}}
    if roof is not None:
        line["roofline"] = roof
    if tp_check is not None:
        line["tp_check"] = tp_check
    if gref is not None:
        line["gpu_reference"] = gref
    if world == 1 and model == "7b":
        line["cpu_baseline"] = cpu_baseline_sample()
    return_line(args, line, dev, rank, world, local_rank)
    if tp_check is not None and not tp_check["ok"]:
        sys.exit(3)


def return_line(args, line: dict, dev, rank: int, world: int, local_rank: int) -> None:
    """Prints the JSON line; the default run (headline workload, one GPU) first adds the two other parts of the metric,
    measured in this process: prefill TFLOP/s at 2048 tokens and decode tokens/s at batch 1 (short runs)."""
    if world == 1 and args.workload == "gemv" and args.batch == 1 and args.model == "7b" and not args.no_extras:
        torch.cuda.empty_cache()
        try:
            line["prefill"] = run_prefill(argparse.Namespace(**{**vars(args), "tokens": 2048, "steps": 3, "warmup": 3}), rank, world, local_rank, emit=False)
        except Exception as e:
            line["prefill"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        torch.cuda.empty_cache()
        try:
            line["decode"] = run_decode(argparse.Namespace(**{**vars(args), "tokens": 2048, "steps": 64, "warmup": 3, "batch": 1}), rank, world, local_rank, emit=False)
        except Exception as e:
            line["decode"] = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
    print(json.dumps(line), flush=True)


def run_prefill(args, rank: int, world: int, local_rank: int, emit: bool = True):
    """Prefill product of the same matrix set: Y = X W^T for --tokens tokens per matrix on the tcgen05
    kernel; metric TFLOPS = 2 * tokens * R * C summed over the matrices / time.  emit=False: no JSON line, a short
    summary is returned (the default run embeds it)."""
    import torch.distributed as dist
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    T = args.tokens
    from quantexperiments_b200.kernels import DenseStack
    from quantexperiments_b200.linear import DENSE_MIN_TOKENS
    SHAPES = MODELS[args.model]["shapes"]
    lins, kinds, _ = build_set(dev, rank, world, 64, args.model)
    g = torch.Generator(device=dev).manual_seed(7)
    # (an input shard of a matrix with several column orders reads the full activation vector: in_features > C)
    xs = {c: torch.randn(T, c, device=dev, generator=g).bfloat16() for c in sorted({l.in_features for l in lins})}
    flops = sum(2.0 * T * l.R * l.C for l in lins)
    # q|k|v and gate|up share their activations: one stacked product each, as the reference's gemm(x, [pieces]) does.
    # From DENSE_MIN_TOKENS tokens on the stack is decoded once into a 16-bit scratch and multiplied by the TMA-fed
    # tcgen05 GEMM; below, every piece runs the kernel that decodes weight tiles on the fly.
    dense = T >= (args.dense_min if args.dense_min is not None else DENSE_MIN_TOKENS)
    groups, launches = [], 0
    for l0 in range(0, len(lins), len(SHAPES)):
        q, k, v, o, gate, up, down = lins[l0:l0 + len(SHAPES)]
        for members, kind in (((q, k, v), "col"), ((o,), "row"), ((gate, up), "col"), ((down,), "row")):
            y = torch.empty(T, sum(m.R for m in members), device=dev, dtype=torch.bfloat16)
            groups.append((DenseStack([m.dm for m in members]) if dense and not members[0].wide else None, members, xs[members[0].in_features], y, kind))
            launches += (len(members) + 2) if dense else 2 * len(members)

    def run_group(stack, members, x, y, kind):
        if stack is not None:
            stack.gemm(x, y)
        elif members[0].wide:
            members[0].forward_into(x, y)              # wide decode into a zeroed scratch + the same GEMM over all columns
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
    if not emit:
        return {"tokens": T, "value": value, "unit": "TFLOP/s", "ms_per_step": ms / args.steps, "steps": args.steps,
                "frac_of_sustained_peak": value / world / peak, "frac_of_burst_peak": value / world / float(peaks.get("bf16_tflops", 1590.0)),
                "kernel": "k_decode_raw + k_gemm_dense_2sm (tcgen05)", "clocks": clocks}
    line = {"metric": "prefill_dequant_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"{MODELS[args.model]['label']} prefill dequant-GEMM set ({len(lins) * (world if False else 1)} codebook matrices), {T} tokens", "accumulate": "fp32",
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


def run_decode(args, rank: int, world: int, local_rank: int, emit: bool = True):
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
    if not emit:
        return {"batch": B, "prompt": T, "value": B * K * world / (ms * 1e-3), "unit": "tok/s", "ms_per_step": ms / K, "steps": K,
                "step_hbm_frac": achieved / peak, "clocks": clocks}
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


# ----------------------------------------------------------------------------------------- small cases for a profiler
def _case_matrix(R: int, C: int, seed: int = 0, books: int = 1):
    from quantexperiments_b200.kernels import DeviceMatrix
    g = torch.Generator(device="cuda").manual_seed(seed)
    W = (C // 8 * 12 + 31) // 32
    kw = {}
    if books == 2:
        kw = {"tags2": torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device="cuda", generator=g),
              "table2": torch.randn(4096, 8, device="cuda", generator=g).half()}
    return DeviceMatrix(torch.randint(-2**31, 2**31 - 1, (R, W), dtype=torch.int32, device="cuda", generator=g),
                        torch.randn(4096, 8, device="cuda", generator=g).half(),
                        (torch.rand(R, device="cuda", generator=g) * 0.02 + 0.01).half(), K=4096, d=8, C=C, **kw)


def _case_gemv_l8(shapes):
    """A grouped batch-1 launch on distinct matrices, a few times (every launch streams its tags from HBM: ncu flushes
    the caches before a captured launch, and 12 matrices of the largest shape exceed L2 anyway)."""
    from quantexperiments_b200.kernels import L8Group, L8Matrix
    grps = [L8Group([L8Matrix(_case_matrix(R, C, seed=7 * i + j)) for j, (R, C) in enumerate(shapes)]) for i in range(4)]
    x = torch.randn(shapes[0][1], device="cuda").bfloat16()
    ys = [torch.empty(R, device="cuda", dtype=torch.bfloat16) for R, _ in shapes]
    for rep in range(2):
        for grp in grps:
            grp.run(x, ys)


def _case_gemv_t16():
    from quantexperiments_b200.kernels import T16Matrix
    ms = [T16Matrix(_case_matrix(18944, 3584, seed=i)) for i in range(6)]
    x, y = torch.randn(1, 3584, device="cuda").bfloat16(), torch.empty(1, 18944, device="cuda", dtype=torch.bfloat16)
    for m in ms:
        m.run(x, y)


def _case_gemv_x16():
    from quantexperiments_b200.kernels import X16Matrix
    xm = X16Matrix(_case_matrix(37888, 3584))
    X, Y = torch.randn(16, 3584, device="cuda").bfloat16(), torch.empty(16, 37888, device="cuda", dtype=torch.bfloat16)
    xp = xm.prep(X, 16)
    for _ in range(3):
        xm.run_prepped(xp, Y, 16)


def _case_gemm(dense: bool):
    from quantexperiments_b200.kernels import DenseStack, L8Matrix
    dm = _case_matrix(18944, 3584)
    X, Y = torch.randn(2048, 3584, device="cuda").bfloat16(), torch.empty(2048, 18944, device="cuda", dtype=torch.bfloat16)
    if dense:
        st = DenseStack([dm])
        for _ in range(3):
            st.gemm(X, Y)
        DenseStack.status("cuda")
    else:
        l8 = L8Matrix(dm)
        for _ in range(3):
            l8.gemm(X, Y)
        l8.status()


def _case_assign():
    from quantexperiments_b200 import codebook as cb
    n = 148 * 2048 * 4
    g = torch.Generator(device="cuda").manual_seed(0)
    x, wt = torch.randn(n, 8, device="cuda", generator=g), torch.rand(n, 8, device="cuda", generator=g)
    book = torch.randn(4096, 8, device="cuda", generator=g).half()
    for w in (None, None, wt, wt):
        cb.assign(x, book, wt=w)


def _case_decode_step(B: int):
    from quantexperiments_b200.engine import Cfg, Qwen2BatchEngine, random_engine
    eng = random_engine(Cfg(max_len=2304, layers=4), seed=0)
    if B > 1:
        eng = Qwen2BatchEngine(eng, B)
    eng.reset()
    eng.pos.fill_(2048)
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    eng.step()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    eng.check()


PROFILE_CASES = {
    "gemv_l8_gateup": lambda: _case_gemv_l8([(18944, 3584), (18944, 3584)]),    # the largest batch-1 launch of the 7B set
    "gemv_l8_down": lambda: _case_gemv_l8([(3584, 18944)]),
    "gemv_l8_qkv": lambda: _case_gemv_l8([(3584, 3584), (512, 3584), (512, 3584)]),
    "gemv_t16_gate": _case_gemv_t16,
    "gemv_x16_gateup": _case_gemv_x16,
    "gemm_dense_gate": lambda: _case_gemm(True),
    "gemm_l8_gate": lambda: _case_gemm(False),
    "assign": _case_assign,
    "decode_step_1": lambda: _case_decode_step(1),                              # uses cudaProfilerStart/Stop around the last step
    "decode_step_32": lambda: _case_decode_step(32),
}


def run_profile_case(name: str) -> None:
    """One small case of a kernel on cuda:0 (sizes chosen so that an ncu capture of one to three launches ends in a
    minute or two): the commands in profiles/*.md run these."""
    torch.cuda.set_device(0)
    PROFILE_CASES[name]()
    torch.cuda.synchronize()
    print("ok", name)


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
    ap.add_argument("--model", default="7b", choices=sorted(MODELS), help="gemv / prefill: the shape set (7b: one book, one column order; "
                    "32b: two summed books and 16 seeded column orders per matrix)")
    ap.add_argument("--no-extras", action="store_true", help="gemv: skip the prefill / decode / reference-kernel legs that the default run adds to its line")
    ap.add_argument("--profile-case", default=None, choices=sorted(PROFILE_CASES),
                    help="run one small case for a profiler (a few launches between cudaProfilerStart/Stop) instead of a benchmark")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if args.profile_case:
        run_profile_case(args.profile_case)
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
