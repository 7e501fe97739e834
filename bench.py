#!/usr/bin/env python
"""Benchmark of the NVFP4 GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic input: one
NVFP4 block-scaled GEMM of the named workload (default: M=N=K=8192, seeded bf16
N(0,1) operands quantised to E2M1 + UE4M3 scales, FP32 accumulation, FP16
output). With N > 1 (one rank per GPU under torchrun) B is sharded by rows over
the ranks (N-column sharding of C) and the same total problem is timed: strong
scaling. Rank 0 prints ONE JSON line.

`--impl reference` times the reference's CPU path (dequantise both operands,
FP32 matmul, FP16 rounding) restated in oracle/ on the host cores.
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

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (M, N, K, sigma of B)
    "gemm8192": (8192, 8192, 8192, 1.0),
    "gemm16384": (16384, 16384, 16384, 1.0),
    "skinny": (128, 28672, 8192, 0.02),
    "gemm256": (256, 256, 256, 1.0),
}
# Routed-MoE expert layer (H=4096, I=2048, 256 experts, top-6), tokens PER GPU; experts are split over the ranks.
MOE_WORKLOADS = {"moe_t1": 1, "moe_t64": 64, "moe_t1024": 1024, "moe_t4096": 4096,
                 # a quarter of the experts at the row count per expert of moe_t4096: small enough for an ncu capture
                 "moe_t1024_e64": 1024, "moe_t4096_e64": 4096}
MOE_EXPERTS = {"moe_t1024_e64": 64, "moe_t4096_e64": 64}
MOE_SHAPE = {"hidden": 4096, "inter": 2048, "experts": 256, "topk": 6, "clamp": 10.0}
# Stand-alone quantise/pack kernel: (rows, K) of a bf16 operand.
QUANT_WORKLOADS = {"quantise8192": (8192, 8192), "quantise16384": (16384, 16384), "quantise_skinny_b": (28672, 8192)}
METRIC = "nvfp4_gemm_tflops"
UNIT = "TFLOP/s"
NOMINAL_FP4_TFLOPS = 9000.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch of nvfp4_gemm_kernel, from the
# ncu captures summarised under profiles/ (None until a capture of that workload exists).
NCU_DRAM_BYTES_PER_LAUNCH = {"gemm8192": 218_190_336, "gemm16384": None, "skinny": 136_602_624,
                             # quantise_kernel<bf16>: part of the output was still in L2 when the capture ended
                             "quantise8192": 155_176_960}


def algorithmic_bytes(m, n, k):
    """Packed A and B, both scale arrays, and C written once (FP16)."""
    return m * k // 2 + n * k // 2 + m * k // 16 + n * k // 16 + 2 * m * n


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"],
                "bf16_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        inside = [r for t, r in self.rows if t0 <= t <= t1 and len(r) >= 7]
        window = "timed region"
        if len(inside) < 3:
            inside = [r for _, r in self.rows if len(r) >= 7]
            window = "warm-up + timed region + continuation"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in inside)]
        nums = lambda j: [float(r[j]) for r in inside if r[j].replace(".", "", 1).isdigit()]
        return {"sm_mhz": statistics.median(nums(0)) if nums(0) else None,
                "sm_max_mhz": max(nums(1)) if nums(1) else None,
                "power_w_max": max(nums(2)) if nums(2) else None,
                "reasons": reasons, "samples": len(inside), "window": window}


def cpu_reference_pass(m, n, k, sigma_b, budget_s=20.0):
    """The reference's CPU path on a bounded sample: all of B, the first rows of A."""
    import numpy as np
    import torch
    from oracle import nvfp4_oracle as O
    cores = os.cpu_count() or 1
    torch.manual_seed(0)
    # measured here at ~0.45 TFLOP/s on 8 cores; size the A slab for about `budget_s` seconds in total
    rows = m
    est = (2.0 * m * n * k) / (0.05e12 * cores) + 3e-8 * (m + n) * k
    if est > budget_s:
        rows = max(128, int(m * budget_s / est) // 128 * 128)
    # Quantising 2 x 64M values with the numpy oracle would take far longer than the timed pass itself,
    # so a 1024-row seeded block of each operand is quantised and repeated down the rows (whole scale
    # atoms, so the repeated arrays are valid operands with the same value distribution).
    def operand(r, sigma):
        base = min(r, 1024)
        x = (torch.randn((base, k), dtype=torch.bfloat16).float() * sigma).numpy()
        p, s = O.quantize(x)
        reps = -(-r // base)
        return np.tile(p, (reps, 1))[:r], np.tile(s, reps)[:r * k // 16]
    pa, sa = operand(rows, 1.0)
    pb, sb = operand(n, sigma_b)
    t0 = time.perf_counter()
    c = O.gemm(pa, sa, pb, sb)
    dt = time.perf_counter() - t0
    assert c.shape == (rows, n)
    return 2.0 * rows * n * k / dt / 1e12, cores, f"rows 0..{rows - 1} of A against all of B ({rows}x{n}x{k}), dequantise + FP32 matmul + FP16, {dt:.1f} s"


def run_reference(args, rank, world):
    if rank != 0:
        return
    m, n, k, sigma = WORKLOADS[args.workload]
    for _ in range(min(args.warmup, 1)):
        cpu_reference_pass(min(m, 256), min(n, 1024), min(k, 1024), sigma, 2.0)
    values = []
    steps = max(1, min(args.steps, 3))
    t0 = time.perf_counter()
    for _ in range(steps):
        v, cores, sample = cpu_reference_pass(m, n, k, sigma, 20.0)
        values.append(v)
    dt = time.perf_counter() - t0
    value = statistics.median(values)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": 1e3 * dt / steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3), f32 accumulate, f16 out",
        "data": "synthetic", "config": {"workload": args.workload, "M": m, "N": n, "K": k, "layout": "TN"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def run_ours(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    import gpu_kernels_b200 as g
    from gpu_kernels_b200 import _lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    m, n, k, sigma = WORKLOADS[args.workload]
    lo, hi = g.slab_rows(n, world, rank)
    n_local = hi - lo
    lib = _lib.load()
    l2 = lib.gpu_kernels_nvfp4_l2_bytes()

    # Seeded synthetic operands (the full B on every rank, then this rank's slab).
    gen = torch.Generator(device=dev).manual_seed(0)
    a = torch.randn((m, k), generator=gen, device=dev, dtype=torch.float32).bfloat16()
    pa, sa = g.quantize(a)
    del a
    b = (torch.randn((n, k), generator=gen, device=dev, dtype=torch.float32) * sigma).bfloat16()
    pb_full, sb_full = g.quantize(b)
    del b
    pb, sb = (t.clone() for t in g.shard_b(pb_full, sb_full, world, rank))
    del pb_full, sb_full
    torch.cuda.empty_cache()

    # Operand rotation: consecutive steps read different copies, together larger than twice the L2.
    in_bytes = sum(t.numel() for t in (pa, sa, pb, sb))
    rotations = max(2, -(-2 * l2 // in_bytes))
    rotations = min(rotations, 64)
    sets = [(pa, sa, pb, sb)] + [tuple(t.clone() for t in (pa, sa, pb, sb)) for _ in range(rotations - 1)]
    plans = [g.Nvfp4Gemm(x[0], x[2], x[1], x[3]) for x in sets]
    for plan in plans:
        # four units per tile where the library offers it (a slab with far fewer tiles than SMs); this
        # process owns the GPU, which is what the option needs
        try:
            plan.set_option("split_k", 1)
        except RuntimeError:
            break
    out = torch.empty((m, n_local), dtype=torch.float16, device=dev)
    full = torch.empty((m, n), dtype=torch.float16, device=dev) if (world > 1 and args.gather == "nccl") else None
    shared = None
    if world > 1 and args.gather == "fused":
        # every rank's full C is mapped into all ranks; the GEMM's epilogue writes the slab into all of them
        shared = g.GatheredOutput(m, n, dev)
        for plan in plans:
            shared.attach(plan, lo)

    def step(i):
        plans[i % rotations].run(out)
        if shared is not None:
            shared.barrier()
        elif full is not None:
            g.gather_columns(out, None, full)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    graph = None
    if args.graph:
        # the steps of one pass over the operand copies recorded once and replayed: no launch cost on the host
        # (every rank captures and replays the same sequence, barriers and collectives included)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(rotations):
                    step(i)
        torch.cuda.current_stream().wait_stream(side)
        args.steps = max(1, args.steps // rotations) * rotations
        for _ in range(2):
            graph.replay()
        barrier()
    launches0 = _lib.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    if graph is not None:
        for _ in range(args.steps // rotations):
            graph.replay()
    else:
        for i in range(args.steps):
            step(i)
    stop.record()
    barrier()
    t1 = time.perf_counter()
    launches = args.steps if graph is not None else _lib.launch_count() - launches0
    ms = start.elapsed_time(stop)
    if sampler is not None and (t1 - t0) < 0.5:
        # the timed region is shorter than a few sampling periods: keep the same load running for the sampler only
        until = time.perf_counter() + 0.7
        i = 0
        while time.perf_counter() < until:
            plans[i % rotations].run(out); i += 1      # kernel only: no collective outside the lock-step region
            if i % 64 == 0:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
    clocks = sampler.stop(t0, t1) if sampler is not None else None
    plans[0].validate()
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())

    # The library bar on the same box in the same run: cuBLASLt's own NVFP4 matmul on the same operands.
    library_bar = None
    if world == 1:
        try:
            ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
            lt_plans = [g.Nvfp4Gemm(x[0], x[2], x[1], x[3], workspace=ws) for x in sets]
            for i in range(3):
                lt_plans[i % rotations].run_cublaslt(out)
            torch.cuda.synchronize()
            start.record()
            for i in range(args.steps):
                lt_plans[i % rotations].run_cublaslt(out)
            stop.record()
            torch.cuda.synchronize()
            lt_ms = start.elapsed_time(stop) / args.steps
            library_bar = {"name": "cuBLASLt NVFP4 matmul (VEC16_UE4M3), same operands, same run",
                           "ms_per_step": lt_ms, "value": 2.0 * m * n * k / (lt_ms * 1e-3) / 1e12, "unit": UNIT}
            for p_ in lt_plans:
                p_.close()
        except Exception as exc:                                  # the bar is informative only
            library_bar = {"name": "cuBLASLt NVFP4 matmul", "unavailable": str(exc)[:200]}

    # End to end through the C ABI with HOST buffers: H2D of the operands, kernel, D2H of C, every step.
    host = [t.cpu().pin_memory() for t in (pa, pb, sa, sb)]
    host_c = torch.empty((m, n_local), dtype=torch.float16).pin_memory()
    e2e_steps = max(2, min(args.steps, 10))
    g.gemm_host(*host, host_c)
    barrier()
    te = time.perf_counter()
    start.record()
    for _ in range(e2e_steps):
        g.gemm_host(*host, host_c)
    stop.record()
    barrier()
    e2e_ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    del te
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = host_c.numel() * 2
    if shared is not None:
        shared.close()                                          # collective: before any rank leaves

    if rank != 0:
        return
    flops = 2.0 * m * n * k
    ms_per_step = ms / args.steps
    value = flops / (ms_per_step * 1e-3) / 1e12
    peaks = measured_peaks()
    timed_s = ms * 1e-3
    bf16 = peaks["bf16_sustained"] if timed_s > 1.0 else peaks["bf16_burst"]
    tensor_peak = 4.0 * bf16
    per_gpu_tflops = value / world
    alg_bytes = algorithmic_bytes(m, n_local, k)
    gbs = alg_bytes / (ms_per_step * 1e-3) / 1e9
    # which roof bounds this workload: compare time at the tensor peak with time at the HBM peak
    t_tensor = (flops / world) / (tensor_peak * 1e12)
    t_hbm = alg_bytes / (peaks["hbm_gbs"] * 1e9)
    if t_tensor >= t_hbm:
        roofline = {"bound": "tensor", "achieved": per_gpu_tflops, "peak": tensor_peak, "unit": "TFLOP/s",
                    "frac": per_gpu_tflops / tensor_peak,
                    "peak_source": f"4 x {peaks['source']} cuBLAS bf16 ({'sustained' if timed_s > 1.0 else 'burst'}): "
                                   "no FP4 peak is measured on this pool; FP4 dense is 4x bf16 on the same pipe",
                    "frac_of_nominal_9pf": per_gpu_tflops / NOMINAL_FP4_TFLOPS}
    else:
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth"}
    roofline["kernel"] = "nvfp4_gemm_kernel"
    roofline["algorithmic_bytes_per_launch"] = alg_bytes
    roofline["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload) if world == 1 else None

    cpu = None
    if world == 1 and not args.no_cpu:
        v, cores, sample = cpu_reference_pass(m, n, k, sigma, 15.0)
        cpu = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    info = plans[0].info()
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3), f32 accumulate, f16 out", "data": "synthetic",
        "config": {"workload": args.workload, "M": m, "N": n, "K": k, "layout": "TN",
                   "sharding": f"B rows over {world} rank(s), {n_local} columns of C per rank",
                   "gather": args.gather if world > 1 else "none",
                   "launch": "CUDA graph of one pass over the operand copies, replayed" if graph is not None else "one launch per step from the host",
                   "l2": f"operand rotation over {rotations} copies ({rotations * in_bytes >> 20} MiB > 2 x L2 {l2 >> 20} MiB)",
                   "plan": info},
        "clocks": clocks,
        "e2e": {"value": flops / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": UNIT,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "call": "gpu_kernels_nvfp4_gemm_host (pinned host buffers)"},
        "gpu_launches": int(launches),
        "roofline": roofline,
        "cpu_baseline": cpu,
        "library_bar": library_bar,
    }))


def run_quantise(args, rank, world, local_rank):
    """One step = quantise one bf16 [rows, K] operand (different copies in turn, together larger than L2)."""
    import torch
    import gpu_kernels_b200 as g
    from gpu_kernels_b200 import _lib
    if rank != 0:
        return
    torch.cuda.set_device(local_rank)
    rows, k = QUANT_WORKLOADS[args.workload]
    copies = max(2, (512 << 20) // (rows * k * 2))
    gen = torch.Generator(device="cuda").manual_seed(0)
    xs = [torch.randn((rows, k), generator=gen, device="cuda").bfloat16() for _ in range(copies)]
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device="cuda")
    scales = torch.empty(rows * k // 16, dtype=torch.uint8, device="cuda")
    lib, stream = _lib.load(), torch.cuda.current_stream().cuda_stream
    def step(i):
        _lib.check(lib.gpu_kernels_nvfp4_quantize(xs[i % copies].data_ptr(), 0, packed.data_ptr(), scales.data_ptr(), rows, k, stream))
    for i in range(max(3, args.warmup)):
        step(i)
    torch.cuda.synchronize()
    n0 = _lib.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        step(i)
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / args.steps
    alg = rows * k * 2 + rows * k // 2 + rows * k // 16
    gbs = alg / (ms * 1e-3) / 1e9
    peaks = measured_peaks()
    cpu = None
    if not args.no_cpu:
        # the same operand through the CPU restatement of the reference's quantiser (numpy, one thread),
        # on a bounded sample of its rows
        from oracle import nvfp4_oracle as O
        sample_rows = 128
        while sample_rows * 2 <= rows and sample_rows * k < (1 << 24):
            sample_rows *= 2
        host = xs[0][:sample_rows].float().cpu().numpy()
        O.quantize(host[:128])
        t0 = time.perf_counter()
        O.quantize(host)
        dt = time.perf_counter() - t0
        cpu = {"value": (alg * sample_rows / rows) / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
               "sample": f"rows 0..{sample_rows - 1} of the operand ({sample_rows}x{k}), {dt:.1f} s"}
    print(json.dumps({
        "metric": "nvfp4_quantise_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 in, e2m1 + ue4m3 out", "data": "synthetic",
        "config": {"workload": args.workload, "rows": rows, "K": k, "l2": f"{copies} input copies in turn ({copies * rows * k * 2 >> 20} MiB)"},
        "gpu_launches": int(_lib.launch_count() - n0),
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                     "peak_source": f"{peaks['source']} copy bandwidth", "kernel": "quantise_kernel<bf16>",
                     "algorithmic_bytes_per_launch": alg, "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(args.workload)},
        "cpu_baseline": cpu, "e2e": None}))


def moe_cpu_baseline(layer, g, sample, hidden, inter, topk, clamp):
    """The reference's CPU statement of the layer (moe_forward: FP32 matmuls with its bf16 rounding points) on the
    dequantised expert weights, for the first tokens of one input set."""
    import numpy as np
    from oracle import moe_oracle as MO
    x, ids, wts = sample
    count = min(2, x.shape[0])
    x, ids, wts = x[:count].float().cpu().numpy(), ids[:count].cpu().numpy(), wts[:count].cpu().numpy()
    used = np.unique(ids)
    two_i = 2 * inter
    w1 = np.empty((len(used), two_i, hidden), np.float32)
    w2 = np.empty((len(used), hidden, inter), np.float32)
    for i, e in enumerate(used):
        r0 = int(e) * two_i
        d = g.dequantize(layer.w1q[r0:r0 + two_i], layer.w1s[r0 * hidden // 16:(r0 + two_i) * hidden // 16])
        if layer.fused:                                         # rows are stored 16 gate / 16 up interleaved
            d = d.reshape(inter // 16, 2, 16, hidden).permute(1, 0, 2, 3).reshape(two_i, hidden)
        w1[i] = d.cpu().numpy()
        r0 = int(e) * hidden
        w2[i] = g.dequantize(layer.w2q[r0:r0 + hidden], layer.w2s[r0 * inter // 16:(r0 + hidden) * inter // 16]).cpu().numpy()
    local_ids = np.searchsorted(used, ids)
    MO.moe_forward(x[:1], local_ids[:1], wts[:1], w1, w2, clamp)
    t0 = time.perf_counter()
    MO.moe_forward(x, local_ids, wts, w1, w2, clamp)
    dt = time.perf_counter() - t0
    flops = count * topk * 2.0 * (two_i * hidden + hidden * inter)
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
            "sample": f"the first {count} token(s) of one input set ({count * topk} routes, {len(used)} experts) through "
                      f"moe_forward on the dequantised weights, numpy BLAS threads, {dt:.3f} s"}


def run_moe(args, rank, world, local_rank):
    """One step = one forward of the NVFP4 expert layer on `tokens` tokens per GPU (weak scaling in tokens)."""
    import torch
    import torch.distributed as dist
    import gpu_kernels_b200 as g
    from gpu_kernels_b200 import _lib

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    tokens = MOE_WORKLOADS[args.workload]
    H, I, E, topk, clamp = (MOE_SHAPE[k] for k in ("hidden", "inter", "experts", "topk", "clamp"))
    E = MOE_EXPERTS.get(args.workload, E)
    local = E // world
    gen = torch.Generator(device=dev).manual_seed(rank)
    w1 = torch.empty((local, 2 * I, H), dtype=torch.bfloat16, device=dev)
    w2 = torch.empty((local, H, I), dtype=torch.bfloat16, device=dev)
    for e in range(local):                                      # expert by expert: keeps the FP32 temporaries small
        w1[e] = (torch.randn((2 * I, H), generator=gen, device=dev) * 0.02).bfloat16()
        w2[e] = (torch.randn((H, I), generator=gen, device=dev) * 0.02).bfloat16()
    layer = g.Nvfp4MoE(w1, w2, E, topk, clamp=clamp, max_tokens=tokens)
    del w1, w2
    torch.cuda.empty_cache()
    sets = []
    for i in range(4):                                          # rotating inputs: routing changes every step
        x = torch.randn((tokens, H), generator=gen, device=dev).bfloat16()
        ids, wts = g.route(torch.randn((tokens, E), generator=gen, device=dev), topk)
        sets.append((x, ids, wts))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    for i in range(max(3, args.warmup)):
        layer(*sets[i % 4])
    barrier()
    launches0 = _lib.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for i in range(args.steps):
        layer(*sets[i % 4])
    stop.record()
    barrier()
    t1 = time.perf_counter()
    launches = _lib.launch_count() - launches0
    ms_eager = start.elapsed_time(stop)
    # the same forward recorded once as a CUDA graph and replayed (inputs copied into the graph's buffers on
    # the device inside the timed region): no per-kernel launch cost on the host
    gx, gids, gwts, gy, graph = layer.capture(tokens)

    def replay(i):
        x_, ids_, wts_ = sets[i % 4]
        gx.copy_(x_); gids.copy_(ids_); gwts.copy_(wts_)
        graph.replay()

    for i in range(3):
        replay(i)
    barrier()
    start.record()
    for i in range(args.steps):
        replay(i)
    stop.record()
    barrier()
    t1 = time.perf_counter()
    ms = start.elapsed_time(stop)
    if (t1 - t0) < 0.5:
        # the timed region is shorter than a few sampling periods of the clock sampler: every rank keeps the same
        # load running for the same number of further steps (the forward is collective), for the sampler only
        more = torch.tensor([0.7 / max(ms / args.steps * 1e-3, 1e-6)], device=dev)
        if world > 1:
            dist.all_reduce(more, op=dist.ReduceOp.MIN)
        for i in range(int(min(more.item(), 20000))):
            replay(i)
        barrier()
    clocks = sampler.stop(t0, t1) if sampler is not None else None
    # end to end: inputs from pinned host memory, result back to the host, every step
    host = [tuple(t.cpu().pin_memory() for t in s_) for s_ in sets]
    y_host = torch.empty((tokens, H), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(2, min(args.steps, 10))
    barrier()
    start.record()
    for i in range(e2e_steps):
        xs = [t.to(dev, non_blocking=True) for t in host[i % 4]]
        y_host.copy_(layer(*xs), non_blocking=True)
    stop.record()
    barrier()
    e2e_ms = start.elapsed_time(stop)
    if world > 1:
        t = torch.tensor([ms, e2e_ms, ms_eager], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, ms_eager = (float(v) for v in t.tolist())
    filler = torch.empty(1 << 28, dtype=torch.uint8, device=dev)
    for _ in range(24):                                         # ~2 ms of device work, so that the host runs ahead and
        filler.zero_()                                          # the marks below time the device, not the launches
    layer.phase_events = []
    layer(*sets[0])
    phases = {k_: round(v_, 1) for k_, v_ in layer.phase_times_us().items()}
    layer.phase_events = None
    touched = int((layer.counts_matrix.sum(0)[rank * local:(rank + 1) * local] > 0).sum().item())
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = moe_cpu_baseline(layer, g, sets[0], H, I, topk, clamp)
    del graph
    layer.close()                                               # collective (unmaps the peers' buffers): every rank
    if rank != 0:
        return
    routes = world * tokens * topk
    flops = routes * 2.0 * (2 * I * H + H * I)
    ms_per_step = ms / args.steps
    value = flops / (ms_per_step * 1e-3) / 1e12
    peaks = measured_peaks()
    weight_bytes = touched * (2 * I * H + H * I) * 9 // 16      # packed values + scale bytes of the experts this rank touched
    act_bytes = tokens * topk * (H // 2 + H // 16 + 2 * (2 * I) * 2 + I // 2 + I // 16 + 2 * H * 2)
    alg_bytes = weight_bytes + act_bytes
    t_hbm = alg_bytes / (peaks["hbm_gbs"] * 1e9)
    tensor_peak = 4.0 * peaks["bf16_burst"]
    t_tensor = (flops / world) / (tensor_peak * 1e12)
    if t_hbm >= t_tensor:
        gbs = alg_bytes / (ms_per_step * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                    "peak_source": f"{peaks['source']} copy bandwidth", "traffic": None,
                    "algorithmic_bytes_per_step": alg_bytes, "kernel": "nvfp4_gemm_kernel<1,256> grouped (FC1 + FC2)",
                    "note": "whole-step time (every kernel and collective of the forward) against the bytes of the two grouped GEMMs"}
    else:
        roofline = {"bound": "tensor", "achieved": value / world, "peak": tensor_peak, "unit": "TFLOP/s",
                    "frac": value / world / tensor_peak, "peak_source": f"4 x {peaks['source']} cuBLAS bf16 (burst)",
                    "traffic": None, "kernel": "nvfp4_gemm_kernel<1,256> grouped (FC1 + FC2)",
                    "note": "whole-step time against the FLOPs of the two grouped GEMMs"}
    print(json.dumps({
        "metric": "nvfp4_moe_tflops", "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 operands, f32 accumulate, bf16 activations and output", "data": "synthetic",
        "config": {"workload": args.workload, "tokens_per_gpu": tokens, **{**MOE_SHAPE, "experts": E}, "expert_parallel": world,
                   "experts_touched_rank0": touched, "launch": "one CUDA graph per forward (Nvfp4MoE.capture)",
                   "ms_per_step_eager": ms_eager / args.steps, "phases_us_rank0_eager": phases, "l2": f"expert weights ({E * 14.2e-3:.1f} GB for {E} experts) far exceed L2; inputs rotate over 4 sets"},
        "clocks": clocks,
        "e2e": {"value": flops / (e2e_ms / e2e_steps * 1e-3) / 1e12, "unit": UNIT,
                "h2d_bytes_per_step": tokens * (H * 2 + topk * 12), "d2h_bytes_per_step": tokens * H * 2, "steps": e2e_steps,
                "call": "Nvfp4MoE.forward on tensors copied from pinned host memory, result copied back"},
        "gpu_launches": int(launches), "roofline": roofline, "cpu_baseline": cpu,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm8192", choices=sorted(WORKLOADS) + sorted(MOE_WORKLOADS) + sorted(QUANT_WORKLOADS))
    ap.add_argument("--gather", nargs="?", const="fused", default="none", choices=["none", "fused", "nccl"],
                    help="N>1: every step also leaves the full C on every rank: 'fused' = the GEMM's epilogue stores the "
                         "slab into all ranks' buffers over NVLink + a barrier; 'nccl' = all-gather + strided copy")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--graph", action="store_true", help="GEMM workloads: time CUDA-graph replays instead of host launches")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if args.workload in MOE_WORKLOADS or args.workload in QUANT_WORKLOADS:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "the CPU reference arm times the GEMM workloads only"}))
            return
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        from datetime import timedelta
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=timedelta(seconds=90))
    try:
        if args.workload in MOE_WORKLOADS:
            run_moe(args, rank, world, local_rank)
        elif args.workload in QUANT_WORKLOADS:
            run_quantise(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
