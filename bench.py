#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path: block-scaled GEMM, quantiser, N-sharded GEMM, routed-MoE expert layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--only]

One "step" is one pass of the hot path over one batch of synthetic input. The headline workload is one NVFP4
block-scaled GEMM with M=N=K=8192 (seeded bf16 N(0,1) operands quantised to E2M1 + UE4M3 scales, FP32
accumulation, FP16 output). With N > 1 (one rank per GPU under torchrun) B is sharded by rows over the ranks
(N-column sharding of C) and the same total problem is timed: strong scaling. Rank 0 prints ONE JSON line.

Timing follows the reference's own harness (benchmarks/common.py:67-115, benchmarks/nvfp4.py:43-57): the step
is recorded as a CUDA graph of at least ten launches over a rotation of operand copies larger than twice the
L2, replayed for a warm-up of one second, then timed in nine samples of at least 20 ms each with CUDA events
(max over ranks per sample); `value` is the median sample. The K steps asked for on the command line are also
timed once, launched from the host right after W warm-up steps, and reported under `burst`.

Unless `--only` is given, the same invocation also measures the other configurations of the path
(16384^3, the skinny decode shape, the stand-alone quantiser, the expert layer at 1/64/1024/4096 tokens per
GPU) with a shorter warm-up, and reports them under `configs`. After timing, results are checked (`parity`):
sampled rows against the FP32 dequantise-then-matmul path and the CPU oracle, the fused all-gather against
the NCCL route bit for bit, the expert layer on sampled tokens against the oracle; the ranks agree on the
verdict through an all-reduce, and a failed check makes every rank exit non-zero.

`--impl reference` times the reference's CPU path (dequantise both operands, FP32 matmul, FP16 rounding:
reference/python/nvfp4.py:40-47, benchmarks/nvfp4.py:41) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GEMM_WORKLOADS = {
    # name: (M, N, K, sigma of B)
    "gemm8192": (8192, 8192, 8192, 1.0),
    "gemm16384": (16384, 16384, 16384, 1.0),
    "skinny": (128, 28672, 8192, 0.02),
    "gemm256": (256, 256, 256, 1.0),
}
# Routed-MoE expert layer (H=4096, I=2048, 256 experts, top-6), tokens PER GPU; experts are split over the ranks.
MOE_WORKLOADS = {"moe_t1": 1, "moe_t64": 64, "moe_t1024": 1024, "moe_t4096": 4096}
MOE_SHAPE = {"hidden": 4096, "inter": 2048, "experts": 256, "topk": 6, "clamp": 10.0}
# Stand-alone quantise/pack kernel: (rows, K) of a bf16 operand.
QUANT_WORKLOADS = {"quantise8192": (8192, 8192), "quantise16384": (16384, 16384), "quantise_skinny_b": (28672, 8192)}
METRIC = "nvfp4_gemm_tflops"
UNIT = "TFLOP/s"
NOMINAL_FP4_TFLOPS = 9000.0
NVLINK_GBS_PER_DIRECTION = 900.0
DTYPE = "nvfp4 (e2m1 x ue4m3), f32 accumulate, f16 out"

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the workload's kernel, from one
# ncu capture of that workload; None where no capture exists. A reported constant, not measured by this run.
NCU_DRAM_BYTES_PER_LAUNCH = {"gemm8192": 222_000_000, "gemm16384": 1_747_000_000, "skinny": 138_900_000,
                             "quantise8192": 156_000_000}
# MXFP4 (the adjacent format of the same kernel; no counterpart in the reference): M, N, K, sigma of B
MX_WORKLOADS = {"mxfp4_gemm8192": (8192, 8192, 8192, 0.02)}

# GEMM acceptance against the FP32 dequantise-then-matmul path (the bound the tests use).
REL_FROBENIUS = 1e-3
MAX_ABS_OVER_RMS = 2e-2
# whole expert layer (two quantised GEMMs with bf16 rounding points in sequence)
LAYER_REL_FROBENIUS = 2e-2
LAYER_MAX_ABS_OVER_RMS = 0.25


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
    """nvidia-smi clocks and throttle reasons while the timed regions run (read-only queries)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "25", "-i", str(index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def window(self, t0, t1):
        """Summary of the samples taken between two host times (both inside a timed region)."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        inside = [r for t, r in list(self.rows) if t0 <= t <= t1 and len(r) >= 7]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"], "samples": 0}
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in inside)]
        nums = lambda j: [float(r[j]) for r in inside if r[j].replace(".", "", 1).isdigit()]
        return {"sm_mhz": statistics.median(nums(0)) if nums(0) else None,
                "sm_max_mhz": max(nums(1)) if nums(1) else None,
                "power_w_max": max(nums(2)) if nums(2) else None,
                "reasons": reasons, "samples": len(inside), "window": "timed samples (first start to last stop)"}

    def stop(self):
        if self.proc:
            self.proc.terminate()
            self.thread.join(timeout=2)


class Ranks:
    """The process group as the timing and checking code needs it (works for one process too)."""

    def __init__(self, rank, world, local_rank):
        self.rank, self.world, self.local_rank = rank, world, local_rank

    def barrier(self):
        import torch
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    def reduce(self, values, op="max"):
        """Element-wise max (or min) of a list of floats over the ranks."""
        if self.world == 1:
            return list(values)
        import torch
        import torch.distributed as dist
        t = torch.tensor(list(values), dtype=torch.float64, device=torch.device("cuda", self.local_rank))
        dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN)
        return t.tolist()

    def all_ok(self, ok: bool) -> bool:
        """True when every rank passed: the ranks learn of a failure together and leave together."""
        return self.reduce([1.0 if ok else 0.0], "min")[0] > 0.5


def time_replays(step, ranks: Ranks, cycle: int, graph_ops: int, warmup_s: float, trials: int, sample_ms: float,
                 sampler: ClockSampler | None = None, prepare=None):
    """The reference harness's method for one workload.

    step(i) enqueues step number i on the current stream; the steps cycle through `cycle` input sets. A CUDA
    graph of a whole number of cycles with at least `graph_ops` steps is captured, replayed for `warmup_s`
    seconds, then timed `trials` times over at least `sample_ms` each (every rank replays the same number of
    times; a sample is the max over ranks). prepare(i), if given, is called before each replay outside the graph
    (e.g. copies the next inputs into the graph's static tensors). Returns a dict with the per-step samples in
    ms, their median, the graph size and the clocks seen while the samples ran.
    """
    import torch
    ops = max(1, math.ceil(graph_ops / cycle)) * cycle
    for i in range(min(ops, 3 * cycle)):
        step(i)
    ranks.barrier()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(ops):
                step(i)
    torch.cuda.current_stream().wait_stream(side)
    ranks.barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    calls = [0]

    def elapsed(replays):
        ranks.barrier()
        start.record()
        for _ in range(replays):
            if prepare is not None:
                prepare(calls[0])
            calls[0] += 1
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return ranks.reduce([start.elapsed_time(stop)])[0]

    per_replay = max(elapsed(3) / 3, 1e-3)
    warm = max(1, math.ceil(warmup_s * 1e3 / per_replay))
    done = 0
    while done < warm:                                         # in slices, so that the host queue stays short
        n = min(warm - done, max(1, math.ceil(50.0 / per_replay)))
        elapsed(n)
        done += n
    per_replay = max(elapsed(3) / 3, 1e-3)
    replays = max(1, math.ceil(sample_ms / per_replay))
    samples = []
    t0 = time.perf_counter()
    for _ in range(trials):
        samples.append(elapsed(replays) / (replays * ops))
    t1 = time.perf_counter()
    clocks = sampler.window(t0, t1) if sampler is not None else None
    del graph
    return {"samples_ms": samples, "median_ms": statistics.median(samples), "min_ms": min(samples),
            "graph_operations": ops, "replays_per_sample": replays, "trials": trials,
            "launches": (3 + 3 + done + trials * replays) * ops, "timed_launches": trials * replays * ops,
            "timed_s": t1 - t0, "clocks": clocks}


def timing_plan(args, main):
    """(seconds of warm-up replays, samples, ms per sample): the reference harness's numbers for the workload the
    line is about, shorter for the other configurations; --capture shrinks everything for a profiler run."""
    if args.capture:
        return 0.02, 2, 2.0
    return (1.0, 9, 20.0) if main else (0.3, 5, 20.0)


def timing_note(r, warmup_s, sample_ms):
    return {"method": "CUDA graph replay, median of samples (the reference harness's method)",
            "graph_operations": r["graph_operations"], "warmup_s": warmup_s, "trials": r["trials"],
            "sample_ms": sample_ms, "replays_per_sample": r["replays_per_sample"],
            "samples_ms_per_step": [round(s, 6) for s in r["samples_ms"]], "min_ms_per_step": r["min_ms"]}


def tensor_roofline(flops_per_gpu, alg_bytes, ms_per_step, peaks, sustained, kernel, traffic):
    """Which roof bounds the launch (time at the tensor peak against time at the HBM peak) and the fraction reached."""
    per_gpu_tflops = flops_per_gpu / (ms_per_step * 1e-3) / 1e12
    gbs = alg_bytes / (ms_per_step * 1e-3) / 1e9
    bf16 = peaks["bf16_sustained"] if sustained else peaks["bf16_burst"]
    tensor_peak = 4.0 * bf16
    t_tensor = flops_per_gpu / (tensor_peak * 1e12)
    t_hbm = alg_bytes / (peaks["hbm_gbs"] * 1e9)
    if t_tensor >= t_hbm:
        roof = {"bound": "tensor", "achieved": per_gpu_tflops, "peak": tensor_peak, "unit": "TFLOP/s",
                "frac": per_gpu_tflops / tensor_peak,
                "peak_source": f"4 x {peaks['source']} cuBLAS bf16 ({'sustained' if sustained else 'burst'}): no FP4 peak is "
                               "measured on this pool; FP4 dense is 4x bf16 on the same pipe",
                "frac_of_4x_bf16_burst": per_gpu_tflops / (4.0 * peaks["bf16_burst"]),
                "frac_of_nominal_9pf": per_gpu_tflops / NOMINAL_FP4_TFLOPS}
    else:
        roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": gbs / peaks["hbm_gbs"], "peak_source": f"{peaks['source']} copy bandwidth"}
    roof["kernel"] = kernel
    roof["algorithmic_bytes_per_launch"] = alg_bytes
    roof["traffic"] = traffic
    roof["traffic_source"] = ("dram__bytes_read.sum + dram__bytes_write.sum of one launch in an ncu capture of this workload"
                              if traffic else None)
    return roof


# ---- the CPU arm: the reference's own CPU path on the box's host cores ------------------------------------

def host_threads():
    """All host cores, whatever OMP_NUM_THREADS the launcher exported (torchrun sets it to 1)."""
    import torch
    want = os.cpu_count() or 1
    if torch.get_num_threads() != want:
        torch.set_num_threads(want)
    return torch.get_num_threads()


def cpu_reference_pass(m, n, k, sigma_b, budget_s=20.0):
    """One pass of the reference's CPU path on a bounded sample: all of B against the first rows of A.

    With the reference's own Python present (oracle/_ref, written by oracle/make_ref.py) the timed code is its
    `dequantize` twice, `@` and `.half()` (reference/python/nvfp4.py:40-47, benchmarks/nvfp4.py:41) in torch on
    all host cores: kind "reference". Otherwise the numpy restatement in oracle/: kind "port".
    Returns (TFLOP/s, threads used, kind, description of the sample).
    """
    import numpy as np
    import torch
    from oracle import make_ref
    from oracle import nvfp4_oracle as O
    threads = host_threads()
    ref = make_ref.reference_python()
    torch.manual_seed(0)
    # about 0.03 TFLOP/s per core for the FP32 matmul plus the two dequantisations: size the A slab for `budget_s`
    rows = m
    est = (2.0 * m * n * k) / (0.03e12 * threads) + 4e-8 * (m + n) * k
    if est > budget_s:
        rows = max(128, int(m * budget_s / est) // 128 * 128)

    # Quantising 2 x 64M values on the CPU would take far longer than the timed pass itself, so a 1024-row
    # seeded block of each operand is quantised and repeated down the rows (whole scale atoms, so the
    # repeated arrays are valid operands with the same value distribution).
    def operand(r, sigma):
        base = min(r, 1024)
        x = torch.randn((base, k), dtype=torch.bfloat16).float() * sigma
        if ref is not None:
            p, s = ref["nvfp4"].quantize(x)
            p, s = p.numpy(), s.numpy()
        else:
            p, s = O.quantize(x.numpy())
        reps = -(-r // base)
        return np.tile(p, (reps, 1))[:r], np.tile(s, reps)[:r * k // 16]

    pa, sa = operand(rows, 1.0)
    pb, sb = operand(n, sigma_b)
    if ref is not None:
        ta, tsa, tb, tsb = (torch.from_numpy(np.ascontiguousarray(v)) for v in (pa, sa, pb, sb))
        deq = ref["nvfp4"].dequantize
        t0 = time.perf_counter()
        c = (deq(ta, tsa) @ deq(tb, tsb).T).half()
        dt = time.perf_counter() - t0
        kind, how = "reference", "reference/python/nvfp4.py dequantize x2 + torch FP32 matmul + .half()"
    else:
        t0 = time.perf_counter()
        c = O.gemm(pa, sa, pb, sb)
        dt = time.perf_counter() - t0
        kind, how = "port", "numpy restatement: dequantise x2 + FP32 matmul + FP16"
    assert tuple(c.shape) == (rows, n)
    return (2.0 * rows * n * k / dt / 1e12, threads, kind,
            f"rows 0..{rows - 1} of A against all of B ({rows}x{n}x{k}), {how}, {threads} threads, {dt:.2f} s")


def run_reference(args, rank, world):
    """`--impl reference`: rank 0 alone times the CPU path; the other ranks leave at once."""
    if rank != 0:
        return
    if args.workload not in GEMM_WORKLOADS:
        print(json.dumps({"impl": "reference", "unavailable": "the CPU reference arm times the GEMM workloads only"}))
        return
    m, n, k, sigma = GEMM_WORKLOADS[args.workload]
    warmup, steps = max(0, args.warmup), max(1, args.steps)
    # every step is a bounded sample of the workload; the whole run stays within about two minutes
    budget = min(20.0, max(1.0, 90.0 / (steps + warmup)))
    for _ in range(warmup):
        cpu_reference_pass(m, n, k, sigma, budget)
    values = []
    t0 = time.perf_counter()
    for _ in range(steps):
        v, threads, kind, sample = cpu_reference_pass(m, n, k, sigma, budget)
        values.append(v)
    dt = time.perf_counter() - t0
    value = statistics.median(values)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": 1e3 * dt / steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": {"workload": args.workload, "M": m, "N": n, "K": k, "layout": "TN",
                   "note": "host cores only: every step is a bounded sample of the workload (operands and inputs "
                           "generated outside the timed pass); value = median over the steps"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ---- GEMM workloads ------------------------------------------------------------------------------------------

def make_operand(g, rows, k, sigma, gen, dev):
    """Seeded bf16 N(0, sigma^2) [rows, k], quantised on the GPU in row chunks (keeps the FP32 temporary small)."""
    import torch
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty(rows * k // 16, dtype=torch.uint8, device=dev)
    chunk = max(128, min(rows, (1 << 26) // k // 128 * 128))
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        x = (torch.randn((r1 - r0, k), generator=gen, device=dev, dtype=torch.float32) * sigma).bfloat16()
        p, s = g.quantize(x)
        packed[r0:r1] = p
        scales[r0 * k // 16:r1 * k // 16] = s
    return packed, scales


def gemm_errors(c, ref):
    """(relative Frobenius error, max abs error / rms of the reference) of an FP16 result against FP32."""
    import torch
    c, ref = c.float(), ref.float()
    if torch.isnan(c).any():
        return float("nan"), float("nan")
    err = (c - ref).double()
    rel = float(err.norm() / ref.double().norm().clamp_min(1e-30))
    worst = float(err.abs().max() / ref.double().pow(2).mean().sqrt().clamp_min(1e-30))
    return rel, worst


def check_gemm(g, out, pa, sa, pb, sb, k, rank):
    """Sampled rows of this rank's C against the FP32 dequantise-then-matmul path (GPU, TF32 off: the check path
    built on the bit-exact dequantise kernel) and one block against the CPU oracle. Returns (ok, details)."""
    import numpy as np
    import torch
    from oracle import nvfp4_oracle as O
    torch.backends.cuda.matmul.allow_tf32 = False
    m, n_local = out.shape
    per_row = k // 16
    b_f32 = g.dequantize(pb, sb)
    details, ok = {}, True
    for r0 in sorted({0, (m // 128 - 1) * 128, (m // 256) * 128}):
        a_f32 = g.dequantize(pa[r0:r0 + 128], sa[r0 * per_row:(r0 + 128) * per_row])
        rel, worst = gemm_errors(out[r0:r0 + 128], a_f32 @ b_f32.T)
        good = rel <= REL_FROBENIUS and worst <= MAX_ABS_OVER_RMS
        ok &= good
        details[f"rows_{r0}_{r0 + 127}_vs_fp32_path"] = {"rel_frobenius": rel, "max_abs_over_rms": worst, "pass": bool(good)}
    del b_f32
    # CPU oracle (numpy restatement of the reference's dequantise + FP32 matmul) on one 128 x 1024 block
    r0, c0 = (m // 256) * 128, (n_local // 2048) * 1024
    cols = min(1024, n_local - c0)
    ref = O.gemm_f32(pa[r0:r0 + 128].cpu().numpy(), sa[r0 * per_row:(r0 + 128) * per_row].cpu().numpy(),
                     pb[c0:c0 + cols].cpu().numpy(), sb[c0 * per_row:(c0 + cols) * per_row].cpu().numpy())
    rel, worst = gemm_errors(out[r0:r0 + 128, c0:c0 + cols].cpu(), torch.from_numpy(np.asarray(ref)))
    good = rel <= REL_FROBENIUS and worst <= MAX_ABS_OVER_RMS
    ok &= good
    details[f"block_r{r0}_c{c0}_vs_cpu_oracle"] = {"rel_frobenius": rel, "max_abs_over_rms": worst, "pass": bool(good)}
    return bool(ok), details


def run_gemm(args, ranks: Ranks, workload, sampler, main, gathers=("none",)):
    """Times one GEMM workload on this process group; returns the result dict (on every rank)."""
    import torch
    import gpu_kernels_b200 as g
    from gpu_kernels_b200 import _lib

    rank, world = ranks.rank, ranks.world
    dev = torch.device("cuda", ranks.local_rank)
    m, n, k, sigma = GEMM_WORKLOADS[workload]
    lo, hi = g.slab_rows(n, world, rank)
    n_local = hi - lo
    lib = _lib.load()
    l2 = lib.gpu_kernels_nvfp4_l2_bytes()
    warmup_s, trials, sample_ms = timing_plan(args, main)

    # Seeded synthetic operands: A on every rank, this rank's row slab of B (drawn with a per-slab seed).
    gen = torch.Generator(device=dev).manual_seed(0)
    pa, sa = make_operand(g, m, k, 1.0, gen, dev)
    gen_b = torch.Generator(device=dev).manual_seed(1 + rank)
    pb, sb = make_operand(g, n_local, k, sigma, gen_b, dev)
    torch.cuda.empty_cache()

    # Operand rotation: consecutive steps read different copies, together larger than twice the L2.
    in_bytes = sum(t.numel() for t in (pa, sa, pb, sb))
    rotations = min(64, max(2, -(-2 * l2 // in_bytes)))
    sets = [(pa, sa, pb, sb)] + [tuple(t.clone() for t in (pa, sa, pb, sb)) for _ in range(rotations - 1)]
    plans = [g.Nvfp4Gemm(x[0], x[2], x[1], x[3]) for x in sets]
    for plan in plans:
        if args.l2_side in ("on", "off"):
            try:
                plan.set_option("l2_side", 1 if args.l2_side == "on" else 0)
            except RuntimeError:
                pass
        # four units per tile where the library offers it (a slab with far fewer tiles than SMs); this
        # process owns the GPU, which is what the option needs
        try:
            plan.set_option("split_k", 1)
        except RuntimeError:
            pass
    out = torch.empty((m, n_local), dtype=torch.float16, device=dev)
    flops = 2.0 * m * n * k
    peaks = measured_peaks()
    result = {"workload": workload, "M": m, "N": n, "K": k, "n_gpus": world,
              "sharding": f"B rows over {world} rank(s), {n_local} columns of C per rank",
              "l2": f"operand rotation over {rotations} copies ({rotations * in_bytes >> 20} MiB > 2 x L2 {l2 >> 20} MiB)"}

    def step(i):
        plans[i % rotations].run(out)

    # burst: W warm-up steps, then exactly K steps launched from the host, timed once
    if main:
        for i in range(max(3, args.warmup)):
            step(i)
        ranks.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(args.steps):
            step(i)
        stop.record()
        ranks.barrier()
        burst_ms = ranks.reduce([start.elapsed_time(stop)])[0] / args.steps
        result["burst"] = {"ms_per_step": burst_ms, "value": flops / (burst_ms * 1e-3) / 1e12, "unit": UNIT,
                           "steps": args.steps, "warmup": max(3, args.warmup),
                           "method": "one launch per step from the host, K steps timed once with CUDA events"}

    # Three ways a chain of launches may overlap (programmatic dependent launch; plan option "static_operands"):
    # 0 = a launch waits for the one in front of it before it touches memory (no promise about its operands);
    # 1 = B and its scales are weights that the launch in front does not write: their first tiles are fetched while
    #     that launch drains (the deployment this path is for: weights quantised once, activations made on the fly);
    # 2 = no operand is written by the launch in front (independent GEMMs): a launch computes while the last tiles
    #     of the one in front finish and only its stores of C wait.
    # All three are timed; `value` is mode 1, which is true of this workload by construction.
    chain = {}
    launches0 = _lib.launch_count()
    for mode, name in ((0, "dependent"), (2, "independent"), (1, "weights_static")):
        for plan in plans:
            plan.set_option("static_operands", mode)
        timed = time_replays(step, ranks, rotations, 10, warmup_s if mode == 1 else min(warmup_s, 0.3), trials, sample_ms, sampler)
        chain[name] = {"static_operands": mode, "ms_per_step": timed["median_ms"],
                       "value": flops / (timed["median_ms"] * 1e-3) / 1e12, "unit": UNIT,
                       "samples_ms_per_step": [round(v, 6) for v in timed["samples_ms"]]}
    plans[0].validate()
    ms = timed["median_ms"]
    info = plans[0].info()
    result.update({"ms_per_step": ms, "value": flops / (ms * 1e-3) / 1e12, "unit": UNIT,
                   "timing": timing_note(timed, warmup_s, sample_ms), "clocks": timed["clocks"], "chain": chain,
                   "gpu_launches": timed["timed_launches"], "launches_counted_by_library": int(_lib.launch_count() - launches0),
                   "plan": info})
    if info.get("l2_side"):
        result["placement_misses"] = plans[0].placement_misses()
    alg_bytes = algorithmic_bytes(m, n_local, k)
    kernel = f"nvfp4_gemm_kernel<{info['cta_group']},{info['tile_n']}>"
    result["roofline"] = tensor_roofline(flops / world, alg_bytes, ms, peaks, True, kernel,
                                         NCU_DRAM_BYTES_PER_LAUNCH.get(workload) if world == 1 else None)

    # The library bar on the same box in the same run: cuBLASLt's own NVFP4 matmul on the same operands,
    # timed by the same method.
    if world == 1 and not args.no_library_bar:
        try:
            ws = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
            lt_plans = [g.Nvfp4Gemm(x[0], x[2], x[1], x[3], workspace=ws) for x in sets]
            lt = time_replays(lambda i: lt_plans[i % rotations].run_cublaslt(out), ranks, rotations, 10, warmup_s, trials,
                              sample_ms, sampler)
            result["library_bar"] = {"name": "cuBLASLt NVFP4 matmul (VEC16_UE4M3), same operands, same run, same method",
                                     "ms_per_step": lt["median_ms"], "value": flops / (lt["median_ms"] * 1e-3) / 1e12,
                                     "unit": UNIT, "ours_over_library": lt["median_ms"] / ms, "clocks": lt["clocks"]}
            for p_ in lt_plans:
                p_.close()
            del ws
        except Exception as exc:                                  # the bar is informative only
            result["library_bar"] = {"name": "cuBLASLt NVFP4 matmul", "unavailable": str(exc)[:200]}

    # parity of what was timed: the last launch of operand set 0
    plans[0].run(out)
    torch.cuda.synchronize()
    ok, details = check_gemm(g, out, pa, sa, pb, sb, k, rank)
    parity = {"gemm_rank0_details": details}

    # N > 1: the full C on every rank, fused into the epilogue or by NCCL; both timed, and compared bit for bit
    gather_results = {}
    fulls = {}
    for mode in gathers:
        if world == 1 or mode == "none":
            continue
        if mode == "fused":
            shared = g.GatheredOutput(m, n, dev)
            objs = [g.ShardedNvfp4Gemm(x[0], x[1], x[2], x[3], split_k=True, gathered=shared) for x in sets]
            gstep = lambda i: objs[i % rotations].run(gather=True)
        else:
            objs, shared = None, None
            full = torch.empty((m, n), dtype=torch.float16, device=dev)

            def gstep(i):
                plans[i % rotations].run(out)
                return g.gather_columns(out, None, full)
        gt = time_replays(gstep, ranks, rotations, 10, warmup_s, trials, sample_ms, sampler)
        fulls[mode] = gstep(0).clone()
        torch.cuda.synchronize()
        ranks.barrier()
        # every rank sends its slab to the world - 1 others (and receives theirs)
        nvlink_bytes = 2 * m * n_local * (world - 1)
        gather_results[mode] = {"ms_per_step": gt["median_ms"], "value": flops / (gt["median_ms"] * 1e-3) / 1e12, "unit": UNIT,
                                "timing": timing_note(gt, warmup_s, sample_ms),
                                "nvlink_bytes_per_step_per_gpu_each_direction": nvlink_bytes,
                                "nvlink_gbs_if_spread_over_the_step": nvlink_bytes / (gt["median_ms"] * 1e-3) / 1e9,
                                "nvlink_frac_of_900_per_direction": nvlink_bytes / (gt["median_ms"] * 1e-3) / 1e9 / NVLINK_GBS_PER_DIRECTION}
        if objs is not None:
            for o in objs:
                o.validate()
                o.close()
            shared.close()
    if gather_results:
        result["gather"] = gather_results
    if "fused" in fulls and "nccl" in fulls:
        same = bool(torch.equal(fulls["fused"], fulls["nccl"]))
        parity["fused_gather_equals_nccl_gather_bitwise"] = same
        ok &= same
        mine = bool(torch.equal(fulls["nccl"][:, lo:hi], out))
        parity["gathered_slab_equals_local_slab"] = mine
        ok &= mine
    del fulls

    # End to end through the C ABI with HOST buffers: H2D of the operands, kernel, D2H of C, every step.
    if main or args.e2e_all:
        host = [t.cpu().pin_memory() for t in (pa, pb, sa, sb)]
        host_c = torch.empty((m, n_local), dtype=torch.float16).pin_memory()
        e2e_steps = max(3, min(args.steps, 10))
        g.gemm_host(*host, host_c)
        ranks.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(e2e_steps):
            g.gemm_host(*host, host_c)
        stop.record()
        ranks.barrier()
        e2e_ms = ranks.reduce([start.elapsed_time(stop)])[0] / e2e_steps
        same = bool(torch.equal(host_c, out.cpu()))
        parity["host_entry_point_equals_device_result"] = same
        ok &= same
        result["e2e"] = {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                         "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host),
                         "d2h_bytes_per_step": host_c.numel() * 2, "steps": e2e_steps,
                         "call": "gpu_kernels_nvfp4_gemm_host (pinned host buffers)"}
        del host, host_c

    all_ok = ranks.all_ok(ok)
    parity["pass_all_ranks"] = all_ok
    result["parity"] = parity
    for plan in plans:
        plan.close()
    del plans, sets, pa, sa, pb, sb, out
    torch.cuda.empty_cache()
    return result


# ---- stand-alone quantiser ---------------------------------------------------------------------------------------

def run_quantise(args, ranks: Ranks, workload, sampler, main):
    """One step = quantise one bf16 [rows, K] operand (different copies in turn, together larger than L2)."""
    import numpy as np
    import torch
    import gpu_kernels_b200 as g
    from gpu_kernels_b200 import _lib
    dev = torch.device("cuda", ranks.local_rank)
    rows, k = QUANT_WORKLOADS[workload]
    warmup_s, trials, sample_ms = timing_plan(args, main)
    copies = max(2, (512 << 20) // (rows * k * 2))
    gen = torch.Generator(device=dev).manual_seed(0)
    xs = []
    for _ in range(copies):
        x = torch.empty((rows, k), dtype=torch.bfloat16, device=dev)
        for r0 in range(0, rows, 4096):
            x[r0:r0 + 4096] = torch.randn((min(4096, rows - r0), k), generator=gen, device=dev).bfloat16()
        xs.append(x)
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty(rows * k // 16, dtype=torch.uint8, device=dev)
    lib = _lib.load()

    def step(i):
        _lib.check(lib.gpu_kernels_nvfp4_quantize(xs[i % copies].data_ptr(), 0, packed.data_ptr(), scales.data_ptr(), rows, k,
                                                  torch.cuda.current_stream().cuda_stream))

    timed = time_replays(step, ranks, copies, 10, warmup_s, trials, sample_ms, sampler)
    ms = timed["median_ms"]
    alg = rows * k * 2 + rows * k // 2 + rows * k // 16
    gbs = alg / (ms * 1e-3) / 1e9
    peaks = measured_peaks()
    # parity: bit-exact against the CPU oracle on sampled 128-row slabs of the last operand quantised
    from oracle import nvfp4_oracle as O
    step(0)
    torch.cuda.synchronize()
    ok = True
    for r0 in sorted({0, (rows // 256) * 128, rows - 128}):
        want_p, want_s = O.quantize(xs[0][r0:r0 + 128].float().cpu().numpy())
        got_p = packed[r0:r0 + 128].cpu().numpy()
        got_s = scales[r0 * k // 16:(r0 + 128) * k // 16].cpu().numpy()
        ok &= bool(np.array_equal(got_p, want_p) and np.array_equal(got_s, want_s))
    cpu = None
    if main and not args.no_cpu and ranks.rank == 0:
        # the same operand through the CPU restatement of the reference's quantiser (numpy, one thread),
        # on a bounded sample of its rows
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
    return {"workload": workload, "rows": rows, "K": k, "metric": "nvfp4_quantise_gbs", "value": gbs, "unit": "GB/s",
            "ms_per_step": ms, "n_gpus": 1, "timing": timing_note(timed, warmup_s, sample_ms), "clocks": timed["clocks"],
            "gpu_launches": timed["timed_launches"],
            "l2": f"{copies} input copies in turn ({copies * rows * k * 2 >> 20} MiB)",
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                         "peak_source": f"{peaks['source']} copy bandwidth", "kernel": "quantise_kernel<bf16>",
                         "algorithmic_bytes_per_launch": alg, "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(workload)},
            "cpu_baseline": cpu, "parity": {"bit_exact_vs_cpu_oracle_on_sampled_slabs": ok, "pass_all_ranks": ok}}


def run_mx(args, ranks: Ranks, workload, sampler, main):
    """One step = one MXFP4 GEMM (E2M1 values, UE8M0 scale per 32) on one GPU, timed like the NVFP4 GEMMs; checked on
    sampled rows and columns against the CPU oracle's dequantise-then-matmul of the stored bytes."""
    import numpy as np
    import torch
    import gpu_kernels_b200 as g
    from gpu_kernels_b200 import _lib
    from oracle import nvfp4_oracle as O
    dev = torch.device("cuda", ranks.local_rank)
    m, n, k, sigma = MX_WORKLOADS[workload]
    warmup_s, trials, sample_ms = timing_plan(args, main)
    l2 = _lib.load().gpu_kernels_nvfp4_l2_bytes()
    gen = torch.Generator(device=dev).manual_seed(7)

    def operand(rows, sd):
        x = torch.empty((rows, k), dtype=torch.bfloat16, device=dev)
        for r0 in range(0, rows, 4096):
            x[r0:r0 + 4096] = (torch.randn((min(4096, rows - r0), k), generator=gen, device=dev) * sd).bfloat16()
        return g.quantize_mx(x)

    pa, sa = operand(m, 1.0)
    pb, sb = operand(n, sigma)
    in_bytes = sum(t.numel() for t in (pa, sa, pb, sb))
    rotations = min(64, max(2, -(-2 * l2 // in_bytes)))
    sets = [(pa, sa, pb, sb)] + [tuple(t.clone() for t in (pa, sa, pb, sb)) for _ in range(rotations - 1)]
    plans = [g.Nvfp4Gemm(x[0], x[2], x[1], x[3], mx=True) for x in sets]
    for plan in plans:
        plan.set_option("static_operands", 1)
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device=dev)
    timed = time_replays(lambda i: plans[i % rotations].run(out), ranks, rotations, 10, warmup_s, trials, sample_ms, sampler)
    ms = timed["median_ms"]
    for plan in plans:
        plan.validate()
    flops = 2.0 * m * n * k
    alg = m * k // 2 + n * k // 2 + (m + n) * k // 32 + m * n * 2
    rows = sorted({0, 129, m // 2 + 5, m - 1})
    cols = sorted({0, 200, n // 2 + 77, n - 1})
    ra = O.dequantize_mx(pa.cpu().numpy(), sa.cpu().numpy())[rows]
    rb = O.dequantize_mx(pb.cpu().numpy(), sb.cpu().numpy())
    got = out.float().cpu().numpy()
    rel_r, worst_r = gemm_errors(torch.from_numpy(got[rows]), torch.from_numpy(ra @ rb.T))
    ra_all = O.dequantize_mx(pa.cpu().numpy(), sa.cpu().numpy())
    rel_c, worst_c = gemm_errors(torch.from_numpy(np.ascontiguousarray(got[:, cols])), torch.from_numpy(ra_all @ rb[cols].T))
    ok = bool(max(rel_r, rel_c) <= REL_FROBENIUS and max(worst_r, worst_c) <= MAX_ABS_OVER_RMS)
    info = plans[0].info()
    for plan in plans:
        plan.close()
    return {"workload": workload, "M": m, "N": n, "K": k, "metric": "mxfp4_gemm_tflops", "value": flops / (ms * 1e-3) / 1e12,
            "unit": UNIT, "ms_per_step": ms, "n_gpus": 1, "timing": timing_note(timed, warmup_s, sample_ms),
            "clocks": timed["clocks"], "gpu_launches": timed["timed_launches"],
            "plan": {k_: info[k_] for k_ in ("units", "cta_group", "tile_n", "stages")},
            "l2": f"operand rotation over {rotations} copies ({rotations * in_bytes >> 20} MiB > 2 x L2 {l2 >> 20} MiB)",
            "roofline": tensor_roofline(flops, alg, ms, measured_peaks(), True, "nvfp4_gemm_kernel<2,256,direct,mx>", None),
            "parity": {"checked": f"rows {rows} and columns {cols} of C against the CPU oracle (dequantize_mx, FP32 matmul); "
                                  "parity unpinned: the reference has no MXFP4",
                       "rel_frobenius": max(rel_r, rel_c), "max_abs_over_rms": max(worst_r, worst_c), "pass_all_ranks": ok}}


# ---- routed-MoE expert layer -------------------------------------------------------------------------------------

def expert_weights(e_global, dev):
    """bf16 W1 [2I, H] and W2 [H, I] of one expert, N(0, 0.02), from a seed of the expert's own: every rank can
    rebuild any expert (the parity check needs the experts a sampled token was routed to, wherever they live)."""
    import torch
    H, I = MOE_SHAPE["hidden"], MOE_SHAPE["inter"]
    gen = torch.Generator(device=dev).manual_seed(10_000 + e_global)
    w1 = (torch.randn((2 * I, H), generator=gen, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn((H, I), generator=gen, device=dev) * 0.02).bfloat16()
    return w1, w2


class MoeBench:
    """The expert layer of this rank (built once) and the measurements at several token counts."""

    def __init__(self, args, ranks: Ranks):
        import torch
        import gpu_kernels_b200 as g
        self.args, self.ranks, self.g = args, ranks, g
        self.dev = torch.device("cuda", ranks.local_rank)
        H, I, E, topk, clamp = (MOE_SHAPE[k] for k in ("hidden", "inter", "experts", "topk", "clamp"))
        self.local = E // ranks.world
        w1 = torch.empty((self.local, 2 * I, H), dtype=torch.bfloat16, device=self.dev)
        w2 = torch.empty((self.local, H, I), dtype=torch.bfloat16, device=self.dev)
        for e in range(self.local):                             # expert by expert: keeps the FP32 temporaries small
            w1[e], w2[e] = expert_weights(ranks.rank * self.local + e, self.dev)
        self.max_tokens = max(MOE_WORKLOADS.values())
        self.layer = g.Nvfp4MoE(w1, w2, E, topk, clamp=clamp, max_tokens=self.max_tokens)
        del w1, w2
        torch.cuda.empty_cache()

    def close(self):
        self.layer.close()                                      # collective (unmaps the peers' buffers): every rank

    def check_tokens(self, x, ids, wts, y, sample):
        """Sampled tokens of this rank against the CPU oracle (moe_forward_nvfp4_experts): the experts a token
        uses are rebuilt from their seeds, quantised and dequantised by the library's (bit-exact) kernels."""
        import numpy as np
        from oracle import moe_oracle as MO
        g = self.g
        H, I, clamp = MOE_SHAPE["hidden"], MOE_SHAPE["inter"], MOE_SHAPE["clamp"]
        cache = {}

        def expert(e):
            if e not in cache:
                w1, w2 = expert_weights(e, self.dev)
                cache[e] = (g.dequantize(*g.quantize(w1)).cpu().numpy(), g.dequantize(*g.quantize(w2)).cpu().numpy())
            return cache[e]

        ref = MO.moe_forward_nvfp4_experts(x[sample].float().cpu().numpy(), ids[sample].cpu().numpy(),
                                           wts[sample].cpu().numpy(), expert, clamp)
        got = y[sample].float().cpu().numpy().astype(np.float64)
        if np.isnan(got).any():
            return False, {"rel_frobenius": float("nan")}
        ref = ref.astype(np.float64)
        rel = float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30))
        worst = float(np.abs(got - ref).max() / max(np.sqrt((ref ** 2).mean()), 1e-30))
        ok = rel <= LAYER_REL_FROBENIUS and worst <= LAYER_MAX_ABS_OVER_RMS
        rms = float(np.sqrt((ref ** 2).mean()))
        ok = ok and rms > 0.0                                   # an all-zero reference would prove nothing
        return bool(ok), {"tokens_checked": len(sample), "experts_rebuilt": len(cache), "rel_frobenius": rel,
                          "max_abs_over_rms": worst, "bound": [LAYER_REL_FROBENIUS, LAYER_MAX_ABS_OVER_RMS],
                          "reference_rms": rms, "output_rms": float(np.sqrt((got ** 2).mean())),
                          "outputs_equal_to_the_oracle": float((got == ref).mean())}

    def run(self, workload, sampler, main):
        import torch
        g, ranks, layer, dev = self.g, self.ranks, self.layer, self.dev
        from gpu_kernels_b200 import _lib
        tokens = MOE_WORKLOADS[workload]
        H, I, E, topk = (MOE_SHAPE[k] for k in ("hidden", "inter", "experts", "topk"))
        world, rank, local = ranks.world, ranks.rank, self.local
        warmup_s, trials, sample_ms = timing_plan(self.args, main)
        gen = torch.Generator(device=dev).manual_seed(77 * tokens + rank)
        sets = []
        for _ in range(4):                                      # rotating inputs: routing changes every step
            x = torch.randn((tokens, H), generator=gen, device=dev).bfloat16()
            ids, wts = g.route(torch.randn((tokens, E), generator=gen, device=dev), topk)
            sets.append((x, ids.contiguous(), wts.contiguous().float()))

        def step(i):
            return layer(*sets[i % 4])

        timed = time_replays(step, ranks, 4, 8, warmup_s, trials, sample_ms, sampler)
        layer.check()
        ms = timed["median_ms"]
        # phase marks of one eager forward (device-bound: a filler keeps the host ahead of the device)
        filler = torch.empty(1 << 28, dtype=torch.uint8, device=dev)
        for _ in range(24):
            filler.zero_()
        layer.phase_events = []
        y = layer(*sets[0]).clone()
        phases = {k_: round(v_, 1) for k_, v_ in layer.phase_times_us().items()}
        layer.phase_events = None
        del filler
        launches_per_forward = None
        n0 = _lib.launch_count()
        layer(*sets[0])
        torch.cuda.synchronize()
        launches_per_forward = int(_lib.launch_count() - n0)
        touched = int((layer.counts_matrix.sum(0)[rank * local:(rank + 1) * local] > 0).sum().item())
        # parity on sampled tokens of every rank; the verdict is shared
        x0, ids0, wts0 = sets[0]
        sample = sorted({0, tokens - 1})
        ok, details = self.check_tokens(x0, ids0, wts0, y, sample)
        all_ok = ranks.all_ok(ok)
        ranks.barrier()

        routes = world * tokens * topk
        flops = routes * 2.0 * (2 * I * H + H * I)
        value = flops / (ms * 1e-3) / 1e12
        peaks = measured_peaks()
        weight_bytes = touched * (2 * I * H + H * I) * 9 // 16  # packed values + scale bytes of the experts this rank touched
        act_bytes = tokens * topk * (H // 2 + H // 16 + I // 2 + I // 16 + 2 * H * 2)
        alg_bytes = weight_bytes + act_bytes
        t_hbm = alg_bytes / (peaks["hbm_gbs"] * 1e9)
        tensor_peak = 4.0 * peaks["bf16_sustained"]
        t_tensor = (flops / world) / (tensor_peak * 1e12)
        note = "whole-step time (every kernel and exchange of the forward) against the work of the two grouped GEMMs"
        if t_hbm >= t_tensor:
            gbs = alg_bytes / (ms * 1e-3) / 1e9
            roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                        "peak_source": f"{peaks['source']} copy bandwidth", "traffic": None,
                        "algorithmic_bytes_per_step": alg_bytes, "kernel": "nvfp4_gemm_kernel grouped (FC1 + FC2)", "note": note}
        else:
            roofline = {"bound": "tensor", "achieved": value / world, "peak": tensor_peak, "unit": "TFLOP/s",
                        "frac": value / world / tensor_peak, "peak_source": f"4 x {peaks['source']} cuBLAS bf16 (sustained)",
                        "traffic": None, "kernel": "nvfp4_gemm_kernel grouped (FC1 + FC2)", "note": note}
        result = {"workload": workload, "metric": "nvfp4_moe_tflops", "value": value, "unit": UNIT, "ms_per_step": ms,
                  "n_gpus": world, "scaling": "weak", "tokens_per_gpu": tokens, **MOE_SHAPE, "expert_parallel": world,
                  "experts_touched_rank0": touched, "exchange": layer.exchange,
                  "launch": "CUDA graph of two passes over four input sets, replayed",
                  "timing": timing_note(timed, warmup_s, sample_ms), "clocks": timed["clocks"],
                  "gpu_launches": timed["timed_launches"] * (launches_per_forward or 1), "launches_per_forward": launches_per_forward,
                  "phases_us_rank0_eager": phases, "roofline": roofline,
                  "parity": {"sampled_tokens_vs_cpu_oracle_rank0": details, "pass_all_ranks": all_ok}}
        if world > 1:
            # rows that cross NVLink: a remote route sends one quantised row out and gets one bf16 row back
            remote = sum(int((s_[1] // local != rank).sum().item()) for s_ in sets) / len(sets)
            out_bytes = remote * (H // 2 + H // 16 + 16)
            in_bytes = remote * H * 2
            result["nvlink"] = {"remote_routes_per_step_rank0": remote, "dispatch_bytes_out_per_step": out_bytes,
                                "combine_bytes_in_per_step": in_bytes,
                                "gbs_if_spread_over_the_step": (out_bytes + in_bytes) / (ms * 1e-3) / 1e9,
                                "frac_of_900_per_direction": max(out_bytes, in_bytes) / (ms * 1e-3) / 1e9 / NVLINK_GBS_PER_DIRECTION}
        return result


def moe_e2e(bench: MoeBench, workload, steps):
    """The expert layer end to end: inputs from pinned host memory every step, result copied back to the host."""
    import torch
    g, ranks, layer, dev = bench.g, bench.ranks, bench.layer, bench.dev
    tokens = MOE_WORKLOADS[workload]
    H, E, topk, I = MOE_SHAPE["hidden"], MOE_SHAPE["experts"], MOE_SHAPE["topk"], MOE_SHAPE["inter"]
    gen = torch.Generator(device=dev).manual_seed(5 + ranks.rank)
    host = []
    for _ in range(4):
        x = torch.randn((tokens, H), generator=gen, device=dev).bfloat16()
        ids, wts = g.route(torch.randn((tokens, E), generator=gen, device=dev), topk)
        host.append(tuple(t.cpu().pin_memory() for t in (x, ids, wts.float())))
    y_host = torch.empty((tokens, H), dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(steps, 10))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one(i):
        xs = [t.to(dev, non_blocking=True) for t in host[i % 4]]
        y_host.copy_(layer(*xs), non_blocking=True)

    one(0)
    ranks.barrier()
    start.record()
    for i in range(e2e_steps):
        one(i)
    stop.record()
    ranks.barrier()
    ms = ranks.reduce([start.elapsed_time(stop)])[0] / e2e_steps
    flops = ranks.world * tokens * topk * 2.0 * (2 * I * H + H * I)
    return {"value": flops / (ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms,
            "h2d_bytes_per_step": tokens * (H * 2 + topk * 12), "d2h_bytes_per_step": tokens * H * 2, "steps": e2e_steps,
            "call": "Nvfp4MoE.forward on tensors copied from pinned host memory, result copied back"}


def run_ours(args, rank, world, local_rank):
    import torch
    torch.cuda.set_device(local_rank)
    ranks = Ranks(rank, world, local_rank)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    wl = args.workload
    configs, failed = [], False
    moe = None
    try:
        # ---- the workload the line is about ----
        if wl in GEMM_WORKLOADS:
            gathers = ("fused", "nccl") if args.gather == "auto" else (args.gather,)
            head = run_gemm(args, ranks, wl, sampler, True, gathers if world > 1 else ("none",))
            if world == 1 and not args.no_cpu and rank == 0:
                m, n, k, sigma = GEMM_WORKLOADS[wl]
                v, threads, kind, sample = cpu_reference_pass(m, n, k, sigma, 15.0)
                head["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample}
        elif wl in QUANT_WORKLOADS:
            if world > 1:
                raise SystemExit("the quantiser workloads run on one GPU")
            head = run_quantise(args, ranks, wl, sampler, True)
        elif wl in MX_WORKLOADS:
            if world > 1:
                raise SystemExit("the MXFP4 workload runs on one GPU")
            head = run_mx(args, ranks, wl, sampler, True)
        else:
            moe = MoeBench(args, ranks)
            head = moe.run(wl, sampler, True)
            head["e2e"] = moe_e2e(moe, wl, args.steps)
        # ---- the other configurations of the path, shorter warm-up ----
        if not args.only:
            order = [w for w in ("gemm16384", "skinny") if w != wl]
            if world == 1:
                order += [w for w in ("quantise8192", "mxfp4_gemm8192") if w != wl]
            order += [w for w in MOE_WORKLOADS if w != wl]
            for name in order:
                t0 = time.perf_counter()
                try:
                    if name in GEMM_WORKLOADS:
                        gathers = ("fused", "nccl") if name == "skinny" else ("none",)
                        r = run_gemm(args, ranks, name, sampler, False, gathers if world > 1 else ("none",))
                    elif name in QUANT_WORKLOADS:
                        r = run_quantise(args, ranks, name, sampler, False)
                    elif name in MX_WORKLOADS:
                        r = run_mx(args, ranks, name, sampler, False)
                    else:
                        if moe is None:
                            moe = MoeBench(args, ranks)
                        r = moe.run(name, sampler, False)
                except Exception as exc:                          # reported, and counted as a failure of the run
                    r = {"workload": name, "error": f"{type(exc).__name__}: {str(exc)[:300]}"}
                r["wall_s"] = round(time.perf_counter() - t0, 1)
                configs.append(r)
    finally:
        if moe is not None:
            moe.close()
        if sampler is not None:
            sampler.stop()
    everything = [head] + configs
    failed = any("error" in r or not r.get("parity", {}).get("pass_all_ranks", False) for r in everything)
    if rank == 0:
        line = {
            "metric": head.get("metric", METRIC), "value": head["value"], "unit": head["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": head.get("scaling", "strong"), "vs_baseline": None,
            "dtype": DTYPE if wl in GEMM_WORKLOADS else ("bf16 in, e2m1 + ue4m3 out" if wl in QUANT_WORKLOADS
                                                         else "nvfp4 operands, f32 accumulate, bf16 activations and output"),
            "data": "synthetic",
            "config": {k_: head[k_] for k_ in ("workload", "M", "N", "K", "rows", "sharding", "l2", "plan", "tokens_per_gpu",
                                               "hidden", "inter", "experts", "topk", "clamp", "expert_parallel", "exchange", "launch")
                       if k_ in head},
            "timing": head["timing"], "chain": head.get("chain"), "burst": head.get("burst"), "clocks": head["clocks"],
            "e2e": head.get("e2e"), "gpu_launches": head["gpu_launches"], "roofline": head["roofline"],
            "cpu_baseline": head.get("cpu_baseline"), "library_bar": head.get("library_bar"),
            "gather": head.get("gather"), "nvlink": head.get("nvlink"), "placement_misses": head.get("placement_misses"),
            "parity": {**head["parity"], "configs": {r["workload"]: r.get("parity", {}).get("pass_all_ranks", False) for r in configs},
                       "all": "pass" if not failed else "FAIL"},
            "configs": configs,
        }
        line["config"]["layout"] = "TN"
        if wl in GEMM_WORKLOADS:
            line["config"]["chain"] = ("launches carry the programmatic stream-serialisation attribute; B and its scales are declared "
                                       "static weights (plan option static_operands = 1), so a launch fetches its first B tiles while "
                                       "the launch in front drains; `chain` holds the same measurement without that promise and "
                                       "with all operands static")
        line["config"]["launch"] = line["config"].get("launch", "CUDA graph of one or more passes over the operand copies, replayed")
        print(json.dumps(line))
    return 1 if failed else 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20, help="steps of the burst leg (host launches, timed once)")
    ap.add_argument("--warmup", type=int, default=5, help="warm-up steps before the burst leg")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gemm8192",
                    choices=sorted(GEMM_WORKLOADS) + sorted(MOE_WORKLOADS) + sorted(QUANT_WORKLOADS) + sorted(MX_WORKLOADS))
    ap.add_argument("--only", action="store_true", help="measure the named workload only (no `configs`)")
    ap.add_argument("--gather", default="auto", choices=["auto", "none", "fused", "nccl"],
                    help="N>1, GEMM workloads: also time the step that leaves the full C on every rank: 'fused' = the GEMM's "
                         "epilogue stores the slab into all ranks' buffers over NVLink + a barrier kernel; 'nccl' = all-gather "
                         "+ strided copy; auto = both (and compared bit for bit)")
    ap.add_argument("--l2-side", default="auto", choices=["auto", "on", "off"],
                    help="tile order of the dense GEMM: the plan's default, or force the L2-side-aware order on / off")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-library-bar", action="store_true", help="skip the cuBLASLt comparison leg")
    ap.add_argument("--capture", action="store_true",
                    help="a few launches only (for a run under a profiler; the numbers it prints mean nothing)")
    ap.add_argument("--e2e-all", action="store_true", help="measure the host-buffer entry point for every GEMM config")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return 0
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        from datetime import timedelta
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=timedelta(seconds=180))
    try:
        return run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
