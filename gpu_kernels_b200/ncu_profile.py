"""Nsight Compute driver for the kernels of this path: capture one launch, print the counters that matter.

The counterpart of the reference's scripts/profile.sh + scripts/extract_ncu.py (which cover its FP32/BF16 GEMMs and
FlashAttention, not NVFP4): run a workload of bench.py plainly, then the same command under `ncu` for ONE kernel
and a few launches, then read the report back as a short table (duration, DRAM bytes and utilisation, FP4 tensor
pipe, L2 -> SM sectors, registers, issue rate, the top warp stalls).

    python -m gpu_kernels_b200.ncu_profile --workload gemm8192 --kernel nvfp4_gemm_kernel --skip 30 --out prof/gemm8192
    python -m gpu_kernels_b200.ncu_profile --workload moe_t1024 --kernel quantise_route --skip 2 --out prof/dispatch
    python -m gpu_kernels_b200.ncu_profile --extract prof/gemm8192.ncu-rep          # no GPU needed

Rules the capture follows: the plain run must exit 0 first (a program that faults is not profiled); the clocks
are left alone (`--clock-control none`: a number printed under ncu is never a benchmark value, and a locked clock
would outlive the run); one kernel name, at most three launches, the small `--capture` mode of bench.py.
"""
from __future__ import annotations

import argparse
import csv
import io
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

# metric -> label; every name is looked up as given and skipped when the report does not have it
METRICS = [
    ("gpu__time_duration.sum", "duration"),
    ("launch__grid_size", "grid"),
    ("launch__block_size", "block"),
    ("launch__registers_per_thread", "registers / thread"),
    ("launch__shared_mem_per_block_dynamic", "dynamic shared memory / block"),
    ("dram__bytes_read.sum", "DRAM read"),
    ("dram__bytes_write.sum", "DRAM written"),
    ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed", "DRAM throughput, % of peak"),
    ("sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed", "tensor pipe active, % of elapsed"),
    ("sm__ops_path_tensor_op_utcomma_src_fp4_dst_fp32_sparsity_off.avg.pct_of_peak_sustained_elapsed",
     "FP4 tensor ops, % of peak"),
    ("lts__t_sectors_srcunit_tex_op_read.sum", "L2 -> SM read sectors (32 B)"),
    ("lts__t_sector_hit_rate.pct", "L2 hit rate"),
    ("sm__warps_active.avg.pct_of_peak_sustained_active", "warps active, % of peak"),
    ("smsp__issue_active.avg.pct_of_peak_sustained_active", "issue slots busy"),
    ("smsp__inst_executed.sum", "warp instructions"),
    ("sm__cycles_elapsed.max", "SM cycles elapsed"),
    ("sm__cycles_elapsed.avg.per_second", "SM clock"),
]
STALL_PREFIX = "smsp__average_warps_issue_stalled_"
STALL_SUFFIX = "_per_issue_active.ratio"


def read_raw_csv(text: str) -> list[dict]:
    """`ncu --page raw --csv` output -> one dict {metric: (value, unit)} per captured launch."""
    rows = list(csv.reader(io.StringIO(text)))
    head = next((i for i, r in enumerate(rows) if r and r[0] == "ID"), None)
    if head is None or len(rows) < head + 3:
        return []
    names, units = rows[head], rows[head + 1]
    out = []
    for r in rows[head + 2:]:
        if len(r) != len(names):
            continue
        out.append({n: (v, u) for n, v, u in zip(names, r, units)})
    return out


def summarise(launch: dict, top_stalls: int = 4) -> list[tuple[str, str]]:
    lines = []
    if "Kernel Name" in launch:
        lines.append(("kernel", launch["Kernel Name"][0][:110]))
    for metric, label in METRICS:
        if metric in launch and launch[metric][0] != "":
            value, unit = launch[metric]
            lines.append((label, f"{value} {unit}".strip()))
    stalls = []
    for name, (value, _) in launch.items():
        if name.startswith(STALL_PREFIX) and name.endswith(STALL_SUFFIX):
            try:
                stalls.append((float(value.replace(",", "")), name[len(STALL_PREFIX):-len(STALL_SUFFIX)]))
            except ValueError:
                pass
    stalls = [s for s in sorted(stalls, reverse=True) if s[1] != "selected"][:top_stalls]
    if stalls:
        lines.append(("top warp stalls per issue", ", ".join(f"{n} {v:.1f}" for v, n in stalls)))
    return lines


def extract(report: Path) -> int:
    ncu = shutil.which("ncu")
    if not ncu:
        print("ncu not found on PATH")
        return 2
    text = subprocess.run([ncu, "-i", str(report), "--page", "raw", "--csv"], capture_output=True, text=True).stdout
    launches = read_raw_csv(text)
    if not launches:
        print(f"no launches in {report}")
        return 1
    for i, launch in enumerate(launches):
        print(f"\n| launch {i} | |\n|---|---|")
        for label, value in summarise(launch):
            print(f"| {label} | {value} |")
    return 0


def capture(args) -> int:
    ncu = shutil.which("ncu")
    if not ncu:
        print("ncu not found on PATH")
        return 2
    out = Path(args.out)
    out.parent.mkdir(parents=True, exist_ok=True)
    cmd = [sys.executable, str(ROOT / "bench.py"), "--only", "--no-cpu", "--no-library-bar", "--capture",
           "--workload", args.workload]
    print("+", " ".join(cmd), flush=True)
    plain = subprocess.run(cmd, capture_output=True, text=True)
    if plain.returncode != 0:
        print(plain.stdout[-2000:], plain.stderr[-2000:])
        print("the plain run failed: not profiled")
        return 1
    prof = [ncu, "--clock-control", "none", "-k", f"regex:{args.kernel}", "-s", str(args.skip), "-c", str(min(3, args.count)),
            "-f", "-o", str(out)]
    prof += ["--set", "full"] if args.set == "full" else ["--section", "SpeedOfLight", "--section", "MemoryWorkloadAnalysis",
                                                         "--section", "LaunchStats", "--section", "WarpStateStats"]
    print("+", " ".join(prof + cmd), flush=True)
    rc = subprocess.run(prof + cmd, capture_output=True, text=True).returncode
    if rc != 0:
        print(f"ncu exited with {rc}")
        return rc
    return extract(out.with_suffix(".ncu-rep") if out.suffix != ".ncu-rep" else out)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--extract", default=None, help="an existing .ncu-rep: print its summary and exit")
    ap.add_argument("--workload", default="gemm8192", help="a --workload of bench.py")
    ap.add_argument("--kernel", default="nvfp4_gemm_kernel", help="regular expression of the kernel name")
    ap.add_argument("--skip", type=int, default=4, help="launches of that kernel to skip first")
    ap.add_argument("--count", type=int, default=1, help="launches to capture (at most 3)")
    ap.add_argument("--set", default="full", choices=["full", "light"], help="full: about 40 passes per launch; light: four sections")
    ap.add_argument("--out", default="ncu_out/profile", help="report path (without .ncu-rep)")
    args = ap.parse_args()
    if args.extract:
        return extract(Path(args.extract))
    return capture(args)


if __name__ == "__main__":
    sys.exit(main())
