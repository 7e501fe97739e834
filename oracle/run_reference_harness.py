"""Runs the reference's own benchmark harness, unmodified, against this repository's library.

    python oracle/run_reference_harness.py --test                 # its correctness cases (256^3, 2048x4096x2048)
    python oracle/run_reference_harness.py --suite b200 [--out DIR]  # its timing of `custom` against cuBLASLt

The harness files are the mirror written by oracle/make_ref.py under baseline/_ref (never committed): the
reference's benchmarks/run.py, benchmarks/common.py, benchmarks/nvfp4.py and its reference/python package. Its
common.py loads ROOT/build/libgpu_kernels_nvfp4_bench.so (benchmarks/common.py:19-20), which in the mirror is
this repository's library; it binds the seven plan symbols (benchmarks/nvfp4.py:21-28), quantises with its own
PyTorch quantiser, pre-fills the output with NaN, rotates operand copies larger than twice the L2, checks
`assert_close(atol = rtol = 2e-3)` against its FP32 dequantise-then-matmul and, in timing mode, replays CUDA
graphs of ten launches (one second of warm-up, nine samples of 20 ms, backends in alternating order, median)
and writes its six-column report (benchmarks/common.py:118-153). Needs a B200. TEST INFRASTRUCTURE ONLY.
"""
from __future__ import annotations

import argparse
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
MIRROR = ROOT / "baseline" / "_ref"
LIB = ROOT / "build" / "libgpu_kernels_nvfp4_bench.so"


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--test", action="store_true")
    ap.add_argument("--suite", default="b200", choices=["quick", "b200"])
    ap.add_argument("--out", default=None, help="copy the harness's report files (profiles/runtime/nvfp4.*) here")
    args = ap.parse_args()
    runner = MIRROR / "benchmarks" / "run.py"
    if not runner.exists():
        print("baseline/_ref is missing: run `python oracle/make_ref.py <reference checkout>` first")
        return 2
    if not LIB.exists():
        print(f"{LIB} is missing: build it with `python -m gpu_kernels_b200.build`")
        return 2
    target = MIRROR / "build" / LIB.name
    if not target.exists():                                     # a link that did not survive a copy of the tree
        target.parent.mkdir(parents=True, exist_ok=True)
        if target.is_symlink():
            target.unlink()
        shutil.copyfile(LIB, target)
    cmd = [sys.executable, str(runner), "nvfp4"]
    cmd += ["--test"] if args.test else ["--suite", args.suite, "--reference", "cublaslt"]
    print("+", " ".join(cmd), flush=True)
    rc = subprocess.run(cmd, cwd=str(MIRROR / "benchmarks")).returncode
    if rc == 0 and not args.test and args.out:
        out = Path(args.out)
        out.mkdir(parents=True, exist_ok=True)
        for f in (MIRROR / "profiles" / "runtime").glob("nvfp4*"):
            shutil.copyfile(f, out / ("reference_harness_" + f.name))
    return rc


if __name__ == "__main__":
    sys.exit(main())
