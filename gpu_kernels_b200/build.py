"""Build the sm_100a shared library in-tree with nvcc (no JIT cache, no pip install).

    python -m gpu_kernels_b200.build          # builds build/libgpu_kernels_nvfp4_bench.so

The output name and directory are the ones the reference's Python harness loads
(benchmarks/common.py:19-20), so the same file serves both this package and that
harness.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
CSRC = ROOT / "gpu_kernels_b200" / "csrc"
OUT_DIR = ROOT / "build"
LIB_NAME = "libgpu_kernels_nvfp4_bench.so"
SOURCES = ("nvfp4_quant.cu", "nvfp4_gemm.cu", "nvfp4_schedule.cu", "nvfp4_moe.cu", "nvfp4_capi.cu")
ARCH = ("-gencode", "arch=compute_100a,code=sm_100a")


def _nvcc() -> str:
    nvcc = os.environ.get("CUDACXX") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; set CUDACXX")
    return nvcc


def _digest() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*")) + list((ROOT / "include").glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def library_path() -> Path:
    return OUT_DIR / LIB_NAME


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a into one shared library; returns its path."""
    OUT_DIR.mkdir(exist_ok=True)
    lib, stamp = library_path(), OUT_DIR / (LIB_NAME + ".sha256")
    digest = _digest()
    if not force and lib.exists() and stamp.exists() and stamp.read_text() == digest:
        return lib
    nvcc = _nvcc()

    def compile_one(src: str):
        obj = OUT_DIR / (src + ".o")
        cmd = [nvcc, "-std=c++17", "-O3", *ARCH, "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
               "-I", str(ROOT / "include"), "-I", str(CSRC), "-c", str(CSRC / src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, r

    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 1)) as pool:
        results = list(pool.map(compile_one, SOURCES))
    objects = []
    for src, obj, r in results:
        if verbose or r.returncode:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode:
            raise RuntimeError(f"nvcc failed on {src}")
        (OUT_DIR / (src + ".ptxas.txt")).write_text(r.stderr)
        objects.append(str(obj))
    cmd = [nvcc, "-shared", *ARCH, "-o", str(lib), *objects, "-lcublasLt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    stamp.write_text(digest)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
