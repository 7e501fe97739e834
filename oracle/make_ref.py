"""Recipe for the two git-ignored mirrors of the reference's own Python files. TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py [REFERENCE_CHECKOUT]

Nothing of the reference is committed here; this script copies, from a checkout of the reference, exactly the
files that are run UNMODIFIED next to this repository's code:

  oracle/_ref/reference/python/{__init__,nvfp4,moe}.py
      the reference's CPU statement of the path (quantize, dequantize, moe_forward). Used to pin the numpy
      oracle and as the timed CPU baseline of bench.py (`cpu_baseline.kind` = "reference").
  baseline/_ref/benchmarks/{run,common,nvfp4}.py + baseline/_ref/reference/python/*.py + baseline/_ref/build/
      the reference's benchmark harness (benchmarks/run.py:38-79, benchmarks/common.py, benchmarks/nvfp4.py),
      laid out as it expects (benchmarks/common.py:14-20 loads ROOT/build/libgpu_kernels_nvfp4_bench.so); the
      build directory holds a link to THIS repository's library, so `python baseline/_ref/benchmarks/run.py
      nvfp4 --test` runs the reference's own correctness and timing code against this library.

Both folders travel to a GPU box with the working tree but stay out of the history. Without a reference
checkout the script does nothing and returns False; callers then fall back to the numpy oracle.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
# a checkout named `reference` beside this repository, unless GPU_KERNELS_REFERENCE names another place
DEFAULT_REFERENCE = Path(os.environ.get("GPU_KERNELS_REFERENCE", str(ROOT.parent / "reference")))

PYTHON_FILES = ("reference/python/__init__.py", "reference/python/nvfp4.py", "reference/python/moe.py")
HARNESS_FILES = ("benchmarks/run.py", "benchmarks/common.py", "benchmarks/nvfp4.py")


def _copy(src_root: Path, rel: str, dst_root: Path) -> None:
    dst = dst_root / rel
    dst.parent.mkdir(parents=True, exist_ok=True)
    shutil.copyfile(src_root / rel, dst)


def make(reference: Path | None = None) -> bool:
    reference = Path(reference) if reference else DEFAULT_REFERENCE
    if not all((reference / rel).exists() for rel in PYTHON_FILES + HARNESS_FILES):
        return False
    oracle_ref, harness = ROOT / "oracle" / "_ref", ROOT / "baseline" / "_ref"
    for rel in PYTHON_FILES:
        _copy(reference, rel, oracle_ref)
        _copy(reference, rel, harness)
    for rel in HARNESS_FILES:
        _copy(reference, rel, harness)
    build = harness / "build"
    build.mkdir(parents=True, exist_ok=True)
    link = build / "libgpu_kernels_nvfp4_bench.so"
    if link.is_symlink() or link.exists():
        link.unlink()
    # relative, so that the link still resolves where the tree is copied to
    link.symlink_to(Path("..") / ".." / ".." / "build" / "libgpu_kernels_nvfp4_bench.so")
    return True


def reference_python():
    """The reference's `reference.python.nvfp4` / `.moe` modules from oracle/_ref, or None when absent."""
    base = ROOT / "oracle" / "_ref"
    if not (base / "reference" / "python" / "nvfp4.py").exists():
        return None
    import importlib.util
    mods = {}
    for name in ("nvfp4", "moe"):
        spec = importlib.util.spec_from_file_location(f"_reference_python_{name}", base / "reference" / "python" / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods


if __name__ == "__main__":
    ok = make(Path(sys.argv[1]) if len(sys.argv) > 1 else None)
    print("mirrors written" if ok else "no reference checkout found: nothing written")
