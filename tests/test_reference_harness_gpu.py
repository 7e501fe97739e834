"""The reference's own benchmark harness (benchmarks/run.py nvfp4 --test), unmodified, against this library.

The harness files are a git-ignored mirror written by oracle/make_ref.py from a checkout of the reference; where
the mirror is absent (a machine that never saw the reference) the test is skipped. The harness loads
build/libgpu_kernels_nvfp4_bench.so through its own ctypes binding (benchmarks/nvfp4.py:21-28), quantises with
its own PyTorch quantiser, pre-fills C with NaN and checks `assert_close(atol = rtol = 2e-3)` against its FP32
dequantise-then-matmul at 256^3 and 2048 x 4096 x 2048 (benchmarks/nvfp4.py:29-31, 69-70), then calls
`validate`. Passing is the drop-in claim itself."""
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_reference_harness_correctness_cases_pass():
    if not (ROOT / "baseline" / "_ref" / "benchmarks" / "run.py").exists():
        pytest.skip("no mirror of the reference's harness here (oracle/make_ref.py needs a reference checkout)")
    r = subprocess.run([sys.executable, str(ROOT / "oracle" / "run_reference_harness.py"), "--test"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "nvfp4: 2 correctness checks passed" in r.stdout, r.stdout[-2000:]
