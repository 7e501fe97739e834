"""The shared library loads without a GPU and exports every symbol the headers declare."""
import ctypes
import re

import pytest

from conftest import ROOT


@pytest.fixture(scope="module")
def lib():
    from gpu_kernels_b200 import build
    return ctypes.CDLL(str(build.build()))


def declared_symbols():
    text = (ROOT / "include" / "nvfp4_capi.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gpu_kernels_nvfp4_\w+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = declared_symbols()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), name


def test_binding_table_matches_header():
    from gpu_kernels_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_reference_harness_symbols_present(lib):
    # the seven names the reference's benchmarks/nvfp4.py:21-28 binds
    for name in ("last_error", "plan_create", "plan_destroy", "cublas", "custom", "validate", "l2_bytes"):
        assert hasattr(lib, "gpu_kernels_nvfp4_" + name)


def test_fails_loudly_without_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    lib.gpu_kernels_nvfp4_last_error.restype = ctypes.c_char_p
    plan = ctypes.c_void_p()
    rc = lib.gpu_kernels_nvfp4_plan_create(ctypes.byref(plan), 256, 256, 256, None, None, None, None, None,
                                           ctypes.c_size_t(0), None)
    assert rc == 1 and lib.gpu_kernels_nvfp4_last_error()
    rc = lib.gpu_kernels_nvfp4_quantize(None, 0, None, None, 128, 64, None)
    assert rc == 1


def test_host_layer_rejects_cpu_tensors():
    import torch
    import gpu_kernels_b200 as g
    with pytest.raises(ValueError):
        g.quantize(torch.zeros(128, 64))
    with pytest.raises(ValueError):
        g.Nvfp4Gemm(*(torch.zeros(128, 128, dtype=torch.uint8),) * 2, *(torch.zeros(2048, dtype=torch.uint8),) * 2)


BRIDGE_LIKE_CONSUMER = r"""
// What a host written against the reference's include/nvfp4.h does with it (benchmarks/bindings/
// nvfp4_bridge.cu:19-21, 83-85, 115 in the reference): value-initialise the params, fetch the
// implementation, call prepare / launch / validate through the function pointers.
#include "nvfp4.h"
#include "nvfp4_capi.h"
struct Plan {
    gpu_kernels::Nvfp4Params params{};
    gpu_kernels::Nvfp4Implementation impl{};
};
int run(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, __half* c, int m, int n, int k,
        cudaStream_t stream) {
    Plan plan;
    plan.impl = gpu_kernels::nvfp4_sm100_implementation();
    plan.impl.prepare(plan.params, a, b, sfa, sfb, m, n, k, stream);
    plan.impl.launch(plan.params, c, stream);
    plan.impl.validate();
    static_assert(offsetof(gpu_kernels::Nvfp4Params, A) == 0, "the tensor maps lead the struct");
    static_assert(offsetof(gpu_kernels::Nvfp4Params, M) == 4 * sizeof(CUtensorMap), "then M, N, K, clusters");
    return plan.params.M + plan.params.N + plan.params.K + plan.params.clusters + gpu_kernels_nvfp4_l2_bytes();
}
"""


def test_headers_compile_for_a_reference_style_host(tmp_path):
    import shutil
    import subprocess
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    src = tmp_path / "consumer.cu"
    src.write_text("#include <cstddef>\n" + BRIDGE_LIKE_CONSUMER)
    done = subprocess.run([nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(ROOT / "include"),
                           "-c", str(src), "-o", str(tmp_path / "consumer.o")], capture_output=True, text=True)
    assert done.returncode == 0, done.stderr
