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
