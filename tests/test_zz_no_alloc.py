"""The allocation-free host GEMM entry point against the allocating one.

`gpu_kernels_nvfp4_gemm_host_static` exists for hosts that may not call cudaMalloc while they run
(their memory pool owns the GPU, or they are in a phase where allocation is forbidden): its device
staging is an array built into the library. It must give the same bytes as
`gpu_kernels_nvfp4_gemm_host` on every call, including a second call that finds the previous call's
data in the shared array. This file is collected last on purpose, and also passes on its own.
"""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from helpers import assert_gemm_close

pytestmark = pytest.mark.gpu


def host_operands(m, n, k, seed):
    rng = np.random.default_rng(seed)
    pa, sa = O.quantize(rng.standard_normal((m, k)).astype(np.float32))
    pb, sb = O.quantize((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    return [torch.from_numpy(t) for t in (pa, pb, sa, sb)]


def run(name, m, n, k, ops, alpha=1.0):
    from gpu_kernels_b200 import _lib
    out = torch.full((m, n), float("nan"), dtype=torch.float16)
    fn = getattr(_lib.load(), name)
    _lib.check(fn(m, n, k, ops[0].data_ptr(), ops[1].data_ptr(), ops[2].data_ptr(), ops[3].data_ptr(),
                  out.data_ptr(), float(alpha), None))
    return out


def test_static_matches_allocating_entry_point_twice_in_a_row():
    assert torch.cuda.is_available()
    # two calls in a row with different shapes and data: the second finds the first one's bytes in the array
    for seed, (m, n, k), alpha in ((1, (256, 384, 512), 1.0), (2, (128, 1024, 2048), 0.5), (3, (512, 256, 256), 1.0)):
        ops = host_operands(m, n, k, seed)
        got = run("gpu_kernels_nvfp4_gemm_host_static", m, n, k, ops, alpha)
        want = run("gpu_kernels_nvfp4_gemm_host", m, n, k, ops, alpha)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"{m}x{n}x{k}: outputs differ"
        ref = O.gemm_f32(*(ops[i].numpy() for i in (0, 2, 1, 3))) * np.float32(alpha)
        assert_gemm_close(got, ref, f"static entry point {m}x{n}x{k}")


def test_static_rejects_shapes_beyond_its_array():
    from gpu_kernels_b200 import _lib
    z = torch.zeros(16, dtype=torch.uint8)
    out = torch.zeros(16, dtype=torch.float16)
    for m, n, k in ((640, 256, 256), (128, 1152, 256), (128, 128, 2304)):
        with pytest.raises(_lib.Nvfp4Error, match="exceeds the built-in staging"):
            _lib.check(_lib.load().gpu_kernels_nvfp4_gemm_host_static(
                m, n, k, z.data_ptr(), z.data_ptr(), z.data_ptr(), z.data_ptr(), out.data_ptr(), 1.0, None))


def test_static_entry_point_leaves_device_memory_alone():
    # what the entry point is for: once a shape has been through it (the first call on a device takes the
    # array's address, and the first launch of a kernel variant lets the driver load that kernel), further
    # calls neither take nor return device memory: cudaMemGetInfo reads the same free bytes before and after
    shapes = ((256, 384, 512), (128, 1024, 2048), (512, 256, 256))
    operands = {s: host_operands(*s, seed=10 + i) for i, s in enumerate(shapes)}
    for s in shapes:
        run("gpu_kernels_nvfp4_gemm_host_static", *s, operands[s])
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        for s in shapes:
            run("gpu_kernels_nvfp4_gemm_host_static", *s, operands[s])
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes"
