"""A wait on another GPU that never arrives must run out, be reported by validate() and leave the context
usable: here one rank of a two-rank barrier is simply never launched (its state block is a second buffer on the
same GPU that nothing updates), so the kernel's bounded wait expires after its 2 s limit."""
import ctypes
import time

import pytest
import torch

from helpers import assert_gemm_close, random_operand

pytestmark = pytest.mark.gpu


def test_barrier_wait_runs_out_and_is_reported():
    import gpu_kernels_b200 as g
    from gpu_kernels_b200 import _lib
    lib = _lib.load()
    lib.gpu_kernels_nvfp4_last_error.restype = ctypes.c_char_p
    assert lib.gpu_kernels_nvfp4_validate(None) == 0                       # nothing pending from earlier tests
    nbytes = ctypes.c_size_t()
    _lib.check(lib.gpu_kernels_nvfp4_peer_state_bytes(2, 16, ctypes.byref(nbytes)))
    states = [torch.zeros(nbytes.value, dtype=torch.uint8, device="cuda") for _ in range(2)]
    table = torch.tensor([s.data_ptr() for s in states], dtype=torch.int64, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _lib.check(lib.gpu_kernels_nvfp4_peer_exchange(states[0].data_ptr(), table.data_ptr(), 2, 0, None, 0, 16, None, stream))
    torch.cuda.synchronize()                                               # rank 1 never comes: the wait gives up
    waited = time.perf_counter() - t0
    assert 1.5 < waited < 20.0, waited
    # the report sits in the device's own status slot: a plan's validate neither sees nor clears it
    pa, sa = g.quantize(random_operand(256, 512, seed=1))
    pb, sb = g.quantize(random_operand(256, 512, seed=2, scale=0.02))
    bystander = g.Nvfp4Gemm(pa, pb, sa, sb)
    bystander.run()
    bystander.validate()
    bystander.close()
    assert lib.gpu_kernels_nvfp4_validate(None) == 1
    message = lib.gpu_kernels_nvfp4_last_error().decode()
    assert "status 0x20" in message, message
    # reported once, then clear; the context still computes
    assert lib.gpu_kernels_nvfp4_validate(None) == 0
    pa, sa = g.quantize(random_operand(256, 512, seed=1))
    pb, sb = g.quantize(random_operand(256, 512, seed=2, scale=0.02))
    plan = g.Nvfp4Gemm(pa, pb, sa, sb)
    out = plan.run()
    plan.validate()
    assert_gemm_close(out, g.dequantize(pa, sa) @ g.dequantize(pb, sb).T, "GEMM after a reported timeout")
    plan.close()
