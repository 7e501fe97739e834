"""MXFP4 (E2M1 values, one UE8M0 scale per 32) through the same kernel as NVFP4 with scale_vec::2X.

The reference has no MXFP4 (its kernel is kind::mxf4nvf4 ... scale_vec::4X only, kernels/gemm/matmul/sm100.cu:341-342),
so there is no golden vector for it: the quantiser is held bit-exact to the CPU oracle's restatement of the OCP
microscaling conversion, and the GEMM to the FP32 dequantise-then-matmul of the stored bytes, with the NVFP4
tests' acceptance.
"""
import numpy as np
import pytest
import torch

from oracle import nvfp4_oracle as O
from helpers import assert_gemm_close, random_operand, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def g():
    import gpu_kernels_b200
    return gpu_kernels_b200


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_quantiser_is_bit_exact(g, dtype):
    rows, k = 256, 640
    x = random_operand(rows, k, seed=11, scale=3.0, dtype=torch.float32)
    x[0, :32] = 0.0
    x[1, 32:64] = -0.0
    x[2, 3] = float("inf")
    x[3, 40] = float("nan")
    x[4, :32] = 6.0
    x[5, :32] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 4.0] * 4)      # every tie, scale 1
    x[6, :32] = -x[5, :32]
    x[7, :64] *= 1e-30
    x[8, :64] *= 1e30 if dtype != torch.float16 else 1e3
    x[9, :32] = 1e-45 if dtype == torch.float32 else 6e-8                            # subnormal inputs
    x = x.to(dtype)
    packed, scales = g.quantize_mx(x)
    want_p, want_s = O.quantize_mx(to_np(x.float()))
    assert np.array_equal(to_np(scales), want_s)
    assert np.array_equal(to_np(packed), want_p)
    back = to_np(g.dequantize_mx(packed, scales))
    assert np.array_equal(back, O.dequantize_mx(want_p, want_s), equal_nan=True)


def test_shape_and_pointer_errors(g):
    with pytest.raises(Exception):
        g.quantize_mx(torch.zeros((128, 64), device="cuda", dtype=torch.bfloat16))   # K % 128
    with pytest.raises(Exception):
        g.quantize_mx(torch.zeros((0, 128), device="cuda", dtype=torch.bfloat16))    # no rows
    pa, sa = g.quantize_mx(random_operand(128, 256, seed=1))
    with pytest.raises(ValueError):
        g.Nvfp4Gemm(pa, pa, sa, sa[:-1].contiguous(), mx=True)
    with pytest.raises(ValueError):
        g.Nvfp4Gemm(pa, pa, sa, sa)                                                   # NVFP4 plan wants K/16 scales


SHAPES = [
    (128, 128, 128),            # one MMA group
    (256, 256, 256),
    (128, 256, 384),            # odd number of 128-wide K atoms
    (384, 640, 1152),           # tails in every dimension of the schedule
    (2048, 4096, 2048),
    (128, 7168, 1024),          # one tile row
    (4096, 1024, 4096),
]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_against_dequantised_matmul(g, m, n, k):
    a = random_operand(m, k, seed=m + k, scale=1.0)
    b = random_operand(n, k, seed=n + k + 1, scale=0.05)
    # block scales that differ along K and between rows, so a scale read from the wrong slot shows
    a *= torch.exp2(torch.randint(-6, 7, (m, k // 32), device="cuda").float()).repeat_interleave(32, dim=1).bfloat16()
    b *= torch.exp2(torch.randint(-6, 7, (n, k // 32), device="cuda").float()).repeat_interleave(32, dim=1).bfloat16()
    pa, sa = g.quantize_mx(a)
    pb, sb = g.quantize_mx(b)
    plan = g.Nvfp4Gemm(pa, pb, sa, sb, mx=True)
    out = torch.full((m, n), float("nan"), dtype=torch.float16, device="cuda")
    plan.run(out)
    plan.validate()
    ref = g.dequantize_mx(pa, sa) @ g.dequantize_mx(pb, sb).T
    assert_gemm_close(out, ref, f"mxfp4 {m}x{n}x{k}")
    plan.close()


def test_gemm_against_cpu_oracle_and_options(g):
    m, n, k = 256, 384, 512
    a = random_operand(m, k, seed=21)
    b = random_operand(n, k, seed=22, scale=0.1)
    pa, sa = g.quantize_mx(a)
    pb, sb = g.quantize_mx(b)
    ref = O.dequantize_mx(to_np(pa), to_np(sa)) @ O.dequantize_mx(to_np(pb), to_np(sb)).T
    plan = g.Nvfp4Gemm(pa, pb, sa, sb, alpha=0.5, mx=True)
    assert_gemm_close(plan.run(), 0.5 * ref, "mxfp4 alpha")
    plan.set_option("out_bf16", 1)
    out = plan.run()
    assert out.dtype == torch.bfloat16
    got = out.float().cpu().numpy()
    assert np.linalg.norm(got - 0.5 * ref) / np.linalg.norm(ref) < 8e-3          # bf16 rounding of the output
    plan.set_option("out_bf16", 0)
    for key, value in (("group_m", 1), ("k_skew", 0), ("static_operands", 2), ("pdl", 0)):
        plan.set_option(key, value)
        assert_gemm_close(plan.run(), 0.5 * ref, f"mxfp4 {key}={value}")
    with pytest.raises(Exception):
        plan.set_option("split_k", 2)
    with pytest.raises(Exception):
        plan.run_cublaslt(torch.empty((m, n), dtype=torch.float16, device="cuda"))
    plan.validate()
    plan.close()
