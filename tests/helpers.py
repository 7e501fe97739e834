"""Shared pieces of the GPU parity tests."""
import numpy as np
import torch

from oracle import nvfp4_oracle as O

# Floating-point acceptance of the GEMM against the FP32 dequantise-then-matmul oracle.
REL_FROBENIUS = 1e-3
MAX_ABS_OVER_RMS = 2e-2


def bf16_from_bits(bits_u16: np.ndarray, device="cuda") -> torch.Tensor:
    return torch.from_numpy(bits_u16.view(np.int16).copy()).to(device).view(torch.bfloat16)


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def assert_gemm_close(c: torch.Tensor, ref_f32, what=""):
    """c: fp16 result (any device); ref_f32: FP32 reference (torch or numpy)."""
    c = c.detach().float().cpu()
    ref = torch.as_tensor(ref_f32).detach().float().cpu()
    assert not torch.isnan(c).any(), f"{what}: NaN in the output (unwritten tile?)"
    err = (c - ref).double()
    rel = err.norm() / ref.double().norm().clamp_min(1e-30)
    rms = ref.double().pow(2).mean().sqrt()
    worst = err.abs().max()
    assert rel <= REL_FROBENIUS, f"{what}: relative Frobenius error {rel:.3e} > {REL_FROBENIUS}"
    assert worst <= MAX_ABS_OVER_RMS * rms, f"{what}: max abs error {worst:.3e} > {MAX_ABS_OVER_RMS} x rms {rms:.3e}"
    return float(rel), float(worst / rms)


def random_operand(rows, k, seed, scale=1.0, device="cuda", dtype=torch.bfloat16):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn((rows, k), generator=g, device=device, dtype=torch.float32) * scale).to(dtype)


def oracle_quantize_t(x: torch.Tensor):
    return O.quantize(to_np(x.float()))
