"""NVFP4 quantise / dequantise on the GPU, with the call shapes of the reference's
reference/python/nvfp4.py (`quantize`, `dequantize`, `pack_scales`, `unpack_scales`).

`quantize(values)` takes a CUDA tensor [rows, K] (bf16, fp16 or fp32) and returns
`(packed uint8 [rows, K/2], scales uint8 [rows*K/16])`, bit-identical to the
reference function of the same name (reference/python/nvfp4.py:30-37). The work
is done by the CUDA kernels in csrc/nvfp4_quant.cu through the C ABI; CPU tensors
are rejected.
"""
from __future__ import annotations

import torch

from . import _lib

_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def scale_rows(rows: int) -> int:
    """Rows the scale array of a `rows`-row tensor covers: whole 128-row atoms. The reference's layout has no
    partial atoms (reference/python/nvfp4.py:20 asserts rows % 128 == 0); a tensor with another row count is
    quantised as if zero rows filled its last atom (their scale bytes are those of zero blocks), and its packed
    array keeps the true row count."""
    return -(-rows // 128) * 128


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor: this package has no CPU path")


def quantize(values: torch.Tensor, tensor_scale: float | None = None):
    """[rows, K] -> (packed [rows, K/2] uint8, scales [scale_rows(rows)*K/16] uint8 in the VEC16 layout).

    tensor_scale (two-level scaling, not in the reference): the values are first multiplied, in FP32, by
    float32(1 / tensor_scale); the GEMM's alpha then carries the product of the operands' tensor scales."""
    _require_cuda(values, "values")
    if values.dim() != 2:
        raise ValueError("values must be 2-D [rows, K]")
    if values.dtype not in _DTYPES:
        values = values.float()
    values = values.contiguous()
    rows, k = values.shape
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=values.device)
    scales = torch.empty((scale_rows(rows) * k // 16,), dtype=torch.uint8, device=values.device)
    with torch.cuda.device(values.device):
        if tensor_scale is None:
            _lib.check(_lib.load().gpu_kernels_nvfp4_quantize(
                values.data_ptr(), _DTYPES[values.dtype], packed.data_ptr(), scales.data_ptr(), rows, k, _stream()))
        else:
            _lib.check(_lib.load().gpu_kernels_nvfp4_quantize_scaled(
                values.data_ptr(), _DTYPES[values.dtype], inverse_tensor_scale(tensor_scale), packed.data_ptr(),
                scales.data_ptr(), rows, k, _stream()))
    return packed, scales


def inverse_tensor_scale(tensor_scale: float) -> float:
    """float32(1 / tensor_scale) as a Python float: the multiplier the scaled quantiser applies."""
    return float(torch.tensor(1.0, dtype=torch.float32) / torch.tensor(float(tensor_scale), dtype=torch.float32))


def tensor_scale_for(values: torch.Tensor) -> float:
    """The usual per-tensor scale of two-level NVFP4: amax / (6 * 448), so that the largest block scale is 448."""
    amax = float(values.detach().abs().max().float())
    return amax / (6.0 * 448.0) if amax > 0.0 else 1.0


def dequantize(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Stored bytes -> FP32 [rows, K] (reference/python/nvfp4.py:40-47)."""
    _require_cuda(packed, "packed")
    _require_cuda(scales, "scales")
    packed, scales = packed.contiguous(), scales.contiguous()
    rows, half_k = packed.shape
    if scales.numel() != scale_rows(rows) * half_k // 8:
        raise ValueError("scales must hold ceil(rows/128)*128*K/16 bytes")
    out = torch.empty((rows, 2 * half_k), dtype=torch.float32, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(_lib.load().gpu_kernels_nvfp4_dequantize(
            packed.data_ptr(), scales.data_ptr(), out.data_ptr(), rows, 2 * half_k, _stream()))
    return out


def pack_scales(scales: torch.Tensor) -> torch.Tensor:
    """[rows, K/16] bytes -> VEC16 byte order (reference/python/nvfp4.py:17-21). A pure view
    permutation, kept for callers that build scales themselves."""
    rows, blocks = scales.shape
    return (scales.view(torch.uint8).reshape(rows // 128, 4, 32, blocks // 4, 4)
            .permute(0, 3, 2, 1, 4).contiguous().reshape(-1))


def unpack_scales(scales: torch.Tensor, rows: int, k: int) -> torch.Tensor:
    """VEC16 bytes -> [rows, K/16] bytes (reference/python/nvfp4.py:24-27, without the float cast)."""
    return (scales.reshape(rows // 128, k // 64, 32, 4, 4)
            .permute(0, 3, 2, 1, 4).contiguous().reshape(rows, k // 16))


def quantize_mx(values: torch.Tensor):
    """MXFP4: [rows, K] -> (packed [rows, K/2] uint8, scales [rows*K/32] uint8 UE8M0 in the VEC32 atom order).
    No counterpart in the reference; see include/nvfp4_capi.h for the rule."""
    _require_cuda(values, "values")
    if values.dim() != 2:
        raise ValueError("values must be 2-D [rows, K]")
    if values.dtype not in _DTYPES:
        values = values.float()
    values = values.contiguous()
    rows, k = values.shape
    packed = torch.empty((rows, k // 2), dtype=torch.uint8, device=values.device)
    scales = torch.empty((scale_rows(rows) * k // 32,), dtype=torch.uint8, device=values.device)
    with torch.cuda.device(values.device):
        _lib.check(_lib.load().gpu_kernels_nvfp4_quantize_mx(
            values.data_ptr(), _DTYPES[values.dtype], packed.data_ptr(), scales.data_ptr(), rows, k, _stream()))
    return packed, scales


def dequantize_mx(packed: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """MXFP4 bytes -> FP32 [rows, K]."""
    _require_cuda(packed, "packed")
    _require_cuda(scales, "scales")
    packed, scales = packed.contiguous(), scales.contiguous()
    rows, half_k = packed.shape
    if scales.numel() != scale_rows(rows) * half_k // 16:
        raise ValueError("scales must hold ceil(rows/128)*128*K/32 bytes")
    out = torch.empty((rows, 2 * half_k), dtype=torch.float32, device=packed.device)
    with torch.cuda.device(packed.device):
        _lib.check(_lib.load().gpu_kernels_nvfp4_dequantize_mx(
            packed.data_ptr(), scales.data_ptr(), out.data_ptr(), rows, 2 * half_k, _stream()))
    return out
