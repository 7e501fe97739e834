"""CPU oracle for the NVFP4 quantise / dequantise / GEMM path (numpy).

TEST INFRASTRUCTURE ONLY. This module restates, on the CPU, the algorithm of
the reference's Python quantiser and FP32 dequantise-then-matmul check so that
the CUDA kernels can be compared with it. The shipped library never imports it;
only the test-suite, the smoke check and the benchmark's CPU-baseline leg do.

Parity status: PINNED. Every function below is checked
  * against the reference's own known-answer tests (tests/test_nvfp4.py:11-35,
    restated in tests/test_oracle_golden.py), and
  * bit-for-bit against outputs of the reference Python itself, frozen as
    fixtures under tests/golden/ by tests/golden/make_golden.py.

The FP8 (E4M3) rounding and the FP32 matmul of the reference come from PyTorch
(torch>=2.11, `.to(torch.float8_e4m3fn)` and `@`); the rounding is restated
here from the published OCP FP8 definition (4 exponent bits, bias 7, 3 mantissa
bits, round-to-nearest-even, subnormal step 2**-9) and the matmul is numpy's
float32 `@`.
"""
from __future__ import annotations

import numpy as np

E2M1_LEVELS = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
# Midpoints between consecutive E2M1 magnitudes (reference/python/nvfp4.py:8).
E2M1_MIDPOINTS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
BLOCK = 16          # values per scale factor
SF_ROWS = 128       # rows per scale atom
SF_KBLOCKS = 4      # K blocks (of 16) per scale atom
SF_ATOM_BYTES = 512


def bf16_to_f32(raw_u16: np.ndarray) -> np.ndarray:
    """uint16 bfloat16 bit patterns -> float32 (exact)."""
    return (raw_u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round-to-nearest-even (NaN kept quiet)."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> 16) & np.uint32(1))) >> 16
    nan = np.isnan(x)
    return np.where(nan, np.uint32(0x7FC0), rounded).astype(np.uint16)


def encode_e2m1(values: np.ndarray) -> np.ndarray:
    """FP32 -> 4-bit E2M1 code, nearest-even, saturating at 6.

    Follows reference/python/nvfp4.py:6-14: the magnitude code is the number of
    midpoints strictly below |v|; a value exactly on a midpoint takes the even
    code of its two neighbours; bit 3 is (v < 0), so a negative value that
    rounds to zero keeps its sign bit while an input of -0.0 does not.
    """
    values = np.asarray(values, dtype=np.float32)
    mag = np.abs(values)
    code = np.searchsorted(E2M1_MIDPOINTS, mag, side="left").astype(np.int64)
    tie = mag == E2M1_MIDPOINTS[np.minimum(code, 6)]
    code = code + (tie & ((code & 1) != 0))
    return (code | ((values < 0).astype(np.int64) << 3)).astype(np.uint8)


def f32_to_ue4m3(t: np.ndarray) -> np.ndarray:
    """Positive FP32 in [2**-9, 448] -> E4M3 byte, round-to-nearest-even.

    Restates the conversion the reference takes from PyTorch at
    reference/python/nvfp4.py:34 (`.to(torch.float8_e4m3fn)`); the clamp there
    keeps the argument inside the finite range, so the sign bit is always 0.
    NaN maps to 0x7F as in PyTorch.
    """
    t = np.ascontiguousarray(t, dtype=np.float32)
    bits = t.view(np.uint32).astype(np.uint64)
    # normal range of E4M3: keep 3 mantissa bits, carry may bump the exponent
    rounded = (bits + np.uint64(0x7FFFF) + ((bits >> np.uint64(20)) & np.uint64(1))) >> np.uint64(20)
    normal = rounded.astype(np.int64) - ((127 - 7) << 3)
    # below 2**-6 the grid is uniform with step 2**-9 (rint is nearest-even)
    with np.errstate(invalid="ignore"):
        sub = np.rint(t.astype(np.float64) * 512.0)
    sub = np.where(np.isnan(sub), 0, sub).astype(np.int64)
    out = np.where(t < np.float32(2.0 ** -6), sub, normal)
    out = np.where(np.isnan(t), 0x7F, out)
    return out.astype(np.uint8)


def ue4m3_to_f32(b: np.ndarray) -> np.ndarray:
    """E4M3 byte (sign bit honoured, 0x7F/0xFF = NaN) -> FP32."""
    b = np.asarray(b, dtype=np.uint8).astype(np.int32)
    e = (b >> 3) & 15
    m = b & 7
    mag = np.where(e == 0, m.astype(np.float64) * 2.0 ** -9,
                   (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float64)))
    mag = np.where((b & 0x7F) == 0x7F, np.nan, mag)
    return np.where(b & 0x80, -mag, mag).astype(np.float32)


def scale_offset(row, kblock, k):
    """Byte offset of the scale of (row, 16-wide K block) in the VEC16 layout.

    Closed form pinned by the reference's tests/test_nvfp4.py:25-26.
    """
    return ((row // 128) * (k // 64) + kblock // 4) * 512 + (row % 32) * 16 + ((row % 128) // 32) * 4 + kblock % 4


def pack_scales(scales_u8: np.ndarray) -> np.ndarray:
    """[rows, K/16] bytes -> flat [rows/128, K/64, 32, 4, 4] (reference/python/nvfp4.py:17-21)."""
    rows, blocks = scales_u8.shape
    assert rows % 128 == 0 and blocks % 4 == 0
    return np.ascontiguousarray(
        scales_u8.reshape(rows // 128, 4, 32, blocks // 4, 4).transpose(0, 3, 2, 1, 4)).reshape(-1)


def unpack_scales_u8(flat: np.ndarray, rows: int, k: int) -> np.ndarray:
    """Inverse of pack_scales, returning bytes [rows, K/16] (reference/python/nvfp4.py:24-27)."""
    return np.ascontiguousarray(
        flat.reshape(rows // 128, k // 64, 32, 4, 4).transpose(0, 3, 2, 1, 4)).reshape(rows, k // 16)


def unpack_scales(flat: np.ndarray, rows: int, k: int) -> np.ndarray:
    return ue4m3_to_f32(unpack_scales_u8(flat, rows, k))


def quantize(values: np.ndarray):
    """FP32 [rows, K] -> (packed uint8 [rows, K/2], scales uint8 [rows*K/16]).

    reference/python/nvfp4.py:30-37: per 16 values scale = e4m3(clamp(amax/6,
    2**-9, 448)); code = e2m1(x / float(scale)); two codes per byte, even k in
    the low nibble; scales stored in the VEC16 layout. Both divisions are IEEE
    float32 divisions.
    """
    values = np.asarray(values, dtype=np.float32)
    rows, k = values.shape
    assert rows % 128 == 0 and k % 64 == 0
    blocks = values.reshape(rows, k // 16, 16)
    with np.errstate(invalid="ignore", divide="ignore", over="ignore"):
        amax = np.abs(blocks).max(axis=-1)          # NaN propagates like torch.amax
        t = amax / np.float32(6.0)
        t = np.where(np.isnan(t), t, np.clip(t, np.float32(2.0 ** -9), np.float32(448.0))).astype(np.float32)
        sbyte = f32_to_ue4m3(t)
        q = blocks / ue4m3_to_f32(sbyte)[..., None]
    codes = encode_e2m1(q).reshape(rows, k)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return np.ascontiguousarray(packed), pack_scales(sbyte)


def quantize_padded(values: np.ndarray, fn=None):
    """Any row count: the reference's `quantize` (which wants rows % 128 == 0, reference/python/nvfp4.py:20)
    applied to the tensor with zero rows appended up to the next multiple of 128; the packed array is cut back
    to the true rows, the scale array keeps its whole atoms. fn: `quantize` (default) or `quantize_mx`."""
    values = np.asarray(values, dtype=np.float32)
    rows = values.shape[0]
    pad = -rows % 128
    packed, scales = (fn or quantize)(np.concatenate([values, np.zeros((pad, values.shape[1]), np.float32)]) if pad else values)
    return np.ascontiguousarray(packed[:rows]), scales


def dequantize_padded(packed: np.ndarray, scales_flat: np.ndarray, fn=None) -> np.ndarray:
    """Inverse companion of quantize_padded: FP32 [rows, K] from a packed array with any row count."""
    rows = packed.shape[0]
    pad = -rows % 128
    full = np.concatenate([packed, np.zeros((pad, packed.shape[1]), np.uint8)]) if pad else packed
    return (fn or dequantize)(full, scales_flat)[:rows]


def quantize_scaled(values: np.ndarray, inv_tensor_scale: float):
    """Two-level scaling (this repository's extension; the reference has block scales only): the reference's
    `quantize` applied to float32(values) * float32(inv_tensor_scale), one FP32 product per value."""
    return quantize(np.asarray(values, dtype=np.float32) * np.float32(inv_tensor_scale))


def quantize_mx(values: np.ndarray):
    """MXFP4 (this repository's extension: PARITY UNPINNED, the reference has no MXFP4 and no fixture for it).

    The OCP Microscaling v1.0 conversion, restated: per 32 values along K the shared exponent is
    e = floor(log2(amax)) - 2 (2 = the exponent of E2M1's largest value, 6 = 1.5 * 2**2), clamped to [-127, 127]
    and stored as the UE8M0 byte e + 127; each value becomes the E2M1 code of x * 2**-e under `encode_e2m1`'s
    rule. An all-zero block takes e = -127; a block with a NaN or an infinity takes byte 0xFF (UE8M0's NaN) and
    codes 0x7. Scales sit in 512-byte atoms of 128 rows x 4 blocks as in the VEC16 layout, [rows/128][K/128].
    Returns (packed uint8 [rows, K/2], scales uint8 [rows*K/32]).
    """
    values = np.asarray(values, dtype=np.float32)
    rows, k = values.shape
    assert rows % 128 == 0 and k % 128 == 0
    blocks = values.reshape(rows, k // 32, 32)
    with np.errstate(invalid="ignore", over="ignore"):
        amax = np.abs(blocks).max(axis=-1)
        special = ~np.isfinite(amax)
        safe = np.where(special | (amax == 0), np.float32(1.0), amax)
        _, ex = np.frexp(safe)                                        # safe = m * 2**ex, m in [0.5, 1)
        e = np.where(amax == 0, -127, np.clip(ex.astype(np.int64) - 3, -127, 127))
        q = blocks * np.ldexp(np.float32(1.0), -e)[..., None].astype(np.float32)
    codes = encode_e2m1(q)
    codes = np.where(special[..., None], np.uint8(7), codes).reshape(rows, k)
    sbyte = np.where(special, 0xFF, e + 127).astype(np.uint8)
    packed = codes[:, 0::2] | (codes[:, 1::2] << 4)
    return np.ascontiguousarray(packed), pack_scales(sbyte)


def dequantize_mx(packed: np.ndarray, scales_flat: np.ndarray) -> np.ndarray:
    """MXFP4 bytes -> FP32 [rows, K]: level * sign * 2**(byte - 127); byte 0xFF gives NaN."""
    rows, half_k = packed.shape
    k = 2 * half_k
    codes = np.stack((packed & 15, packed >> 4), axis=-1).reshape(rows, k)
    vals = E2M1_LEVELS[codes & 7] * (1.0 - 2.0 * (codes >> 3).astype(np.float32))
    sb = unpack_scales_u8(scales_flat, rows, k // 2).astype(np.int64)  # blocks of 32: the K/2-wide VEC16 order
    s = np.where(sb == 0xFF, np.float32(np.nan), np.ldexp(np.float32(1.0), np.minimum(sb, 254) - 127)).astype(np.float32)
    with np.errstate(invalid="ignore"):
        return (vals.reshape(rows, -1, 32) * s[..., None]).reshape(rows, k).astype(np.float32)


def dequantize(packed: np.ndarray, scales_flat: np.ndarray) -> np.ndarray:
    """Stored bytes -> FP32 [rows, K] (reference/python/nvfp4.py:40-47)."""
    rows, half_k = packed.shape
    k = 2 * half_k
    codes = np.stack((packed & 15, packed >> 4), axis=-1).reshape(rows, k)
    vals = E2M1_LEVELS[codes & 7] * (1.0 - 2.0 * (codes >> 3).astype(np.float32))
    s = unpack_scales(scales_flat, rows, k)
    return (vals.reshape(rows, -1, 16) * s[..., None]).reshape(rows, k).astype(np.float32)


def gemm(packed_a, sfa, packed_b, sfb, alpha: float = 1.0) -> np.ndarray:
    """C[M,N] fp16 = alpha * dequant(A) @ dequant(B).T, FP32 accumulation.

    The reference's check: benchmarks/nvfp4.py:41 (alpha = 1 there; the FP32
    global scale multiplies the FP32 accumulator before the FP16 rounding).
    """
    a = dequantize(packed_a, sfa)
    b = dequantize(packed_b, sfb)
    c = a @ b.T
    if alpha != 1.0:
        c = c * np.float32(alpha)
    return c.astype(np.float16)


def gemm_f32(packed_a, sfa, packed_b, sfb, alpha: float = 1.0) -> np.ndarray:
    """Same product kept in FP32 (for error metrics that should not see FP16 rounding)."""
    c = dequantize(packed_a, sfa) @ dequantize(packed_b, sfb).T
    return c * np.float32(alpha) if alpha != 1.0 else c
