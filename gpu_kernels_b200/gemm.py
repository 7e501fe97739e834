"""NVFP4 block-scaled GEMM plans (C[M,N] fp16 = alpha * A @ B.T on packed E2M1 operands).

`Nvfp4Gemm` wraps the plan calls the reference's harness makes
(benchmarks/nvfp4.py:52-66: plan_create / custom / cublas / validate / destroy)
with the same argument meaning: operands are baked into the plan and must stay
alive; `run(C)` is asynchronous on the current stream and capture-safe;
`validate()` synchronises and raises if the kernel reported an error.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class Nvfp4Gemm:
    def __init__(self, a_packed, b_packed, sfa, sfb, alpha: float = 1.0, workspace: torch.Tensor | None = None,
                 mx: bool = False):
        """mx = True: the operands are MXFP4 (one UE8M0 scale per 32 values, from `quantize_mx`)."""
        for name, t in (("a_packed", a_packed), ("b_packed", b_packed), ("sfa", sfa), ("sfb", sfb)):
            if not (t.is_cuda and t.dtype == torch.uint8 and t.is_contiguous()):
                raise ValueError(f"{name} must be a contiguous CUDA uint8 tensor")
        self.m, half_k = a_packed.shape
        self.n, half_kb = b_packed.shape
        if half_k != half_kb:
            raise ValueError("A and B disagree on K")
        self.k = 2 * half_k
        per = 32 if mx else 16
        from .nvfp4 import scale_rows
        if sfa.numel() != scale_rows(self.m) * self.k // per or sfb.numel() != scale_rows(self.n) * self.k // per:
            raise ValueError(f"scale tensors must hold ceil(rows/128)*128*K/{per} bytes")
        self.mx = mx
        self._keep = (a_packed, b_packed, sfa, sfb, workspace)
        self.device = a_packed.device
        self.out_dtype = torch.float16
        self._plan = ctypes.c_void_p()
        lib = _lib.load()
        with torch.cuda.device(self.device):
            if mx:
                _lib.check(lib.gpu_kernels_nvfp4_plan_create_mx(
                    ctypes.byref(self._plan), self.m, self.n, self.k, a_packed.data_ptr(), b_packed.data_ptr(),
                    sfa.data_ptr(), sfb.data_ptr(), _stream()))
            else:
                _lib.check(lib.gpu_kernels_nvfp4_plan_create(
                    ctypes.byref(self._plan), self.m, self.n, self.k, a_packed.data_ptr(), b_packed.data_ptr(),
                    sfa.data_ptr(), sfb.data_ptr(),
                    workspace.data_ptr() if workspace is not None else None,
                    workspace.numel() if workspace is not None else 0, _stream()))
        if alpha != 1.0:
            self.set_alpha(alpha)

    def set_alpha(self, alpha: float) -> None:
        _lib.check(_lib.load().gpu_kernels_nvfp4_plan_set_alpha(self._plan, float(alpha)))

    def set_option(self, key: str, value: int) -> None:
        # some options allocate or launch (split_k, l2_side): on the plan's own device
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_plan_set_option(self._plan, key.encode(), int(value)))
        if key == "out_bf16":
            self.out_dtype = torch.bfloat16 if value else torch.float16

    def info(self) -> dict:
        buf = (ctypes.c_int * 16)()
        _lib.check(_lib.load().gpu_kernels_nvfp4_plan_info(self._plan, buf))
        keys = ("M", "N", "K", "units", "cta_group", "tile_n", "group_m", "stages", "split_k", "k_skew",
                "direct_store", "out_bf16", "l2_side", "side0_units", "side1_units", "ragged_tiles")
        return dict(zip(keys, list(buf)))

    def placement_misses(self) -> int:
        """Clusters (summed over launches) that ran on the other L2 side than the tile route assumed."""
        n = ctypes.c_uint()
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_plan_placement_misses(self._plan, ctypes.byref(n)))
        return int(n.value)

    def run(self, out: torch.Tensor | None = None) -> torch.Tensor:
        if out is None:
            out = torch.empty((self.m, self.n), dtype=self.out_dtype, device=self.device)
        if not (out.is_cuda and out.dtype == self.out_dtype and out.is_contiguous() and out.shape == (self.m, self.n)):
            raise ValueError(f"out must be a contiguous CUDA {self.out_dtype} tensor [M, N]")
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_custom(self._plan, out.data_ptr(), _stream()))
        return out

    def linear(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x [M, K] in bf16 / fp16 / fp32 -> C = alpha * quantize(x) @ B.T: the quantiser writes the plan's own
        A and SFA tensors (the ones given to the constructor), the GEMM starts while it runs."""
        from .nvfp4 import _DTYPES
        if not x.is_cuda or x.dtype not in _DTYPES or x.shape != (self.m, self.k) or not x.is_contiguous():
            raise ValueError("x must be a contiguous CUDA tensor [M, K] of bf16, fp16 or fp32")
        if self.mx:
            raise ValueError("linear: NVFP4 plans only")
        if out is None:
            out = torch.empty((self.m, self.n), dtype=self.out_dtype, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_linear(self._plan, x.data_ptr(), _DTYPES[x.dtype], out.data_ptr(), _stream()))
        return out

    def profile(self, out: torch.Tensor):
        """One launch with the kernel's per-role wait counters on. Returns a list of dicts, one per CTA."""
        n = 4096 * 16
        buf = (ctypes.c_ulonglong * n)()
        written = ctypes.c_int()
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_plan_profile(self._plan, out.data_ptr(), _stream(), buf, n,
                                                                  ctypes.byref(written)))
        keys = ("producer_wait", "producer_total", "mma_wait_data", "mma_wait_acc", "mma_total",
                "epi_wait_acc", "epi_wait_store", "epi_total", "smid",
                "t_enter_ns", "t_first_data_ns", "t_last_issue_ns", "t_epi_done_ns")
        ctas = (written.value - 128) // 16
        self.handover = [tuple(buf[ctas * 16 + 8 * i: ctas * 16 + 8 * i + 8]) for i in range(16)]
        self.raw_profile = [tuple(buf[i:i + 16]) for i in range(0, ctas * 16, 16)]
        return [dict(zip(keys, buf[i:i + len(keys)])) for i in range(0, ctas * 16, 16)]

    def run_cublaslt(self, out: torch.Tensor) -> torch.Tensor:
        """cuBLASLt's NVFP4 matmul on the same operands (comparison only)."""
        a, b = self._keep[0], self._keep[1]
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_cublas(self._plan, out.data_ptr(), a.data_ptr(), b.data_ptr(), _stream()))
        return out

    def validate(self) -> None:
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().gpu_kernels_nvfp4_validate(self._plan))

    def close(self) -> None:
        if self._plan:
            _lib.load().gpu_kernels_nvfp4_plan_destroy(self._plan)
            self._plan = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def gemm_host(a_packed, b_packed, sfa, sfb, out, alpha: float = 1.0) -> torch.Tensor:
    """End-to-end GEMM on HOST tensors (pinned memory recommended): H2D, kernel, D2H, synchronised."""
    for t in (a_packed, b_packed, sfa, sfb, out):
        if t.is_cuda or not t.is_contiguous():
            raise ValueError("gemm_host takes contiguous host tensors")
    m, half_k = a_packed.shape
    n = b_packed.shape[0]
    _lib.check(_lib.load().gpu_kernels_nvfp4_gemm_host(
        m, n, 2 * half_k, a_packed.data_ptr(), b_packed.data_ptr(), sfa.data_ptr(), sfb.data_ptr(),
        out.data_ptr(), float(alpha), _stream()))
    return out


def l2_census() -> list[int]:
    """Cycles per dependent atomic that each SM of the current device measured in the L2-side census,
    by SM id; empty before the first plan asked for the "l2_side" order on this device."""
    buf = (ctypes.c_uint * 256)()
    n = ctypes.c_int()
    _lib.check(_lib.load().gpu_kernels_nvfp4_l2_census(buf, 256, ctypes.byref(n)))
    return list(buf[:n.value])
