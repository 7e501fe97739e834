"""ctypes binding of build/libgpu_kernels_nvfp4_bench.so (declarations: include/nvfp4_capi.h).

The library is the product; there is no Python or CPU fallback. Importing this
module without the built library raises, and every compute call raises on a
machine without an sm_100 GPU (the message comes from the library).
"""
from __future__ import annotations

import ctypes
from pathlib import Path

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

ROOT = Path(__file__).resolve().parents[1]
LIB_PATH = ROOT / "build" / "libgpu_kernels_nvfp4_bench.so"

# name -> (argtypes, restype); mirrors include/nvfp4_capi.h one to one
SIGNATURES = {
    "gpu_kernels_nvfp4_last_error": ([], ctypes.c_char_p),
    "gpu_kernels_nvfp4_plan_create": ([ctypes.POINTER(P), I, I, I, P, P, P, P, P, ctypes.c_size_t, P], I),
    "gpu_kernels_nvfp4_plan_destroy": ([P], None),
    "gpu_kernels_nvfp4_cublas": ([P, P, P, P, P], I),
    "gpu_kernels_nvfp4_custom": ([P, P, P], I),
    "gpu_kernels_nvfp4_validate": ([P], I),
    "gpu_kernels_nvfp4_l2_bytes": ([], I),
    "gpu_kernels_nvfp4_quantize": ([P, I, P, P, I, I, P], I),
    "gpu_kernels_nvfp4_quantize_scaled": ([P, I, F, P, P, I, I, P], I),
    "gpu_kernels_nvfp4_dequantize": ([P, P, P, I, I, P], I),
    "gpu_kernels_nvfp4_linear": ([P, P, I, P, P], I),
    "gpu_kernels_nvfp4_quantize_mx": ([P, I, P, P, I, I, P], I),
    "gpu_kernels_nvfp4_dequantize_mx": ([P, P, P, I, I, P], I),
    "gpu_kernels_nvfp4_plan_create_mx": ([ctypes.POINTER(P), I, I, I, P, P, P, P, P], I),
    "gpu_kernels_nvfp4_plan_set_alpha": ([P, F], I),
    "gpu_kernels_nvfp4_plan_set_option": ([P, ctypes.c_char_p, I], I),
    "gpu_kernels_nvfp4_moe_quantise_route": ([P, P, P, I, I, I, I, P, P, ctypes.POINTER(P), ctypes.POINTER(P), I, I, I, P, P, P, P, P, P], I),
    "gpu_kernels_nvfp4_peer_state_bytes": ([I, I, ctypes.POINTER(ctypes.c_size_t)], I),
    "gpu_kernels_nvfp4_peer_exchange": ([P, P, I, I, P, I, I, P, P], I),
    "gpu_kernels_nvfp4_plan_set_gather": ([P, ctypes.POINTER(P), I, I, I], I),
    "gpu_kernels_nvfp4_plan_info": ([P, ctypes.POINTER(I)], I),
    "gpu_kernels_nvfp4_plan_placement_misses": ([P, ctypes.POINTER(ctypes.c_uint)], I),
    "gpu_kernels_nvfp4_side_route": ([ctypes.c_char_p, I, I, ctypes.POINTER(ctypes.c_uint)], I),
    "gpu_kernels_nvfp4_l2_census": ([ctypes.POINTER(ctypes.c_uint), I, ctypes.POINTER(I)], I),
    "gpu_kernels_nvfp4_plan_profile": ([P, P, P, ctypes.POINTER(ctypes.c_ulonglong), I, ctypes.POINTER(I)], I),
    "gpu_kernels_nvfp4_last_kernel_cycles": ([], ctypes.c_uint),
    "gpu_kernels_nvfp4_gemm_host": ([I, I, I, P, P, P, P, P, F, P], I),
    "gpu_kernels_nvfp4_grouped_plan_create": ([ctypes.POINTER(P), I, I, I, I, I, P, P, P, P, P, P], I),
    "gpu_kernels_nvfp4_grouped_plan_destroy": ([P], None),
    "gpu_kernels_nvfp4_grouped_run": ([P, P, I, P], I),
    "gpu_kernels_nvfp4_grouped_run_swiglu": ([P, P, F, P, P, P], I),
    "gpu_kernels_nvfp4_grouped_run_scatter": ([P, P, P, P, I, I, I, P], I),
    "gpu_kernels_nvfp4_moe_payload_bytes": ([I], I),
    "gpu_kernels_nvfp4_moe_route_count": ([P, I, I, P, P], I),
    "gpu_kernels_nvfp4_moe_route_plan": ([P, I, P, I, I, I, P, P, P, P, P, P, P, P, P], I),
    "gpu_kernels_nvfp4_moe_clear_live": ([P, I, I, I, P, P, P, P], I),
    "gpu_kernels_nvfp4_moe_plan": ([P, I, I, I, I, I, P, P, P, P, P, P, P, I, P, P, P], I),
    "gpu_kernels_nvfp4_grouped_set_valid_rows": ([P, P], I),
    "gpu_kernels_nvfp4_moe_unpack_meta": ([P, I, P, I, I, I, P, P, P, P, P, P], I),
    "gpu_kernels_nvfp4_moe_count_exchange": ([P, I, I, P, P, I, I, I, P, P], I),
    "gpu_kernels_nvfp4_moe_pack": ([P, P, P, P, I, I, I, I, P, P, P, P, P], I),
    "gpu_kernels_nvfp4_moe_pack_to_pool": ([P, P, P, P, I, I, I, I, P, P, P, P, P, P, P], I),
    "gpu_kernels_nvfp4_moe_unpack": ([P, I, P, I, I, I, P, P, P, P, P, P, P, P], I),
    "gpu_kernels_nvfp4_moe_swiglu_quant": ([P, P, P, I, I, I, F, P, P, P], I),
    "gpu_kernels_nvfp4_moe_return_rows": ([P, P, P, I, I, P, P], I),
    "gpu_kernels_nvfp4_moe_reduce": ([P, P, I, I, I, P, P, I, P], I),
    "gpu_kernels_nvfp4_gemm_host_static": ([I, I, I, P, P, P, P, P, F, P], I),
    "gpu_kernels_nvfp4_moe_pack_peer": ([P, P, P, P, I, I, I, I, I, P, P, ctypes.POINTER(P), I, P, P], I),
    "gpu_kernels_nvfp4_moe_return_peer": ([P, P, P, P, P, I, I, I, I, ctypes.POINTER(P), I, P, P], I),
    "gpu_kernels_nvfp4_ipc_alloc": ([ctypes.c_size_t, ctypes.POINTER(P), P], I),
    "gpu_kernels_nvfp4_ipc_open": ([P, ctypes.POINTER(P)], I),
    "gpu_kernels_nvfp4_ipc_close": ([P], I),
    "gpu_kernels_nvfp4_ipc_free": ([P], I),
    "gpu_kernels_nvfp4_version": ([], ctypes.c_char_p),
    "gpu_kernels_nvfp4_launch_count": ([], ctypes.c_ulonglong),
}

_lib = None


class Nvfp4Error(RuntimeError):
    """Raised when a library call returns non-zero; carries the library's message."""


def load() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m gpu_kernels_b200.build` "
                "(there is no fallback path)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (argtypes, restype) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, restype
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status:
        raise Nvfp4Error(load().gpu_kernels_nvfp4_last_error().decode())


def launch_count() -> int:
    return int(load().gpu_kernels_nvfp4_launch_count())
