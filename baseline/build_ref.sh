#!/bin/bash
# Builds the reference's own sm_100a NVFP4 kernel and bridge, from the sources where they lie, into
# baseline/_ref/libgpu_kernels_nvfp4_bench.so (git-ignored). It is the same-box timing bar for
# 1-GPU runs only: its loads use cluster multicast, so baseline/_ref is listed in .gpurunignore.multi
# and never travels to a multi-GPU run. CUDA 12.9 rejects the `__block_size__` hint next to
# `__cluster_dims__`; the hint is emptied by the force-included ref_shim.h (it does not change the kernel).
set -e
REF=${1:-/root/reference}
HERE=$(cd "$(dirname "$0")" && pwd)
mkdir -p "$HERE/_ref"
nvcc -std=c++17 -O3 -gencode arch=compute_100a,code=sm_100a -lineinfo -Xcompiler -fPIC -shared \
  -include "$HERE/ref_shim.h" -I "$REF/include" \
  "$REF/kernels/gemm/matmul/sm100.cu" "$REF/benchmarks/bindings/nvfp4_bridge.cu" \
  -o "$HERE/_ref/libgpu_kernels_nvfp4_bench.so" -lcublasLt -lcuda -L/usr/local/cuda/lib64/stubs
echo "built $HERE/_ref/libgpu_kernels_nvfp4_bench.so"
