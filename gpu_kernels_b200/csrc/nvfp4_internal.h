// Declarations shared by the translation units of the NVFP4 library (not installed).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace nvfp4_b200 {

enum InputDtype : int { DTYPE_BF16 = 0, DTYPE_F16 = 1, DTYPE_F32 = 2 };

inline void cuda_check(cudaError_t e) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA: ") + cudaGetErrorString(e));
}

// Refuse to run on anything but a compute-capability 10.x device: there is no
// other code path in this library.
void require_sm100();

// nvfp4_quant.cu
void check_quant_shape(int rows, int K);
void quantise(const void* x, int dtype, uint8_t* packed, uint8_t* scales, int rows, int K, cudaStream_t stream);
void dequantise(const uint8_t* packed, const uint8_t* scales, float* out, int rows, int K, cudaStream_t stream);

}  // namespace nvfp4_b200
