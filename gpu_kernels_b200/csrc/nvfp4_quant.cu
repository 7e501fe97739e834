// NVFP4 quantise / pack and dequantise kernels for sm_100a.
//
// quantise: x[rows, K] (bf16 / fp16 / fp32) -> packed E2M1 [rows, K/2] plus one
// UE4M3 scale per 16 values, written directly in the 128-row x 4-block scale
// atoms that cuBLASLt's VEC16 mode and the tcgen05 block-scaled MMA read.
// Arithmetic follows the reference's PyTorch quantiser step by step
// (reference/python/nvfp4.py:30-37 and :6-14): amax -> IEEE divide by 6 ->
// clamp [2^-9, 448] -> E4M3 nearest-even -> IEEE divide -> E2M1 nearest-even
// with sign bit (q < 0), bit for bit. The kernel is HBM-bound: 2 B read (bf16) and 0.5625 B
// written per value; a CTA owns a 128-row x 256-column tile so that each scale
// atom (512 B) and each packed row segment (128 B) leaves in full lines.
#include "nvfp4_internal.h"
#include "quant_device.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace nvfp4_b200 {
namespace {

constexpr int Q_ROWS = 128;      // rows per CTA tile = rows of one scale atom
constexpr int Q_THREADS = 256;

template <typename T> struct Loader;
template <> struct Loader<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[16]) {
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 f = __ldg(reinterpret_cast<const float4*>(p) + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    }
};

template <typename T> struct PairFormat { using type = void; };
template <> struct PairFormat<__nv_bfloat16> { using type = Bf16Pairs; };
template <> struct PairFormat<__half> { using type = Fp16Pairs; };

// One block of 16 values straight from global memory to its scale byte and packed codes.
template <typename T>
__device__ __forceinline__ uint32_t quantise_from(const T* p, uint2& out) {
    if constexpr (sizeof(T) == 2) {
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(p));
        const uint4 b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        return quantise_block_pairs<typename PairFormat<T>::type>(w, out);
    } else {
        float v[16];
        Loader<T>::load(p, v);
        return quantise_block<true>(v, out);
    }
}

// Four CTAs per SM: the register cap this implies (64) keeps 32 warps resident, which together with the loads
// kept ahead is what it takes to cover the memory latency (measured on 8192 x 8192 bf16: 3 CTAs 37.3 us,
// 4 CTAs 34.9 us, 5 CTAs, which leaves no registers for the loads ahead, 39.1 us).
// COLS: K values per CTA tile (256 = four scale atoms, or 128 = two). The narrower tile gives twice the CTAs,
// which evens out the last wave of a grid that is only a few waves long.
// TAIL: the instance for a last row tile that the tensor fills only in part (rows % 128 != 0), launched for that
// tile alone (row_tile0 = its index): rows the tensor does not have are read as zeros, which gives them the scale
// byte of a zero block (0x01) in the atom and no packed bytes.
template <typename T, int COLS, bool TAIL = false>
__global__ void __launch_bounds__(Q_THREADS, 4)
quantise_kernel(const T* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                int rows, int K, int row_tile0) {
    // A kernel behind this one on the stream that was launched with the programmatic stream-serialisation
    // attribute may set itself up now; it still waits for this grid to finish before it reads what is written here.
    asm volatile("griddepcontrol.launch_dependents;");
    constexpr int BLOCKS = COLS / 16;                           // 16-value blocks across the tile
    constexpr int ROWS_PER_PASS = Q_THREADS / BLOCKS;
    constexpr int PASSES = Q_ROWS / ROWS_PER_PASS;
    constexpr int ATOMS = COLS / 64;
    __shared__ __align__(16) uint8_t sf_tile[ATOMS * 512];
    const int kb = threadIdx.x % BLOCKS;                        // 16-value block inside the tile
    const int row_in_pass = threadIdx.x / BLOCKS;
    const int col0 = blockIdx.x * COLS;
    const int row_tile = TAIL ? row_tile0 : int(blockIdx.y);
    const int row_base = row_tile * Q_ROWS;
    const int k = col0 + kb * 16;
    const bool live = k < K;                                    // K is a multiple of 64, the tile of COLS
    auto emit = [&](int r, uint32_t sbyte, const uint2& out) {
        if (!TAIL || row_base + r < rows)
            *reinterpret_cast<uint2*>(packed + size_t(row_base + r) * (K / 2) + k / 2) = out;
        sf_tile[(kb >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = static_cast<uint8_t>(sbyte);
    };
    if constexpr (sizeof(T) == 2) {
        // 16-bit inputs: the loads of two passes are kept in flight ahead of the arithmetic (32 bytes per thread
        // and pass), so that a warp waits for memory once per tile rather than once per pass.
        constexpr int AHEAD = 2;
        uint4 lo[AHEAD], hi[AHEAD];
        auto fetch = [&](int pass, uint4& a, uint4& b) {
            const int r = pass * ROWS_PER_PASS + row_in_pass;
            const uint4* p = reinterpret_cast<const uint4*>(x + size_t(row_base + r) * K + k);
            if (TAIL && row_base + r >= rows) { a = b = make_uint4(0u, 0u, 0u, 0u); return; }
            a = __ldg(p);
            b = __ldg(p + 1);
        };
        if (live) {
            #pragma unroll
            for (int i = 0; i < AHEAD; ++i) fetch(i, lo[i], hi[i]);
            #pragma unroll
            for (int pass = 0; pass < PASSES; ++pass) {
                const uint4 a = lo[pass % AHEAD], b = hi[pass % AHEAD];
                if (pass + AHEAD < PASSES) fetch(pass + AHEAD, lo[pass % AHEAD], hi[pass % AHEAD]);
                const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                uint2 out;
                const uint32_t sbyte = quantise_block_pairs<typename PairFormat<T>::type>(w, out);
                emit(pass * ROWS_PER_PASS + row_in_pass, sbyte, out);
            }
        }
    } else {
        #pragma unroll 4
        for (int pass = 0; pass < PASSES; ++pass) {
            const int r = pass * ROWS_PER_PASS + row_in_pass;
            if (live) {
                uint2 out;
                uint32_t sbyte = 0x01u;
                if (TAIL && row_base + r >= rows) out = make_uint2(0u, 0u);
                else sbyte = quantise_from(x + size_t(row_base + r) * K + k, out);
                emit(r, sbyte, out);
            }
        }
    }
    __syncthreads();
    // The tile's atoms are consecutive in the VEC16 layout: one 16-byte store per thread.
    const int atoms = min(ATOMS, (K - col0) / 64);
    if (int(threadIdx.x) < atoms * 32) {
        const size_t first_atom = size_t(row_tile) * (K / 64) + size_t(blockIdx.x) * ATOMS;
        reinterpret_cast<uint4*>(scales + first_atom * 512)[threadIdx.x] =
            reinterpret_cast<const uint4*>(sf_tile)[threadIdx.x];
    }
}

// Two-level scaling: every value is first multiplied (in FP32) by the reciprocal of a per-tensor scale, then
// quantised as above; the GEMM undoes the tensor scales through its alpha. One 16-value block per thread and pass,
// through the FP32 block routine whatever the input type (the product is no longer a 16-bit value).
template <typename T>
__global__ void __launch_bounds__(Q_THREADS)
quantise_scaled_kernel(const T* __restrict__ x, float inv_global, uint8_t* __restrict__ packed,
                       uint8_t* __restrict__ scales, int rows, int K) {
    __shared__ __align__(16) uint8_t sf_tile[4 * 512];
    const int kb = threadIdx.x & 15, row_in_pass = threadIdx.x >> 4;
    const int col0 = blockIdx.x * 256, row_base = blockIdx.y * Q_ROWS;
    const int k = col0 + kb * 16;
    if (k < K) {
        #pragma unroll 2
        for (int pass = 0; pass < 8; ++pass) {
            const int r = pass * 16 + row_in_pass;
            const T* p = x + size_t(row_base + r) * K + k;
            if (row_base + r >= rows) {                         // a row the tensor does not have: a zero block's scale
                sf_tile[(kb >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = 0x01u;
                continue;
            }
            float v[16];
            if constexpr (sizeof(T) == 4) {
                Loader<float>::load(reinterpret_cast<const float*>(p), v);
            } else {
                const uint4 a = __ldg(reinterpret_cast<const uint4*>(p)), b = __ldg(reinterpret_cast<const uint4*>(p) + 1);
                const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    v[2 * i] = PairFormat<T>::type::widen(w[i] & 0xFFFFu);
                    v[2 * i + 1] = PairFormat<T>::type::widen(w[i] >> 16);
                }
            }
            #pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __fmul_rn(v[i], inv_global);
            uint2 out;
            const uint32_t sbyte = quantise_block<true>(v, out);
            *reinterpret_cast<uint2*>(packed + size_t(row_base + r) * (K / 2) + k / 2) = out;
            sf_tile[(kb >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = static_cast<uint8_t>(sbyte);
        }
    }
    __syncthreads();
    const int atoms = min(4, (K - col0) / 64);
    if (int(threadIdx.x) < atoms * 32) {
        const size_t first_atom = size_t(blockIdx.y) * (K / 64) + size_t(blockIdx.x) * 4;
        reinterpret_cast<uint4*>(scales + first_atom * 512)[threadIdx.x] = reinterpret_cast<const uint4*>(sf_tile)[threadIdx.x];
    }
}

// packed + scales -> FP32 [rows, K]; one thread per 16-value block
// (reference/python/nvfp4.py:40-47).
__global__ void __launch_bounds__(256)
dequantise_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                  float* __restrict__ out, int rows, int K) {
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int blocks_per_row = K / 16;
    if (idx >= size_t(rows) * blocks_per_row) return;
    const int r = static_cast<int>(idx / blocks_per_row), b = static_cast<int>(idx % blocks_per_row);
    const size_t off = (size_t(r / 128) * (K / 64) + b / 4) * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + b % 4;
    const uint32_t sb = scales[off];
    // 0x7F / 0xFF are NaN in E4M3 (finite-only format); the quantiser never sets the sign bit.
    float s = (sb & 0x7Fu) == 0x7Fu ? __uint_as_float(0x7FC00000u) : ue4m3_to_float(sb & 0x7Fu);
    if (sb & 0x80u) s = -s;
    const uint2 p = __ldg(reinterpret_cast<const uint2*>(packed + size_t(r) * (K / 2) + b * 8));
    const uint32_t w[2] = {p.x, p.y};
    float4* dst = reinterpret_cast<float4*>(out + size_t(r) * K + b * 16);
    #pragma unroll
    for (int h = 0; h < 2; ++h) {
        float f[8];
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t c = (w[h] >> (4 * i)) & 15u;
            const uint32_t m = c & 7u;
            // levels 0, .5, 1, 1.5, 2, 3, 4, 6
            const float level = m < 2u ? 0.5f * m : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
            f[i] = level * (1.0f - 2.0f * static_cast<float>(c >> 3)) * s;
        }
        dst[2 * h] = make_float4(f[0], f[1], f[2], f[3]);
        dst[2 * h + 1] = make_float4(f[4], f[5], f[6], f[7]);
    }
}

// ---- MXFP4 (OCP microscaling): E2M1 values, one UE8M0 power-of-two scale per 32 values ------------------------
// Per block: e = floor(log2(amax)) - 2 (2 = the largest exponent of E2M1), clamped to [-127, 127]; scale byte
// e + 127; q = x * 2^-e (exact but for underflow) encoded as E2M1 with the quantiser's rounding and sign rule.
// An all-zero block takes e = -127; a block with a NaN or an infinity takes the NaN scale 0xFF and the codes of
// the NVFP4 NaN block. One thread per block. The scale bytes go to cuBLASLt's VEC32 order: the VEC16 atoms with
// K/32 blocks per row.
template <typename T>
__global__ void __launch_bounds__(256)
quantise_mx_kernel(const T* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, int rows, int K) {
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int blocks_per_row = K / 32;
    if (idx >= size_t((rows + 127) / 128 * 128) * blocks_per_row) return;
    const int r = int(idx / blocks_per_row), b = int(idx % blocks_per_row);
    if (r >= rows) {                                            // a row the tensor does not have: a zero block's scale
        scales[scale_byte_offset(r, b, K / 2)] = 0u;
        return;
    }
    const T* p = x + size_t(r) * K + size_t(b) * 32;
    float v[32];
    if constexpr (sizeof(T) == 4) {
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 f = __ldg(reinterpret_cast<const float4*>(p) + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    } else {
        #pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(p) + i);
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[8 * i + 2 * j] = PairFormat<T>::type::widen(w[j] & 0xFFFFu);
                v[8 * i + 2 * j + 1] = PairFormat<T>::type::widen(w[j] >> 16);
            }
        }
    }
    uint32_t mx = 0;
    #pragma unroll
    for (int i = 0; i < 32; ++i) mx = max(mx, __float_as_uint(v[i]) & 0x7FFFFFFFu);
    uint4* out = reinterpret_cast<uint4*>(packed + size_t(r) * (K / 2) + size_t(b) * 16);
    // the scale of (row, block of 32) sits where the VEC16 layout of a K/2-wide tensor puts (row, block of 16)
    uint8_t* sbyte = scales + scale_byte_offset(r, b, K / 2);
    if (mx >= 0x7F800000u) {
        *out = make_uint4(0x77777777u, 0x77777777u, 0x77777777u, 0x77777777u);
        *sbyte = 0xFFu;
        return;
    }
    int e = mx ? ilogbf(__uint_as_float(mx)) - 2 : -127;
    e = min(max(e, -127), 127);
    const float inv = scalbnf(1.0f, -e);
    uint32_t words[4];
    #pragma unroll
    for (int h = 0; h < 4; ++h) {
        float q[8];
        uint32_t signs = 0;
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float t = __fmul_rn(v[8 * h + i], inv);
            q[i] = fabsf(t);
            signs |= t < 0.0f ? (8u << (4 * i)) : 0u;
        }
        words[h] = e2m1x8_from_quotients(q) | signs;
    }
    *out = make_uint4(words[0], words[1], words[2], words[3]);
    *sbyte = static_cast<uint8_t>(e + 127);
}

// MXFP4 bytes -> FP32 [rows, K]; one thread per block of 32 (the check path).
__global__ void __launch_bounds__(256)
dequantise_mx_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales, float* __restrict__ out,
                     int rows, int K) {
    const size_t idx = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    const int blocks_per_row = K / 32;
    if (idx >= size_t(rows) * blocks_per_row) return;
    const int r = int(idx / blocks_per_row), b = int(idx % blocks_per_row);
    const uint32_t sb = scales[scale_byte_offset(r, b, K / 2)];
    const float s = sb == 0xFFu ? __uint_as_float(0x7FC00000u) : scalbnf(1.0f, int(sb) - 127);
    const uint4 p = __ldg(reinterpret_cast<const uint4*>(packed + size_t(r) * (K / 2) + size_t(b) * 16));
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
    float* dst = out + size_t(r) * K + size_t(b) * 32;
    #pragma unroll
    for (int h = 0; h < 4; ++h)
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t c = (w[h] >> (4 * i)) & 15u, m = c & 7u;
            const float level = m < 2u ? 0.5f * m : __uint_as_float(((126u + (m >> 1)) << 23) | ((m & 1u) << 22));
            dst[8 * h + i] = level * (1.0f - 2.0f * static_cast<float>(c >> 3)) * s;
        }
}

}  // namespace

void check_quant_shape(int rows, int K) {
    if (rows <= 0 || K <= 0) throw std::invalid_argument("nvfp4 quantise: rows and K must be positive");
    if (K % 64 != 0) throw std::invalid_argument("nvfp4 quantise: K must be a multiple of 64");
}

void quantise(const void* x, int dtype, uint8_t* packed, uint8_t* scales, int rows, int K, cudaStream_t stream) {
    check_quant_shape(rows, K);
    if (!x || !packed || !scales) throw std::invalid_argument("nvfp4 quantise: null pointer");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(scales)) & 15)
        throw std::invalid_argument("nvfp4 quantise: pointers must be 16-byte aligned");
    // 256-column tiles; 128-column ones when the grid would otherwise be less than two waves of resident CTAs
    // (four per SM). Measured, 128 / 256 columns: 4096 x 4096 bf16 12.3 / 14.4 us, 8192 x 8192 36.9 / 34.0 us.
    int device = 0, sms = 0;
    cuda_check(cudaGetDevice(&device));
    cuda_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const long long wide_ctas = (long long)((K + 255) / 256) * (rows / Q_ROWS);
    const bool narrow = K % 128 == 0 && wide_ctas < 2LL * 4 * sms;
    auto launch = [&](auto tag) {
        using T = decltype(tag);
        const int full = rows / Q_ROWS;                         // whole row tiles; a last partial one goes to the TAIL instance
        if (narrow) {
            if (full) quantise_kernel<T, 128><<<dim3(K / 128, full), Q_THREADS, 0, stream>>>(static_cast<const T*>(x), packed, scales, rows, K, 0);
            if (rows % Q_ROWS) quantise_kernel<T, 128, true><<<dim3(K / 128, 1), Q_THREADS, 0, stream>>>(static_cast<const T*>(x), packed, scales, rows, K, full);
        } else {
            if (full) quantise_kernel<T, 256><<<dim3((K + 255) / 256, full), Q_THREADS, 0, stream>>>(static_cast<const T*>(x), packed, scales, rows, K, 0);
            if (rows % Q_ROWS) quantise_kernel<T, 256, true><<<dim3((K + 255) / 256, 1), Q_THREADS, 0, stream>>>(static_cast<const T*>(x), packed, scales, rows, K, full);
        }
    };
    switch (dtype) {
        case DTYPE_BF16: launch(__nv_bfloat16{}); break;
        case DTYPE_F16: launch(__half{}); break;
        case DTYPE_F32: launch(float{}); break;
        default:
            throw std::invalid_argument("nvfp4 quantise: dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)");
    }
    cuda_check(cudaGetLastError());
}

void quantise_scaled(const void* x, int dtype, float inv_global, uint8_t* packed, uint8_t* scales, int rows, int K,
                     cudaStream_t stream) {
    check_quant_shape(rows, K);
    if (!x || !packed || !scales) throw std::invalid_argument("nvfp4 quantise: null pointer");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(scales)) & 15)
        throw std::invalid_argument("nvfp4 quantise: pointers must be 16-byte aligned");
    if (!(inv_global > 0.0f) || !(inv_global < 3.0e38f)) throw std::invalid_argument("nvfp4 quantise: the tensor scale must be positive and finite");
    const dim3 grid((K + 255) / 256, (rows + Q_ROWS - 1) / Q_ROWS);
    switch (dtype) {
        case DTYPE_BF16:
            quantise_scaled_kernel<<<grid, Q_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), inv_global, packed, scales, rows, K);
            break;
        case DTYPE_F16:
            quantise_scaled_kernel<<<grid, Q_THREADS, 0, stream>>>(static_cast<const __half*>(x), inv_global, packed, scales, rows, K);
            break;
        case DTYPE_F32:
            quantise_scaled_kernel<<<grid, Q_THREADS, 0, stream>>>(static_cast<const float*>(x), inv_global, packed, scales, rows, K);
            break;
        default:
            throw std::invalid_argument("nvfp4 quantise: dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)");
    }
    cuda_check(cudaGetLastError());
}

void check_mx_shape(int rows, int K) {
    if (rows <= 0 || K <= 0) throw std::invalid_argument("mxfp4: rows and K must be positive");
    if (K % 128 != 0) throw std::invalid_argument("mxfp4: K must be a multiple of 128 (one scale atom covers 4 blocks of 32)");
}

void quantise_mx(const void* x, int dtype, uint8_t* packed, uint8_t* scales, int rows, int K, cudaStream_t stream) {
    check_mx_shape(rows, K);
    if (!x || !packed || !scales) throw std::invalid_argument("mxfp4 quantise: null pointer");
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(scales)) & 15)
        throw std::invalid_argument("mxfp4 quantise: pointers must be 16-byte aligned");
    const size_t blocks = size_t((rows + 127) / 128 * 128) * (K / 32);    // the rows of the last atom the tensor lacks get their scale byte
    const unsigned grid = static_cast<unsigned>((blocks + 255) / 256);
    switch (dtype) {
        case DTYPE_BF16: quantise_mx_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), packed, scales, rows, K); break;
        case DTYPE_F16: quantise_mx_kernel<<<grid, 256, 0, stream>>>(static_cast<const __half*>(x), packed, scales, rows, K); break;
        case DTYPE_F32: quantise_mx_kernel<<<grid, 256, 0, stream>>>(static_cast<const float*>(x), packed, scales, rows, K); break;
        default: throw std::invalid_argument("mxfp4 quantise: dtype must be 0 (bf16), 1 (fp16) or 2 (fp32)");
    }
    cuda_check(cudaGetLastError());
}

void dequantise_mx(const uint8_t* packed, const uint8_t* scales, float* out, int rows, int K, cudaStream_t stream) {
    check_mx_shape(rows, K);
    if (!packed || !scales || !out) throw std::invalid_argument("mxfp4 dequantise: null pointer");
    const size_t blocks = size_t(rows) * (K / 32);
    dequantise_mx_kernel<<<static_cast<unsigned>((blocks + 255) / 256), 256, 0, stream>>>(packed, scales, out, rows, K);
    cuda_check(cudaGetLastError());
}

void dequantise(const uint8_t* packed, const uint8_t* scales, float* out, int rows, int K, cudaStream_t stream) {
    check_quant_shape(rows, K);
    if (!packed || !scales || !out) throw std::invalid_argument("nvfp4 dequantise: null pointer");
    const size_t blocks = size_t(rows) * (K / 16);
    dequantise_kernel<<<static_cast<unsigned>((blocks + 255) / 256), 256, 0, stream>>>(packed, scales, out, rows, K);
    cuda_check(cudaGetLastError());
}

}  // namespace nvfp4_b200
