/* C ABI of libgpu_kernels_nvfp4_bench.so (B200 / sm_100a only).
 *
 * Plain pointers and sizes; no exception crosses this boundary. Every function
 * that returns int returns 0 on success and 1 on failure, after storing a
 * message that gpu_kernels_nvfp4_last_error() returns (thread-local), as the
 * reference's bridge does (benchmarks/bindings/nvfp4_bridge.cu:11,41-43,88-91).
 * Streams are passed as void* (cudaStream_t). All device pointers must be
 * 16-byte aligned. There is no CPU fallback: on a machine without an sm_100
 * GPU every compute entry point fails with an error.
 */
#ifndef GPU_KERNELS_NVFP4_CAPI_H
#define GPU_KERNELS_NVFP4_CAPI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- the seven symbols the reference's Python harness binds
 *      (benchmarks/nvfp4.py:21-28; defined at benchmarks/bindings/nvfp4_bridge.cu:41-139) ---- */

/* replaces nvfp4_bridge.cu:41-43 */
const char* gpu_kernels_nvfp4_last_error(void);
/* replaces nvfp4_bridge.cu:45-92. A [M,K/2], B [N,K/2] packed E2M1; SFA/SFB VEC16 UE4M3 scales;
 * workspace is only used by the cuBLASLt comparison path. Device pointers are baked into the
 * plan and must outlive it. Not capture-safe. */
int gpu_kernels_nvfp4_plan_create(void** plan, int M, int N, int K, const void* A, const void* B,
                                  const void* SFA, const void* SFB, void* workspace, size_t workspace_bytes,
                                  void* stream);
/* replaces nvfp4_bridge.cu:94-96 */
void gpu_kernels_nvfp4_plan_destroy(void* plan);
/* replaces nvfp4_bridge.cu:98-110: cuBLASLt NVFP4 matmul on the same operands (comparison only) */
int gpu_kernels_nvfp4_cublas(void* plan, void* C, const void* A, const void* B, void* stream);
/* replaces nvfp4_bridge.cu:112-121: C[M,N] fp16 = A * B^T with this library's kernel; capture-safe */
int gpu_kernels_nvfp4_custom(void* plan, void* C, void* stream);
/* replaces nvfp4_bridge.cu:123-132: synchronises and reports a kernel that gave up waiting */
int gpu_kernels_nvfp4_validate(void* plan);
/* replaces nvfp4_bridge.cu:134-139 */
int gpu_kernels_nvfp4_l2_bytes(void);

/* ---- entry points the reference only has in Python (reference/python/nvfp4.py) ---- */

/* replaces reference/python/nvfp4.py:30-37 `quantize` (+ :17-21 `pack_scales`, :6-14 `encode_e2m1`).
 * x [rows,K] device, dtype 0 = bf16, 1 = fp16, 2 = fp32; packed [rows,K/2]; scales rows*K/16 bytes.
 * rows % 128 == 0, K % 64 == 0. Bit-exact with the reference on finite and non-finite input. */
int gpu_kernels_nvfp4_quantize(const void* x, int dtype, void* packed, void* scales, int rows, int K, void* stream);
/* replaces reference/python/nvfp4.py:40-47 `dequantize`: FP32 [rows,K] out. */
int gpu_kernels_nvfp4_dequantize(const void* packed, const void* scales, void* out_f32, int rows, int K, void* stream);

/* ---- extensions of the plan ---- */

/* FP32 global scale: C = fp16(alpha * accumulator). The reference fixes alpha = 1 (nvfp4_bridge.cu:101). */
int gpu_kernels_nvfp4_plan_set_alpha(void* plan, float alpha);
/* Tuning knobs. key: "group_m" (tile rows per rasterisation band, >= 1); "c_evict_first" (0/1: L2 policy
 * of the C stores). */
int gpu_kernels_nvfp4_plan_set_option(void* plan, const char* key, int value);
/* Fills info[0..7] = {M, N, K, units, cta_group, tile_n, group_m, stages}. */
int gpu_kernels_nvfp4_plan_info(void* plan, int* info);

/* Diagnostic: one launch with per-role wait counters on; writes 16 words per CTA
 * {producer wait, producer total, MMA wait-for-data, MMA wait-for-accumulator, MMA total, epilogue
 * wait-for-accumulator, epilogue wait-for-store, epilogue total, SM id, ...} in SM clock cycles.
 * Allocates and frees a small device buffer and synchronises the stream. */
int gpu_kernels_nvfp4_plan_profile(void* plan, void* C, void* stream, unsigned long long* counters, int max_words,
                                   int* words_written);

/* Diagnostic: SM clock cycles that the first CTA of the most recent finished GEMM launch on the current
 * device spent inside the kernel (synchronising copy of one word); 0 on error. */
unsigned gpu_kernels_nvfp4_last_kernel_cycles(void);

/* Whole GEMM from HOST buffers: copies the four operands to the device, runs the kernel and copies
 * C back, all on `stream`, then synchronises it. Device staging is cached per (M,N,K) inside the
 * library. This is the end-to-end call a host-side user of the reference path would make in place
 * of its CPU dequantise + matmul (benchmarks/nvfp4.py:41). */
int gpu_kernels_nvfp4_gemm_host(int M, int N, int K, const void* A, const void* B, const void* SFA, const void* SFB,
                                void* C, float alpha, void* stream);

/* Library version string and the number of kernels this library has launched so far in this process. */
const char* gpu_kernels_nvfp4_version(void);
unsigned long long gpu_kernels_nvfp4_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
