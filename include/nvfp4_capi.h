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
 * plan and must outlive it. Not capture-safe.
 * Shapes: K % 64 == 0, N % 8 == 0, any M >= 1 (the reference wants multiples of 256 in all three,
 * include/nvfp4.h:11). The scale arrays always end in whole atoms: ceil(rows/128)*128 * K/16 bytes; what the
 * bytes of the rows beyond M (or N) hold does not matter. A plan whose M or N is no multiple of 128 has plain
 * launches only (no split_k, gather, profile). */
int gpu_kernels_nvfp4_plan_create(void** plan, int M, int N, int K, const void* A, const void* B,
                                  const void* SFA, const void* SFB, void* workspace, size_t workspace_bytes,
                                  void* stream);
/* replaces nvfp4_bridge.cu:94-96 */
void gpu_kernels_nvfp4_plan_destroy(void* plan);
/* replaces nvfp4_bridge.cu:98-110: cuBLASLt NVFP4 matmul on the same operands (comparison only) */
int gpu_kernels_nvfp4_cublas(void* plan, void* C, const void* A, const void* B, void* stream);
/* replaces nvfp4_bridge.cu:112-121: C[M,N] fp16 = A * B^T with this library's kernel; capture-safe */
int gpu_kernels_nvfp4_custom(void* plan, void* C, void* stream);
/* replaces nvfp4_bridge.cu:123-132: synchronises and reports a kernel that gave up waiting or skipped an
 * out-of-range store. Every plan reports to a status slot of its own, so this call neither reports nor clears
 * another plan's error. plan may be NULL: checks every slot of the current device (this is how grouped
 * launches and the expert-path kernels, which report to the device's own slot, are checked). */
int gpu_kernels_nvfp4_validate(void* plan);
/* replaces nvfp4_bridge.cu:134-139 */
int gpu_kernels_nvfp4_l2_bytes(void);

/* ---- entry points the reference only has in Python (reference/python/nvfp4.py) ---- */

/* replaces reference/python/nvfp4.py:30-37 `quantize` (+ :17-21 `pack_scales`, :6-14 `encode_e2m1`).
 * x [rows,K] device, dtype 0 = bf16, 1 = fp16, 2 = fp32; packed [rows,K/2]; scales ceil(rows/128)*128 * K/16 bytes.
 * K % 64 == 0. Bit-exact with the reference on finite and non-finite input. The reference wants rows % 128 == 0
 * (reference/python/nvfp4.py:20); for another row count the result is the reference's for the tensor with zero
 * rows appended up to the next multiple of 128 (their scale bytes are 0x01, a zero block's), with the packed array
 * cut back to `rows` rows. */
int gpu_kernels_nvfp4_quantize(const void* x, int dtype, void* packed, void* scales, int rows, int K, void* stream);
/* Two-level scaling (no counterpart in the reference, whose quantiser has the block scales only): the same as
 * gpu_kernels_nvfp4_quantize applied to fp32(x) * inv_tensor_scale (one FP32 product per value), i.e.
 * reference `quantize(values.float() * inv_tensor_scale)`. With tensor scales gA, gB (typically amax / (6 * 448), so
 * that the block scales use the whole E4M3 range) the product is recovered by alpha = gA * gB
 * (gpu_kernels_nvfp4_plan_set_alpha). Bit-exact with that definition. */
int gpu_kernels_nvfp4_quantize_scaled(const void* x, int dtype, float inv_tensor_scale, void* packed, void* scales, int rows,
                                      int K, void* stream);
/* replaces reference/python/nvfp4.py:40-47 `dequantize`: FP32 [rows,K] out. */
int gpu_kernels_nvfp4_dequantize(const void* packed, const void* scales, void* out_f32, int rows, int K, void* stream);

/* ---- MXFP4: the adjacent format of the same instruction (no counterpart in the reference, whose kernel is
 *      scale_vec::4X only, kernels/gemm/matmul/sm100.cu:341-342). OCP microscaling: E2M1 values packed as above, one
 *      UE8M0 power-of-two scale per 32 values along K, in cuBLASLt's VEC32 order: the same 512-byte atoms of 128 rows x
 *      4 scales, ordered [row/128][k/128]. K % 128 == 0; scale arrays of ceil(rows/128)*128 * K/32 bytes. ---- */

/* Per block of 32: e = floor(log2(amax)) - 2 clamped to [-127, 127], scale byte e + 127, codes = E2M1 of x * 2^-e with
 * the NVFP4 quantiser's rounding (nearest, ties to the even code, saturating at 6) and sign rule (bit 3 = q < 0); an
 * all-zero block takes e = -127; a block holding a NaN or an infinity takes scale byte 0xFF and codes 0x7. */
int gpu_kernels_nvfp4_quantize_mx(const void* x, int dtype, void* packed, void* scales, int rows, int K, void* stream);
/* level * sign * 2^(byte - 127) -> FP32 [rows,K]; scale byte 0xFF gives NaN. */
int gpu_kernels_nvfp4_dequantize_mx(const void* packed, const void* scales, void* out_f32, int rows, int K, void* stream);
/* A plan like gpu_kernels_nvfp4_plan_create's for MXFP4 operands (tcgen05.mma ... block_scale.scale_vec::2X with
 * UE8M0 scales); run it with gpu_kernels_nvfp4_custom, check it with gpu_kernels_nvfp4_validate, free it with
 * gpu_kernels_nvfp4_plan_destroy. Options alpha, group_m, k_skew, out_bf16, pdl, static_operands, l2_side apply;
 * split_k, the gather and the cuBLASLt comparison do not. */
int gpu_kernels_nvfp4_plan_create_mx(void** plan, int M, int N, int K, const void* A, const void* B, const void* SFA,
                                     const void* SFB, void* stream);

/* Activations that arrive in bf16 / fp16 / fp32 (no counterpart in the reference, which quantises in PyTorch before
 * it builds a plan): quantises x [M,K] (dtype as gpu_kernels_nvfp4_quantize) into the plan's own A and SFA buffers
 * (the pointers given to plan_create, which the caller therefore leaves to the plan) and runs the GEMM behind it on
 * the same stream. B and SFB are taken to be weights nothing on the stream writes: the GEMM starts under
 * programmatic dependent launch while the quantiser runs, requests its first tiles of B and waits for the
 * quantiser only before it reads A. Asynchronous, capture-safe. */
int gpu_kernels_nvfp4_linear(void* plan, const void* x, int dtype, void* C, void* stream);

/* ---- extensions of the plan ---- */

/* FP32 global scale: C = fp16(alpha * accumulator). The reference fixes alpha = 1 (nvfp4_bridge.cu:101). */
int gpu_kernels_nvfp4_plan_set_alpha(void* plan, float alpha);
/* Tuning knobs. key: "group_m" (tile rows per rasterisation band, >= 1); "c_evict_first" (0/1: L2 policy
 * of the C stores); "direct_store" (0/1: epilogue writes C from registers instead of staging it for TMA stores);
 * "ragged_tiles" (T: deal the columns of a plan with M = 128, in units of 64, to T single-CTA tiles of two widths
 * (2/3 or 3/4 units) instead of N/256 tiles of 256 columns, e.g. T = the SM count where N/256 tiles would leave SMs idle; 0 = uniform
 * tiles, the default);
 * "pdl" (0/1, default 1: launches carry the programmatic stream-serialisation attribute, so that this kernel's
 * set-up overlaps the tail of the kernel in front of it in the stream; 0 = ordinary launches);
 * "static_operands" (0/1/2, default 0: the caller's promise about the kernel that runs in front of each launch
 * on the stream, used only with "pdl": 1 = that kernel does not write B or SFB (weights): this launch fetches its
 * first B tiles while that kernel drains; 2 = it writes none of A, B, SFA, SFB (a chain of independent GEMMs, or
 * inputs that were produced earlier): this launch computes its tiles while that kernel's last tiles finish and
 * only holds back its stores of C until that kernel has completed; ignored by split-K launches);
 * "out_bf16" (0/1: C is written as bfloat16 instead of FP16 through the same pointer; the reference's output
 * is FP16 only, include/nvfp4.h:21); "l2_side" (0/1: L2-side-aware tile order, the counterpart of the
 * reference's prepare_schedule, kernels/gemm/matmul/sm100.cu:566-673: a census at this call labels the SMs by
 * the side of the L2 they sit on and deals each side one contiguous part of the tile sequence; fails when the
 * plan's grid does not fill the GPU or the census finds no two sides; results never depend on it; not inside
 * stream capture);
 * "k_skew" (>= 0: tile t starts its K walk at step (t * k_skew) % steps; 0 = every tile at K = 0);
 * "split_k" (0/1, default 0: four units per tile, each with a quarter of the K steps, partial sums combined
 * through a workspace the plan allocates. Offered for shapes with at most a quarter as many tiles as SMs and
 * at least 16 K steps of 256 (10-13 % faster there); refused for others. The units of such a launch wait
 * for each other, so the GPU's SMs must not be held by other kernels; a wait that runs out is reported by
 * validate. Not inside stream capture: switching it on may allocate and clears flags). */
int gpu_kernels_nvfp4_plan_set_option(void* plan, const char* key, int value);
/* The GEMM fused with the all-gather of C (N sharded over the GPUs of one NVLink node; no counterpart in the
 * reference, whose GEMM is single-GPU): the plan's [M, N] result is the column slab [col0, col0 + N) of a
 * full [M, n_total] FP16 matrix, and every later gpu_kernels_nvfp4_custom(plan, C, stream) writes that slab
 * from its epilogue into ALL `world` buffers (host array of device pointers: this rank's full C and the
 * peers', opened with gpu_kernels_nvfp4_ipc_open); nothing is written through C then (still a valid device
 * pointer of M * N elements, e.g. this rank's buffer). The caller puts a
 * barrier between the ranks before reading, and before the next launch overwrites. world = 0 switches it
 * off. Not inside stream capture (synchronises once). */
int gpu_kernels_nvfp4_plan_set_gather(void* plan, void* const* buffers, int world, int col0, int n_total);
/* Fills info[0..15] = {M, N, K, units, cta_group, tile_n, group_m, stages, split_k, k_skew, direct_store,
 * out_bf16, l2_side order in use, clusters on L2 side 0, on side 1, ragged tiles (0 = uniform tiling)}. */
int gpu_kernels_nvfp4_plan_info(void* plan, int* info);

/* With the "l2_side" order: how many clusters, summed over this plan's launches, found themselves on the
 * other side of the L2 than the plan's tile route assumed (they lose locality, nothing else). Synchronising copy. */
int gpu_kernels_nvfp4_plan_placement_misses(void* plan, unsigned* misses);
/* Host arithmetic of the "l2_side" order (no GPU involved): unit_side[u] in {0, 1} for the `units` persistent
 * units of a grid; route[w] (w < tiles) = the tile that work item w (= unit + trip * units) computes. The
 * units of side 0 share the first part of the tile sequence, those of side 1 the rest, each part as long as
 * its side's share of the work; every trip of a side is a dense run of its part. Always a permutation. */
int gpu_kernels_nvfp4_side_route(const unsigned char* unit_side, int units, int tiles, unsigned* route);
/* Diagnostic: cycles per dependent atomic that every SM of the current device measured in the L2-side census,
 * indexed by SM id (0 = no CTA ran there); *written = 0 when no census has run on this device yet. */
int gpu_kernels_nvfp4_l2_census(unsigned* cycles_by_sm, int capacity, int* written);

/* Diagnostic: one launch with per-role wait counters on; writes 16 words per CTA
 * {producer wait, producer total, MMA wait-for-data, MMA wait-for-accumulator, MMA total, epilogue
 * wait-for-accumulator, epilogue wait-for-store, epilogue total, SM id, ...} in SM clock cycles.
 * Allocates and frees a small device buffer and synchronises the stream. */
int gpu_kernels_nvfp4_plan_profile(void* plan, void* C, void* stream, unsigned long long* counters, int max_words,
                                   int* words_written);

/* Diagnostic: SM clock cycles that the first CTA of the most recent finished GEMM launch on the current
 * device spent inside the kernel (synchronising copy of one word); 0 on error. */
unsigned gpu_kernels_nvfp4_last_kernel_cycles(void);

/* Whole GEMM from HOST buffers (pinned memory recommended): copies the four operands to the device, runs
 * the kernel and copies C back, then synchronises. From M = 1024 the product goes in 2 or 4 row pieces and (from
 * N = 1024) as many column pieces: copies in and kernels on `stream` in the order A piece, B piece, block, next B
 * piece, block, ...; every block's result leaves on a second stream of the library's as soon as it is computed,
 * so C starts to travel back after one piece of each operand has arrived and both directions of the host link
 * stay busy. Device staging is cached per device and (M,N,K) inside the library. This is the end-to-end call a
 * host-side user of the reference path would make in place of its CPU dequantise + matmul (benchmarks/nvfp4.py:41). */
int gpu_kernels_nvfp4_gemm_host(int M, int N, int K, const void* A, const void* B, const void* SFA, const void* SFB,
                                void* C, float alpha, void* stream);

/* ---- routed-MoE expert path in NVFP4 (phase structure of the reference's gpu_kernels_moe_phase,
 *      benchmarks/bindings/fused_moe_bridge.cu:11-26: metadata / FC1 / FC2 / reduce; the reference's
 *      kernels are BF16 for sm_90a and move tokens through peer pointers). These move quantised rows, either
 *      by stores into the peers' memory from the dispatch kernel and from FC2's epilogue (quantise_route /
 *      pack_peer, grouped_run_scatter, peer_exchange as the barrier), or through an all-to-all that the caller
 *      runs between pack and unpack. All pointers are device pointers unless said otherwise. ---- */

/* Grouped GEMM: pool A [pool_rows, K/2] of blocks of block_rows (128 or 256) rows, stacked weights
 * B [experts*n, K/2] (+ scales); block i multiplies expert block_expert[i]; *num_blocks blocks are live (device
 * values, read by the kernel). 128-row blocks run on single CTAs, 256-row blocks on CTA pairs (for experts with
 * many rows). C [pool_rows, n], fp16 or bf16. Replaces the two WGMMA phases of kernels/moe/fused/sm90.cu:209-550. */
int gpu_kernels_nvfp4_grouped_plan_create(void** plan, int pool_rows, int n, int k, int experts, int block_rows,
                                          const void* A, const void* B, const void* SFA, const void* SFB,
                                          const void* block_expert, const void* num_blocks);
void gpu_kernels_nvfp4_grouped_plan_destroy(void* plan);
/* block_valid: device array from the plan kernel (real rows per block), or NULL. With it gpu_kernels_nvfp4_grouped_run
 * writes only the real rows of C: the padding rows of a pool of 128- or 256-row blocks (most of the pool when an
 * expert sees a few rows) stay out of HBM, and the caller must not read them. */
int gpu_kernels_nvfp4_grouped_set_valid_rows(void* plan, const void* block_valid);
int gpu_kernels_nvfp4_grouped_run(void* plan, void* C, int out_bf16, void* stream);

/* The first expert GEMM with the activation fused into its epilogue (FC1 + kernels/moe/swiglu.cu:12-26 + the
 * re-quantisation for FC2 in one kernel): the plan's B must hold each expert's W1 with rows interleaved as
 * 16 gate rows, 16 up rows, 16 gate rows, ...; writes act_packed [pool_rows, n/4] and act_scales (VEC16 layout
 * of [pool_rows, n/2]) instead of C. row_weight f32 [pool_rows], 0 marks a padding row. */
int gpu_kernels_nvfp4_grouped_run_swiglu(void* plan, const void* row_weight, float clamp, void* act_packed,
                                         void* act_scales, void* stream);

/* The second expert GEMM fused with the combine: instead of C, pool row r is written (bf16 or fp16, from the
 * epilogue while the GEMM runs: register stores for 128-row blocks, one 512-byte bulk copy per row and tile
 * from shared memory for 256-row blocks) to row (row_dst[r] & 0xFFFFFF) - 1 of slots[row_dst[r] >> 24], a
 * [slot_rows, n] buffer per rank: this rank's own, or a peer's mapped through gpu_kernels_nvfp4_ipc_open, in
 * which case the stores cross NVLink. row_dst[r] == 0 marks a padding row. Out-of-range destinations are
 * skipped and reported by gpu_kernels_nvfp4_validate. Replaces FC2 + the peer scatter of
 * kernels/moe/fused/sm90.cu:514-544. slots: DEVICE array of `world` buffer addresses (8 bytes each);
 * own_slots: this rank's own buffer (= slots[rank]). */
int gpu_kernels_nvfp4_grouped_run_scatter(void* plan, const void* row_dst, const void* slots, void* own_slots, int world,
                                          int slot_rows, int out_bf16, void* stream);

/* Bytes of one dispatched token row: hidden/2 packed + hidden/16 scale bytes + 16 (route weight). */
int gpu_kernels_nvfp4_moe_payload_bytes(int hidden);
/* replaces metadata_kernel's histogram (kernels/moe/fused/sm90.cu:43-101): counts[e] += routes to global expert e
 * (ids int64 [routes]); counts must be zeroed by the caller. */
int gpu_kernels_nvfp4_moe_route_count(const void* ids, int routes, int experts, void* counts, void* stream);
/* replaces offsets_kernel (sm90.cu:103-119): counts_matrix int32 [world, experts] (all ranks' counts) ->
 * send_offset [experts+1], seg_src_offset [world*local+1], seg_pool_offset [world*local],
 * block_expert [capacity_rows/block_rows], num_blocks [1], totals [3] = {rows received, pool rows used, overflow};
 * peer_offset [experts] (may be null): where this rank's rows for each global expert start in the receive
 * buffer of the rank that owns it, for gpu_kernels_nvfp4_moe_pack_peer; with peer_to_pool != 0 instead the row of
 * that rank's POOL where they start (every rank can do the owner's layout arithmetic from the gathered counts), for
 * the dispatch that writes packed rows straight into the pools. cursor [experts] (may be null): the arrival
 * counters of the dispatch kernels, zeroed here. block_valid [capacity_rows/block_rows] (may be null): the number
 * of real rows at the head of every live block, for gpu_kernels_nvfp4_grouped_set_valid_rows. */
int gpu_kernels_nvfp4_moe_plan(const void* counts_matrix, int world, int rank, int experts, int capacity_rows,
                               int block_rows, void* send_offset, void* seg_src_offset, void* seg_pool_offset, void* block_expert,
                               void* num_blocks, void* totals, void* peer_offset, int peer_to_pool, void* cursor, void* block_valid,
                               void* stream);
/* One rank (nothing to exchange): histogram of the routes (ids int64 [routes] -> counts int32 [experts], written
 * here) and the plan above in ONE launch, which also zeroes cursor [experts], the arrival counters of the
 * dispatch kernels. Replaces a memset, route_count, a copy, plan and another memset. */
int gpu_kernels_nvfp4_moe_route_plan(const void* ids, int routes, void* counts, int experts, int capacity_rows, int block_rows,
                                     void* send_offset, void* seg_src_offset, void* seg_pool_offset, void* block_expert,
                                     void* num_blocks, void* totals, void* cursor, void* block_valid, void* stream);
/* Clears scale bytes, route weights and (if not null) destination codes of the pool rows of the live blocks
 * (num_blocks [1] on the device, from the plan), so that padding rows contribute nothing; rows beyond the live
 * blocks are not touched. pool_rows: allocated rows (multiple of 128). Run between the plan and the dispatch. */
int gpu_kernels_nvfp4_moe_clear_live(const void* num_blocks, int block_rows, int pool_rows, int hidden, void* pool_scales,
                                     void* pool_weight, void* pool_dst, void* stream);
/* quantised tokens (xq [T_pad, hidden/2], xs VEC16 scales), ids int64 [T, topk], weights f32 [T, topk] ->
 * send_rows [T*topk, payload] ordered by destination expert; send_pos [T*topk] = row of each route (-1 for a
 * route whose expert id lies outside [0, experts): it is dropped, i.e. adds nothing to its token's result);
 * cursor int32 [experts] zeroed by the caller. */
int gpu_kernels_nvfp4_moe_pack(const void* xq, const void* xs, const void* ids, const void* weights, int tokens,
                               int topk, int hidden, int experts, const void* send_offset, void* cursor, void* send_rows,
                               void* send_pos, void* stream);
/* Single-rank shortcut (world = 1): the same as pack + unpack in one kernel, rows written straight into the pool;
 * route_row [T*topk] receives each route's pool row, so reduce can read the second GEMM's output directly
 * (pass the output pool as `returned` and route_row as `send_pos`). seg_pool_offset from moe_plan. */
int gpu_kernels_nvfp4_moe_pack_to_pool(const void* xq, const void* xs, const void* ids, const void* weights, int tokens,
                                       int topk, int hidden, int experts, const void* seg_pool_offset, void* cursor,
                                       void* pool_packed, void* pool_scales, void* pool_weight, void* route_row,
                                       void* stream);
/* received rows (source-major) -> expert-major pool: packed rows, scale atoms (zeroed by the caller first),
 * per-row route weight, pool_of_recv [recv_capacity] for the way back, and (if not null; rows packed by
 * pack_peer only) pool_dst [pool_rows] = (source rank << 24) | (route index + 1) for grouped_run_scatter;
 * the caller zeroes pool_dst first so that padding rows read 0. */
int gpu_kernels_nvfp4_moe_unpack(const void* recv_rows, int recv_capacity, const void* totals, int world,
                                 int local_experts, int hidden, const void* seg_src_offset, const void* seg_pool_offset,
                                 void* pool_packed, void* pool_scales, void* pool_weight, void* pool_of_recv,
                                 void* pool_dst, void* stream);
/* replaces kernels/moe/swiglu.cu:12-26 fused with the re-quantisation for the second GEMM:
 * gate_up bf16 [pool_rows, 2*intermediate] -> NVFP4 activation [pool_rows, intermediate/2] + scales. */
int gpu_kernels_nvfp4_moe_swiglu_quant(const void* gate_up, const void* pool_weight, const void* num_blocks,
                                       int block_rows, int pool_rows, int intermediate, float clamp, void* act_packed,
                                       void* act_scales, void* stream);
/* expert outputs bf16 [pool_rows, hidden] -> rows in the order they were received (for the all-to-all back). */
int gpu_kernels_nvfp4_moe_return_rows(const void* out_pool, const void* pool_of_recv, const void* totals, int capacity,
                                      int hidden, void* return_rows, void* stream);
/* replaces reduce_kernel (sm90.cu:121-139): y[t] = bf16(sum_j fp32(returned[send_pos[t*topk+j]])), j ascending.
 * Routes with send_pos < 0, or (ids int64 [T*topk] not NULL) an expert id outside [0, experts), are skipped. */
int gpu_kernels_nvfp4_moe_reduce(const void* returned, const void* send_pos, int tokens, int topk, int hidden, void* y,
                                 const void* ids, int experts, void* stream);

/* No counterpart in the reference. The same whole GEMM from HOST buffers as gpu_kernels_nvfp4_gemm_host,
 * for callers that must not allocate device memory while they run (a process whose memory pool owns
 * the GPU and forbids later cudaMalloc, or a phase of a program in which allocation is not allowed):
 * the device copies of A, B, the scales and C live in one array built into the library instead of
 * cudaMalloc'ed buffers, and the call itself allocates nothing. Limits: M <= 512, N <= 1024, K <= 2048
 * (plus the usual multiples of 128 / 128 / 256); larger shapes are refused with a message. The array
 * (2.7 MiB) is held on every GPU that loads the library until the process exits. The first call on
 * each device looks up the array's device address (make that call before any stream capture begins);
 * every call shares the array, which keeps the previous call's data; calls that overlap on the GPU,
 * from several threads or streams, would race on it, so the library serialises them and each call
 * synchronises `stream` before it returns. */
int gpu_kernels_nvfp4_gemm_host_static(int M, int N, int K, const void* A, const void* B, const void* SFA,
                                       const void* SFB, void* C, float alpha, void* stream);

/* Expert parallelism over peer memory: the fused replacement of pack + all-to-all and of return_rows +
 * all-to-all. The reference moves tokens the same way, by device-initiated peer loads and stores
 * (kernels/moe/fused/sm90.cu:296-319 pulls, :532-541 pushes); here both directions are stores.
 * pack_peer writes each route's quantised row (+ weight and route index) straight into the receive buffer
 * of the rank that owns its expert; return_peer writes each expert output row straight into slot
 * [route] of the [T*topk, hidden] bf16 buffer of the rank the token came from. peer_recv / peer_slots are
 * host arrays of `world` device pointers (this process's mappings of every rank's buffer, own included).
 * Every peer write is bounds-checked against the capacities (rows); a violation sets *error (device int)
 * and skips the write. The caller must put a stream-ordered collective between pack_peer and unpack, and
 * between return_peer and reduce (and nothing here waits on another GPU). */
/* Token quantisation fused with the dispatch (one CTA per token; replaces quantize + pack_peer, or quantize +
 * pack_to_pool, with the same bits): x [tokens, hidden] bf16 is quantised row by row in shared memory and each
 * route's row (codes, scale bytes, weight, route index) goes straight to its expert. world > 0: into
 * peer_recv[expert / local_experts] (host array of `world` device pointers) at row offsets[expert] + arrival
 * order, refused and flagged in `error` beyond recv_capacity; with peer_meta (another such array) not null,
 * peer_recv are the ranks' POOLS (packed rows, hidden/2 bytes each) and the row's scale bytes, weight and route
 * index go to row offsets[expert] + arrival order of peer_meta[owner] (hidden/16 + 16 bytes per row), for
 * gpu_kernels_nvfp4_moe_unpack_meta on the owner. world == 0: into this rank's pool (packed rows, VEC16 scale
 * atoms, weights) at row offsets[expert] + arrival order, which route_row [tokens * topk] records. */
int gpu_kernels_nvfp4_moe_quantise_route(const void* x_bf16, const void* ids, const void* weights, int tokens, int topk,
                                         int hidden, int experts, const void* offsets, void* cursor, void* const* peer_recv,
                                         void* const* peer_meta, int world, int local_experts, int recv_capacity, void* error,
                                         void* pool_packed, void* pool_scales, void* pool_weight, void* route_row, void* stream);
/* The receiving side of that dispatch: for each received row (recv_capacity bounds their number, totals[0] on the
 * device gives it) lays the scale bytes from `side` into the pool's scale atoms and fills pool_weight and
 * pool_dst = (source rank << 24) | (route index + 1). seg_src_offset / seg_pool_offset: the plan's tables. */
int gpu_kernels_nvfp4_moe_unpack_meta(const void* side, int recv_capacity, const void* totals, int world, int local_experts,
                                      int hidden, const void* seg_src_offset, const void* seg_pool_offset, void* pool_scales,
                                      void* pool_weight, void* pool_dst, void* stream);
int gpu_kernels_nvfp4_moe_pack_peer(const void* xq, const void* xs, const void* ids, const void* weights, int tokens,
                                    int topk, int hidden, int world, int local_experts, const void* peer_offset,
                                    void* cursor, void* const* peer_recv, int recv_capacity, void* error, void* stream);
int gpu_kernels_nvfp4_moe_return_peer(const void* out_pool, const void* recv_rows, const void* pool_of_recv,
                                      const void* totals, const void* seg_src_offset, int world, int local_experts,
                                      int hidden, int recv_capacity, void* const* peer_slots, int slot_capacity,
                                      void* error, void* stream);
/* Barrier, or barrier plus all-gather of a few integers, between the GPUs of one NVLink node without a
 * collective library: one small kernel per rank that stores into the peers' memory and waits (at most 2 s,
 * then validate reports it) for their stores. Every rank owns a state block of peer_state_bytes(world,
 * max_ints) bytes from gpu_kernels_nvfp4_ipc_alloc (zeroed) that all ranks map; `peers_device` is a DEVICE
 * array of the world blocks' addresses in rank order (own = entry `rank`). After the call completes on a
 * rank's stream, everything every rank had stored into peer memory before ITS call (on its stream) is visible
 * there. ints > 0: `payload` [ints] of each rank arrives in `out` [world][ints] on every rank. All ranks call
 * it the same number of times, each on its own GPU (never two ranks on one GPU). Capturable in a CUDA graph.
 * No counterpart in the reference (its peer signalling is inside kernels/moe/fused/sm90.cu:296-319). */
int gpu_kernels_nvfp4_peer_state_bytes(int world, int max_ints, size_t* bytes);
/* The count all-gather of the expert layer in one launch for small batches: the histogram of this rank's routes
 * (ids int64 [routes], `experts` <= 4096 bins) is taken inside the exchange kernel and arrives, with every
 * other rank's, in counts_matrix int32 [world, experts]. Arguments as gpu_kernels_nvfp4_peer_exchange. */
int gpu_kernels_nvfp4_moe_count_exchange(const void* ids, int routes, int experts, void* own, const void* peers_device, int world,
                                         int rank, int max_ints, void* counts_matrix, void* stream);
int gpu_kernels_nvfp4_peer_exchange(void* own, const void* peers_device, int world, int rank, const void* payload, int ints,
                                    int max_ints, void* out, void* stream);

/* Device memory that the other processes of the box can map: ipc_alloc = cudaMalloc (zeroed) + a 64-byte handle
 * to hand to the peers; ipc_open maps a peer's handle (lazy peer access); ipc_close / ipc_free undo them. */
int gpu_kernels_nvfp4_ipc_alloc(size_t bytes, void** ptr, void* handle64);
int gpu_kernels_nvfp4_ipc_open(const void* handle64, void** ptr);
int gpu_kernels_nvfp4_ipc_close(void* ptr);
int gpu_kernels_nvfp4_ipc_free(void* ptr);

/* Library version string and the number of kernels this library has launched so far in this process. */
const char* gpu_kernels_nvfp4_version(void);
unsigned long long gpu_kernels_nvfp4_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
