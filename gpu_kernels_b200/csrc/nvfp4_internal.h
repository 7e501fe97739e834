// Declarations shared by the translation units of the NVFP4 library (not installed).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace nvfp4_b200 {

enum InputDtype : int { DTYPE_BF16 = 0, DTYPE_F16 = 1, DTYPE_F32 = 2 };

inline void cuda_check(cudaError_t e) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA: ") + cudaGetErrorString(e));
}

// Refuse to run on anything but a compute-capability 10.x device: there is no
// other code path in this library.
void require_sm100();

// nvfp4_schedule.cu: L2-side-aware tile order (tables live in a per-process cache, per device and shape).
struct TileRoute {
    const uint32_t* route;          // [tiles]: work item -> tile of the band order
    const uint8_t* sm_side;         // [256]: L2 side by SM id
    const uint8_t* unit_side;       // [units]: side each unit of the grid was seen on
    int side_units[2];
};
bool l2_side_route(int device, int cta_group, int units, int tiles_m, int tiles_n, int group_m, size_t smem_bytes,
                   cudaStream_t stream, TileRoute& out);
std::vector<uint32_t> build_side_route(const std::vector<uint8_t>& sides, int tiles);
int l2_side_census_cycles(int device, unsigned* out, int capacity);

// nvfp4_quant.cu
void check_quant_shape(int rows, int K);
void quantise(const void* x, int dtype, uint8_t* packed, uint8_t* scales, int rows, int K, cudaStream_t stream);
void quantise_scaled(const void* x, int dtype, float inv_global, uint8_t* packed, uint8_t* scales, int rows, int K,
                     cudaStream_t stream);
void quantise_mx(const void* x, int dtype, uint8_t* packed, uint8_t* scales, int rows, int K, cudaStream_t stream);
void dequantise_mx(const uint8_t* packed, const uint8_t* scales, float* out, int rows, int K, cudaStream_t stream);
void dequantise(const uint8_t* packed, const uint8_t* scales, float* out, int rows, int K, cudaStream_t stream);

// nvfp4_gemm.cu: grouped GEMM for routed-MoE experts. A is a pool of 128-row blocks
// [pool_rows, K/2]; B stacks the experts' weights [experts * n, K/2]; block i of the pool uses
// expert block_expert[i]; only the first *num_blocks blocks are computed (both device arrays are
// read by the kernel, so no host synchronisation is needed between routing and the GEMM).
struct GroupedGemm {
    CUtensorMap A, B, SFA, SFB;
    int pool_rows, n, k, experts, units, tile_n, device, block_rows;
    const int* block_expert;
    const int* num_blocks;
    const int* block_valid;     // real rows per block (device, from the plan kernel); null = every row of C is written
};
void grouped_prepare(GroupedGemm& p, const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                     int pool_rows, int n, int k, int experts, int block_rows, const int* block_expert,
                     const int* num_blocks);
void grouped_launch(const GroupedGemm& p, void* C, int out_bf16, cudaStream_t stream);
// First expert GEMM with the SwiGLU + re-quantise epilogue: B's rows must be interleaved 16 gate / 16 up;
// writes the NVFP4 activation [pool_rows, n/2] instead of C.
// row_dst != null: the second expert GEMM fused with the combine: pool row r goes to row
// (row_dst[r] & 0xFFFFFF) - 1 of slots[row_dst[r] >> 24] (a [slot_rows, n] buffer per rank, peer memory
// included) instead of C; row_dst[r] == 0 is a padding row.
void grouped_launch_fused(const GroupedGemm& p, void* C, int out_bf16, uint8_t* act_packed, uint8_t* act_scales,
                          const float* row_weight, float clamp, const int* row_dst, void* const* slots, int world,
                          int slot_rows, cudaStream_t stream);

// nvfp4_moe.cu: routing metadata, dispatch packing, SwiGLU + re-quantise, top-k reduce.
struct MoeShape {
    int tokens, hidden, intermediate, experts, topk, rank, world;
    float clamp;
};
void moe_route_count(const long long* ids, int routes, int experts, int* counts, cudaStream_t stream);
// block_valid (may be null): [pool_capacity_rows / block_rows], the real rows of every live block.
void moe_plan(int* block_valid, int* counts_matrix, int world, int rank, int experts, int pool_capacity_rows, int block_rows,
              int* send_offset, int* seg_src_offset, int* seg_pool_offset, int* block_expert, int* num_blocks,
              int* totals, int* peer_offset, const long long* ids, int routes, int* cursor, int peer_to_pool,
              cudaStream_t stream);
void moe_clear_live(const int* num_blocks, int block_rows, int pool_rows, int hidden, uint8_t* pool_scales,
                    float* pool_weight, int* pool_dst, cudaStream_t stream);
// Expert parallelism over peer memory (NVLink stores into buffers of the other ranks' processes).
void moe_pack_peer(const uint8_t* xq, const uint8_t* xs, const long long* ids, const float* weights, int tokens,
                   int topk, int hidden, int world, int local_experts, const int* peer_offset, int* cursor,
                   void* const* peer_recv, int recv_capacity, int* error, cudaStream_t stream);
void moe_return_peer(const void* out_pool_bf16, const uint8_t* recv_rows, const int* pool_of_recv, const int* totals,
                     const int* seg_src_offset, int world, int local_experts, int hidden, int recv_capacity,
                     void* const* peer_slots, int slot_capacity, int* error, cudaStream_t stream);
void moe_pack(const uint8_t* xq, const uint8_t* xs, const long long* ids, const float* weights, int tokens, int topk,
              int hidden, int experts, const int* send_offset, int* cursor, uint8_t* send_rows, int* send_pos,
              cudaStream_t stream);
// Single-rank shortcut: rows go straight into the expert-major pool (no send buffer, no unpack);
// route_row[route] is then the pool row, which moe_reduce can read the second GEMM's output by.
void moe_pack_to_pool(const uint8_t* xq, const uint8_t* xs, const long long* ids, const float* weights, int tokens,
                      int topk, int hidden, int experts, const int* seg_pool_offset, int* cursor, uint8_t* pool_packed,
                      uint8_t* pool_scales, float* pool_weight, int* route_row, cudaStream_t stream);
void moe_unpack(const uint8_t* recv_rows, int recv_count_capacity, const int* totals, int world, int local_experts,
                int hidden, const int* seg_src_offset, const int* seg_pool_offset, uint8_t* pool_packed,
                uint8_t* pool_scales, float* pool_weight, int* pool_of_recv, int* pool_dst, cudaStream_t stream);
void moe_swiglu_quant(const void* gate_up_bf16, const float* pool_weight, const int* num_blocks, int block_rows, int pool_rows,
                      int intermediate, float clamp, uint8_t* act_packed, uint8_t* act_scales, cudaStream_t stream);
void moe_return_rows(const void* out_pool_bf16, const int* pool_of_recv, const int* totals, int capacity, int hidden,
                     void* return_rows_bf16, cudaStream_t stream);
// Token quantisation fused with the dispatch: x [tokens, hidden] bf16 -> each route's quantised row delivered
// to its expert, world > 0: into peer_recv[owner] at offsets[expert] + arrival order (bounds-checked against
// recv_capacity); world == 0: into this rank's pool at row offsets[expert] + arrival order (route_row gets it).
void moe_quantise_route(const void* x_bf16, const long long* ids, const float* weights, int tokens, int topk, int hidden,
                        int experts, const int* offsets, int* cursor, void* const* peer_recv, void* const* peer_meta, int world,
                        int local_experts, int recv_capacity, int* error, uint8_t* pool_packed, uint8_t* pool_scales,
                        float* pool_weight, int* route_row, cudaStream_t stream);
void moe_unpack_meta(const uint8_t* side, int recv_count_capacity, const int* totals, int world, int local_experts, int hidden,
                     const int* seg_src_offset, const int* seg_pool_offset, uint8_t* pool_scales, float* pool_weight,
                     int* pool_dst, cudaStream_t stream);
int moe_payload_bytes(int hidden);
// The device's four status words: [0] bits of ptx.cuh's StatusBits, [1] first tag, [2] cycles of the last GEMM.
uint32_t* device_status_word(int device);
// Barrier (ints = 0) or barrier + all-gather of `ints` integers per rank between the GPUs of one node, through
// state blocks (peer_state_bytes each, zeroed) that every rank maps: own = this rank's, peers_device = device
// array of all ranks' blocks in rank order. out [world][ints].
size_t peer_state_bytes(int world, int max_ints);
// ids != null: the payload is the histogram of ids [routes] over `ints` bins, taken inside the kernel.
void peer_exchange(void* own, void* const* peers_device, int world, int rank, const int* payload, int ints, int max_ints,
                   int* out, const long long* ids, int routes, cudaStream_t stream);
// ids (may be null) and experts: routes whose expert id lies outside [0, experts) add nothing, as do negative
// send_pos entries: a dropped route has a defined result on every path.
void moe_reduce(const void* returned_bf16, const int* send_pos, int tokens, int topk, int hidden, void* y_bf16,
                const long long* ids, int experts, cudaStream_t stream);

}  // namespace nvfp4_b200
