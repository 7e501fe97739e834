// C++ boundary of the B200 NVFP4 block-scaled GEMM.
//
// Same names, argument order and ownership rules as the reference's
// include/nvfp4.h:13-25 (struct Nvfp4Params, struct Nvfp4Implementation,
// factory nvfp4_sm100_implementation()), so host code written against that
// header — benchmarks/bindings/nvfp4_bridge.cu:19-21,83-85,115 in the reference
// — compiles against this one unchanged. The implementation behind it is a
// different kernel (gpu_kernels_b200/csrc/nvfp4_gemm.cu).
//
// Data contract (reference include/nvfp4.h:10-12):
//   A [M, K/2], B [N, K/2]  packed E2M1, two values per byte, K contiguous,
//                           even k in the low nibble ("TN": C = A * B^T);
//   SFA, SFB                one UE4M3 byte per 16 K-values, stored in cuBLASLt's
//                           VEC16 layout: 512-byte atoms of 128 rows x 4 blocks,
//                           atoms ordered [row/128][k/64];
//   C [M, N]                row-major FP16, leading dimension N, overwritten.
// Extensions the reference does not have: an FP32 global scale `alpha`
// (C = fp16(alpha * acc), default 1), M that is only a multiple of 128, and a
// status word that reports a wait that gave up instead of hanging.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace gpu_kernels {

// The four tensor maps and the four integers lead the struct exactly as in the
// reference (callers value-initialise it and never read the rest).
struct Nvfp4Params {
    CUtensorMap A, B, SFA, SFB;
    int M, N, K, clusters;          // clusters = persistent scheduling units in the grid
    // ---- extensions (filled by prepare) ----
    float alpha;                    // FP32 global scale applied to the accumulator
    int cta_group;                  // 2: CTA pairs on 256-row tiles; 1: single CTAs on 128-row tiles
    int tile_n;                     // columns of C per tile (256 or 128)
    int group_m;                    // tile rows per rasterisation band
    int device;                     // device the plan was prepared on
    int c_evict_first;              // 1: C is stored with the evict-first L2 policy
    int direct_store;               // 1: epilogue writes C from registers instead of TMA stores
    int k_skew;                     // tile t starts its K walk at step (t * k_skew) % steps and wraps; 0 = off
    int split_k;                    // S > 1: S units per tile, each with 1/S of the K steps (see below)
    void* split_k_workspace;        // flags + FP32 partial tiles, owned by the caller
    int gather_world;               // > 0: C goes to this many full-width buffers instead (see nvfp4_set_gather)
    int gather_col0, gather_ldc;
    const void* gather_maps;
    const void* gather_ptrs;
    int out_bf16;                   // 1: launch() writes bfloat16 instead of FP16 through the same pointer
    int status_slot;                // which of the device's status slots this plan reports to
    // L2-side-aware tile order (see nvfp4_set_l2_side_order); device tables owned by a per-process cache
    const void* route;              // null: arithmetic band order
    const void* sm_side;
    const void* unit_side;
    int side_units[2];              // clusters the census found on either side of the L2
    int pdl;                        // 1: launches carry the programmatic stream-serialisation attribute
    // What the caller promises about the kernel in front of each launch in the stream (which this launch may
    // overlap under pdl): 0 = nothing (default): the launch waits for it before touching memory; 1 = it does not
    // write B or SFB (weights): their first tiles are fetched while it drains; 2 = it writes none of A, B, SFA,
    // SFB: this launch computes while it drains and only holds back its stores of C until it has finished.
    int static_operands;
    // Ragged tiling of a one-tile-row plan (M = 128) whose 256-column tiles would leave SMs without a tile:
    // ragged_units tiles (0 = off), the first ragged_extra of them ragged_base + 1 units of 64 columns wide, the
    // others ragged_base; B64 is B's tensor map with 64-row boxes.
    CUtensorMap B64;
    int ragged_base, ragged_extra, ragged_units;
    int mx;                         // 1: MXFP4 operands (one UE8M0 scale per 32 values), see mxfp4_prepare
};

struct Nvfp4Implementation {
    // Builds descriptors for the given device buffers, which must outlive the
    // plan. May query the device; never call it during stream capture.
    // Throws std::invalid_argument on a shape or pointer it cannot serve: M >= 1, N a multiple of 8 (rows of C start
    // on 16-byte boundaries), K a multiple of 64 (the quantiser's own rule; the reference kernel needs multiples of
    // 256 in all three), pointers 16-byte aligned. SFA and SFB always hold whole 128-row atoms: ceil(rows / 128) *
    // 128 * K / 16 bytes; the bytes of the rows beyond M and N may hold anything.
    void (*prepare)(Nvfp4Params&, const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                    int M, int N, int K, cudaStream_t);
    // One asynchronous kernel launch on `stream`; safe inside stream capture.
    void (*launch)(const Nvfp4Params&, __half* C, cudaStream_t);
    // Synchronises the device and throws std::runtime_error if any launch of any plan since
    // the last call reported a wait that timed out (nvfp4_validate_plan checks one plan only).
    void (*validate)();
};

Nvfp4Implementation nvfp4_sm100_implementation();

// Extension: set the FP32 global scale of a prepared plan (takes effect at the next launch).
void nvfp4_set_alpha(Nvfp4Params&, float alpha);

// Extension: the MXFP4 flavour of the same path (OCP microscaling: E2M1 values, one UE8M0 power-of-two scale per 32
// values along K, stored in cuBLASLt's VEC32 order: the same 512-byte atoms of 128 rows x 4 scales, ordered
// [row/128][k/128]). Same arguments and ownership as Nvfp4Implementation::prepare; K a multiple of 128; launch and
// validate are the implementation's. The reference has no MXFP4 path (its kernel is scale_vec::4X only,
// kernels/gemm/matmul/sm100.cu:341-342).
void mxfp4_prepare(Nvfp4Params&, const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int M, int N,
                   int K, cudaStream_t);

// Extension: synchronises the device and throws if a launch of THIS plan reported an error since the last
// check of this plan; other plans' reports are left alone.
void nvfp4_validate_plan(const Nvfp4Params&);

// Extension: ragged tiling for plans with one tile row (M = 128) whose uniform 256-column tiles number fewer
// than the SMs (off unless asked for). B: the pointer
// the plan was prepared with. tiles = 0 returns to uniform tiles. Returns whether ragged tiles are in use.
bool nvfp4_set_ragged_tiles(Nvfp4Params&, const uint8_t* B, int tiles);

// Extension: L2-side-aware tile order, the counterpart of the reference's prepare_schedule
// (kernels/gemm/matmul/sm100.cu:566-673). B200's L2 has two sides; an SM reaches the far one more slowly.
// on = 1: a census (one short kernel: every SM times a chain of dependent atomics on one line, taking turns
// with a time limit on every wait; nothing spins without a limit) labels each SM near or far, a second
// launch with the GEMM's own geometry records which SMs each cluster of the persistent grid lands on, and
// the tile sequence is dealt so that the clusters of one side work through one contiguous part of the
// band order (their A and B panels stay in that side's L2). The tables are cached per device and shape for
// the life of the process. Returns false (and leaves the arithmetic order) when the census does not split
// the SMs into two groups, when a wait in it ran out, or when the grid is smaller than the GPU. Results never
// depend on it: a cluster that lands elsewhere than assumed only loses the locality, and is counted
// (nvfp4_placement_misses). Not during stream capture.
bool nvfp4_set_l2_side_order(Nvfp4Params&, int on, cudaStream_t stream);
unsigned nvfp4_placement_misses(const Nvfp4Params&);

// Extension: split-K (off unless enabled). For shapes with at most a quarter as many tiles as SMs and a long
// K loop (decode-like: M = 128, a slab of N) the K steps of every tile can be dealt to 4 units; each writes FP32 partial sums to a
// workspace, and once a tile's slices are there every slice adds them up, in slice order, for its share of
// the columns and writes that part of C. nvfp4_split_k_workspace_bytes returns 0 when the shape would not
// gain. The workspace (256-byte aligned device memory) belongs to the caller, must outlive the plan, and
// serves one plan: launches of that plan must not overlap each other. The grid then has one unit per
// (tile, slice) and they wait for each other, so all of them must be resident: launch it on a GPU whose SMs
// are not held by other kernels (a wait that runs out is reported by validate()). Results are reproducible
// but differ in the last bits from the unsplit schedule. After validate() has reported an error, enable it
// again (the flag area is cleared on `stream`).
size_t nvfp4_split_k_workspace_bytes(const Nvfp4Params&);
void nvfp4_enable_split_k(Nvfp4Params&, void* workspace, size_t bytes, cudaStream_t stream);

// Extension: the GEMM fused with the all-gather of C, for N sharded over the GPUs of one NVLink node. This
// rank's [M, N] result is the column slab [col0, col0 + N) of a full [M, n_total] C; with a gather set, the
// epilogue writes the slab straight into the full C of every rank in `buffers` (this rank's own and its
// peers', mapped into this process, e.g. through CUDA IPC), so no collective has to move C afterwards: the
// caller only needs a barrier between the ranks before reading. launch() then writes nothing through its C
// argument (still a valid device pointer of M * N elements, e.g. this rank's buffer). `table` is device memory of nvfp4_gather_table_bytes(world), 128-byte aligned, owned by the
// caller and filled here. world = 0 switches the gather off again.
size_t nvfp4_gather_table_bytes(int world);
void nvfp4_set_gather(Nvfp4Params&, void* const* buffers, int world, int col0, int n_total, void* table,
                      cudaStream_t stream);

}  // namespace gpu_kernels
