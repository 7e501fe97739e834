// Routed-MoE expert path in NVFP4: the small kernels around the two grouped GEMMs.
//
//   route_count   histogram of this rank's routes per global expert
//   plan          (one CTA) from the all-gathered count matrix: where each route goes in the send
//                 buffer, where each (source rank, local expert) segment lands in the expert-major
//                 pool, which expert owns each 128-row pool block
//   pack          token rows (already quantised: packed E2M1 + scale bytes) + route weight ->
//                 send buffer ordered by destination expert
//   unpack        received rows -> pool (packed rows, scale bytes in the 128-row atom layout)
//   swiglu_quant  gate_up (bf16) -> bf16(silu(min(g,c)) * clamp(u,+-c) * w) -> NVFP4 for the second GEMM
//   return_rows   expert outputs back into the order the rows were received in
//   reduce        y[t] = bf16(sum_j fp32(row of route (t,j))), fixed j order
//
// The reference's expert path is BF16 on sm_90a with device-side peer pulls
// (kernels/moe/fused/sm90.cu:32-139 metadata/offsets/reduce kernels, :209-550 the fused kernel;
// activation maths kernels/moe/swiglu.cu:12-26; whole-layer semantics reference/python/moe.py:7-26).
// This file keeps those semantics (rounding points, clamp order, fixed-order top-k sum) and the
// phase structure (metadata / FC1 / FC2 / reduce), with NVFP4 operands and an all-to-all exchange.
#include "nvfp4_internal.h"
#include "ptx.cuh"
#include "quant_device.cuh"

#include <cuda_bf16.h>

#include <algorithm>
#include <cstddef>
#include <cstdlib>
#include <string>

namespace nvfp4_b200 {
namespace {

constexpr int ROUTE_BUFFERS = 4;          // row buffers of quantise_route_kernel
constexpr int PAYLOAD_TAIL = 16;          // route weight (float) + padding, keeps rows 16-byte aligned

__host__ __device__ inline int payload_bytes(int hidden) { return hidden / 2 + hidden / 16 + PAYLOAD_TAIL; }

// Every kernel of this file opens with chain_point(): it lets the kernel behind it in the stream be scheduled
// early and then waits until the kernel in front of it has finished, so under programmatic dependent launch
// the launch latencies of the forward's dozen small kernels overlap instead of adding up. Launched through
// launch_chained() (the attribute that permits the early start); an ordinary launch behaves as before.
__device__ __forceinline__ void chain_point() {
    ptx::grid_launch_dependents();
    ptx::grid_dependency_wait();
}

template <typename... Params, typename... Args>
void launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    static const bool pdl = [] { const char* v = std::getenv("NVFP4_B200_PDL"); return !(v && v[0] == '0'); }();
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = &attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cuda_check(cudaLaunchKernelEx(&cfg, kernel, Params(args)...));
}

__global__ void route_count_kernel(const long long* __restrict__ ids, int routes, int experts, int* __restrict__ counts) {
    chain_point();
    extern __shared__ int local[];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) local[e] = 0;
    __syncthreads();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < routes; i += gridDim.x * blockDim.x) {
        const long long e = ids[i];
        if (e >= 0 && e < experts) atomicAdd(&local[int(e)], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        if (local[e]) atomicAdd(&counts[e], local[e]);
}

// Exclusive prefix sum over n <= 4096 ints held in shared memory, by one CTA of 256 threads: each thread
// scans a contiguous chunk serially, the chunk totals are scanned by one thread (<= 256 values).
__device__ void block_exclusive_scan(int* data, int n, int* chunk_sums) {
    const int per = (n + int(blockDim.x) - 1) / int(blockDim.x);
    const int lo = min(int(threadIdx.x) * per, n), hi = min(lo + per, n);
    int acc = 0;
    for (int i = lo; i < hi; ++i) { const int v = data[i]; data[i] = acc; acc += v; }
    chunk_sums[threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (unsigned i = 0; i < blockDim.x; ++i) { const int v = chunk_sums[i]; chunk_sums[i] = run; run += v; }
        chunk_sums[blockDim.x] = run;
    }
    __syncthreads();
    for (int i = lo; i < hi; ++i) data[i] += chunk_sums[threadIdx.x];
    __syncthreads();
}

// counts[r * experts + ge]: routes rank r sends to global expert ge. One CTA of 256 threads; experts <= 4096.
__global__ void plan_kernel(int* __restrict__ block_valid, int* counts, int world, int rank, int experts, int capacity_rows,
                            int block_rows,
                            int* __restrict__ send_offset, int* __restrict__ seg_src_offset,
                            int* __restrict__ seg_pool_offset, int* __restrict__ block_expert,
                            int* __restrict__ num_blocks, int* __restrict__ totals, int* __restrict__ peer_offset,
                            const long long* __restrict__ ids, int routes, int* __restrict__ cursor, int peer_to_pool) {
    chain_point();
    extern __shared__ int sh[];
    const int local_experts = experts / world;
    const int segments = world * local_experts;          // == experts
    int* scan = sh;                                       // [experts] scratch for the three scans
    int* pool_off = sh + experts;                         // [local_experts] padded start of each expert
    int* chunk = pool_off + local_experts;                // [blockDim.x + 1]
    if (ids) {
        // One rank: nothing to exchange, so the histogram of the routes is taken right here (the counts row is
        // this kernel's own output) instead of by a zeroing memset and a counting kernel before it.
        for (int e = threadIdx.x; e < experts; e += blockDim.x) scan[e] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < routes; i += blockDim.x) {
            const long long e = ids[i];
            if (e >= 0 && e < experts) atomicAdd(&scan[int(e)], 1);
        }
        __syncthreads();
        for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = scan[e];
        __syncthreads();
    }
    if (cursor)
        for (int e = threadIdx.x; e < experts; e += blockDim.x) cursor[e] = 0;    // arrival counters of the dispatch
    // 1. where this rank's routes go in its send buffer (ordered by global expert = by destination rank)
    for (int ge = threadIdx.x; ge < experts; ge += blockDim.x) scan[ge] = counts[rank * experts + ge];
    __syncthreads();
    block_exclusive_scan(scan, experts, chunk);
    for (int ge = threadIdx.x; ge < experts; ge += blockDim.x) send_offset[ge] = scan[ge];
    if (threadIdx.x == 0) send_offset[experts] = chunk[blockDim.x];
    if (peer_offset && !peer_to_pool) {
        // Where this rank's rows for global expert ge start in the RECEIVE buffer of the rank that owns ge
        // (source-major there): rows of lower-ranked sources for that destination, then this rank's rows
        // for the destination's earlier experts. Lets pack write straight into the peer's buffer.
        for (int ge = threadIdx.x; ge < experts; ge += blockDim.x) {
            const int d = ge / local_experts;
            int base = 0;
            for (int r = 0; r < rank; ++r)
                for (int e = 0; e < local_experts; ++e) base += counts[r * experts + d * local_experts + e];
            peer_offset[ge] = base + scan[ge] - scan[d * local_experts];
        }
    }
    __syncthreads();
    // 2. segments (source rank r, local expert e) in the receive buffer: source-major, expert order inside
    //    a source, which is the order pack() wrote them
    for (int i = threadIdx.x; i < segments; i += blockDim.x) {
        const int r = i / local_experts, e = i - r * local_experts;
        scan[i] = counts[r * experts + rank * local_experts + e];
    }
    __syncthreads();
    block_exclusive_scan(scan, segments, chunk);
    for (int i = threadIdx.x; i < segments; i += blockDim.x) seg_src_offset[i] = scan[i];
    if (threadIdx.x == 0) { seg_src_offset[segments] = chunk[blockDim.x]; totals[0] = chunk[blockDim.x]; }
    __syncthreads();
    // 3. expert-major pool, every expert padded to whole blocks of block_rows (128 or 256) rows
    for (int e = threadIdx.x; e < local_experts; e += blockDim.x) {
        int sum = 0;
        for (int r = 0; r < world; ++r) sum += counts[r * experts + rank * local_experts + e];
        scan[e] = (sum + block_rows - 1) / block_rows * block_rows;
    }
    __syncthreads();
    block_exclusive_scan(scan, local_experts, chunk);
    const int pool_rows = chunk[blockDim.x];
    const bool overflow = pool_rows > capacity_rows;
    for (int e = threadIdx.x; e < local_experts; e += blockDim.x) {
        pool_off[e] = scan[e];
        const int end = e + 1 < local_experts ? scan[e + 1] : pool_rows;
        if (!overflow)
            for (int blk = scan[e] / block_rows; blk < end / block_rows; ++blk) block_expert[blk] = e;
        int acc = scan[e];
        for (int r = 0; r < world; ++r) {
            seg_pool_offset[r * local_experts + e] = acc;
            acc += counts[r * experts + rank * local_experts + e];
        }
        if (block_valid && !overflow)                           // acc: one past the expert's last real row
            for (int blk = scan[e] / block_rows; blk < end / block_rows; ++blk)
                block_valid[blk] = min(block_rows, max(0, acc - blk * block_rows));
    }
    if (threadIdx.x == 0) {
        *num_blocks = overflow ? 0 : pool_rows / block_rows;     // an overflowing plan computes nothing; the host reports it
        totals[1] = pool_rows;
        totals[2] = overflow ? 1 : 0;
    }
    if (peer_offset && peer_to_pool) {
        // Where this rank's rows for global expert ge start in the POOL of the rank that owns ge: that rank's
        // padded expert-major layout (the same arithmetic its own plan does in step 3), then the rows of
        // lower-ranked sources for that expert. Lets the dispatch write packed rows straight into the pool.
        __syncthreads();
        for (int ge = threadIdx.x; ge < experts; ge += blockDim.x) {
            int sum = 0;
            for (int r = 0; r < world; ++r) sum += counts[r * experts + ge];
            scan[ge] = (sum + block_rows - 1) / block_rows * block_rows;
        }
        __syncthreads();
        block_exclusive_scan(scan, experts, chunk);
        for (int ge = threadIdx.x; ge < experts; ge += blockDim.x) {
            int before = 0;
            for (int r = 0; r < rank; ++r) before += counts[r * experts + ge];
            peer_offset[ge] = scan[ge] - scan[ge / local_experts * local_experts] + before;
        }
    }
}

// One warp per route: copies the token's quantised row and gathers its scale bytes out of the atom layout.
__global__ void pack_kernel(const uint8_t* __restrict__ xq, const uint8_t* __restrict__ xs,
                            const long long* __restrict__ ids, const float* __restrict__ weights, int routes,
                            int topk, int hidden, int experts, const int* __restrict__ send_offset, int* __restrict__ cursor,
                            uint8_t* __restrict__ send_rows, int* __restrict__ send_pos,
                            const int* __restrict__ seg_pool_offset, uint8_t* __restrict__ pool_packed,
                            uint8_t* __restrict__ pool_scales, float* __restrict__ pool_weight) {
    chain_point();
    const int lane = threadIdx.x & 31;
    const int route = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (route >= routes) return;
    const int token = route / topk;
    const long long id = ids[route];
    if (id < 0 || id >= experts) {
        // an id outside the expert range (a router's "dropped" mark) takes no row anywhere; the reduce skips it
        if (lane == 0) send_pos[route] = -1;
        return;
    }
    const int expert = int(id);
    int dst = 0;
    if (lane == 0) {
        const int slot = atomicAdd(&cursor[expert], 1);
        // one rank: the row goes straight into its expert's group of the pool, no send buffer in between
        dst = (pool_packed ? seg_pool_offset[expert] : send_offset[expert]) + slot;
        send_pos[route] = dst;
    }
    dst = __shfl_sync(0xFFFFFFFFu, dst, 0);
    const uint4* src = reinterpret_cast<const uint4*>(xq + size_t(token) * (hidden / 2));
    if (pool_packed) {
        uint4* row = reinterpret_cast<uint4*>(pool_packed + size_t(dst) * (hidden / 2));
        for (int i = lane; i < hidden / 32; i += 32) row[i] = __ldg(src + i);
        for (int b = lane; b < hidden / 16; b += 32)
            pool_scales[scale_byte_offset(dst, b, hidden)] = xs[scale_byte_offset(token, b, hidden)];
        if (lane == 0) pool_weight[dst] = weights[route];
        return;
    }
    uint8_t* out = send_rows + size_t(dst) * payload_bytes(hidden);
    for (int i = lane; i < hidden / 32; i += 32) reinterpret_cast<uint4*>(out)[i] = __ldg(src + i);
    for (int b = lane; b < hidden / 16; b += 32) out[hidden / 2 + b] = xs[scale_byte_offset(token, b, hidden)];
    if (lane == 0) *reinterpret_cast<float*>(out + hidden / 2 + hidden / 16) = weights[route];
}

__global__ void unpack_kernel(const uint8_t* __restrict__ recv_rows, const int* __restrict__ totals, int segments,
                              int hidden, const int* __restrict__ seg_src_offset, const int* __restrict__ seg_pool_offset,
                              uint8_t* __restrict__ pool_packed, uint8_t* __restrict__ pool_scales,
                              float* __restrict__ pool_weight, int* __restrict__ pool_of_recv, int local_experts,
                              int* __restrict__ pool_dst) {
    chain_point();
    const int lane = threadIdx.x & 31;
    const int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (p >= totals[0] || totals[2]) return;
    // last segment whose start is <= p (segments may be empty, so starts repeat): the starts are
    // non-decreasing, so it is the number of starts <= p, minus one. The lanes count 32 starts at a
    // time with independent, coalesced loads (a binary search would be eight dependent loads per row).
    int below = 0;
    for (int base = 0; base < segments; base += 32) {
        const int i = base + lane;
        below += __popc(__ballot_sync(0xFFFFFFFFu, i < segments && __ldg(seg_src_offset + i) <= p));
    }
    const int lo = below - 1;
    const int row = seg_pool_offset[lo] + (p - seg_src_offset[lo]);
    const uint8_t* in = recv_rows + size_t(p) * payload_bytes(hidden);
    uint4* dst = reinterpret_cast<uint4*>(pool_packed + size_t(row) * (hidden / 2));
    for (int i = lane; i < hidden / 32; i += 32) dst[i] = reinterpret_cast<const uint4*>(in)[i];
    // four scale bytes (64 K-values) are contiguous in the atom layout, and 4-byte aligned in the dispatch row
    for (int q = lane; q < hidden / 64; q += 32)
        *reinterpret_cast<uint32_t*>(pool_scales + scale_byte_offset(row, 4 * q, hidden)) =
            *reinterpret_cast<const uint32_t*>(in + hidden / 2 + 4 * q);
    if (lane == 0) {
        pool_weight[row] = *reinterpret_cast<const float*>(in + hidden / 2 + hidden / 16);
        pool_of_recv[p] = row;
        // where the result of this row goes: (source rank << 24) | (route index + 1); 0 stays "padding"
        if (pool_dst)
            pool_dst[row] = ((lo / local_experts) << 24) | (*reinterpret_cast<const int*>(in + hidden / 2 + hidden / 16 + 4) + 1);
    }
}

// After a dispatch that wrote the packed rows straight into this rank's pool: one warp per received row lays
// the row's scale bytes (row-major in the side buffer) into the pool's scale atoms and records its route
// weight and where its result goes. p counts received rows source-major, as the plan's segment tables do.
__global__ void unpack_meta_kernel(const uint8_t* __restrict__ side, const int* __restrict__ totals, int segments, int hidden,
                                   const int* __restrict__ seg_src_offset, const int* __restrict__ seg_pool_offset,
                                   uint8_t* __restrict__ pool_scales, float* __restrict__ pool_weight,
                                   int* __restrict__ pool_dst, int local_experts) {
    chain_point();
    const int lane = threadIdx.x & 31;
    const int p = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (p >= totals[0] || totals[2]) return;
    int below = 0;
    for (int base = 0; base < segments; base += 32) {
        const int i = base + lane;
        below += __popc(__ballot_sync(0xFFFFFFFFu, i < segments && __ldg(seg_src_offset + i) <= p));
    }
    const int lo = below - 1;
    const int row = seg_pool_offset[lo] + (p - seg_src_offset[lo]);
    const uint8_t* in = side + size_t(row) * (hidden / 16 + PAYLOAD_TAIL);
    for (int q = lane; q < hidden / 64; q += 32)
        *reinterpret_cast<uint32_t*>(pool_scales + scale_byte_offset(row, 4 * q, hidden)) =
            *reinterpret_cast<const uint32_t*>(in + 4 * q);
    if (lane == 0) {
        pool_weight[row] = *reinterpret_cast<const float*>(in + hidden / 16);
        pool_dst[row] = ((lo / local_experts) << 24) | (*reinterpret_cast<const int*>(in + hidden / 16 + 4) + 1);
    }
}

// gate_up [rows, 2I] bf16 (gate columns first) -> act = bf16(silu(min(g,c)) * clamp(u,-c,c) * w_row)
// -> NVFP4 along I. Same tiling as the stand-alone quantiser: a CTA owns 128 rows x 256 columns of
// the activation so that every scale atom and packed row segment leaves in full lines.
__global__ void __launch_bounds__(256)
swiglu_quant_kernel(const __nv_bfloat16* __restrict__ gate_up, const float* __restrict__ pool_weight,
                    const int* __restrict__ num_blocks, int block_rows, int inter, float clamp,
                    uint8_t* __restrict__ act_packed, uint8_t* __restrict__ act_scales) {
    chain_point();
    __shared__ __align__(16) uint8_t sf_tile[4 * 512];
    if (int(blockIdx.y) * 128 >= *num_blocks * block_rows) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kb = lane & 15;
    const int col0 = blockIdx.x * 256;
    const int row_base = blockIdx.y * 128;
    const int k = col0 + kb * 16;
    #pragma unroll 1
    for (int pass = 0; pass < 8; ++pass) {
        const int r = pass * 16 + warp * 2 + (lane >> 4);
        const size_t row = size_t(row_base + r);
        const uint4* gp = reinterpret_cast<const uint4*>(gate_up + row * (2 * inter) + k);
        const uint4* up = reinterpret_cast<const uint4*>(gate_up + row * (2 * inter) + inter + k);
        const float w = pool_weight[row];
        if (w == 0.0f) {
            // Padding row of the pool (or a route that contributes nothing): act is all zeros, whose NVFP4
            // encoding is the smallest scale and zero codes. No reason to read gate_up or evaluate anything.
            *reinterpret_cast<uint2*>(act_packed + row * (inter / 2) + k / 2) = make_uint2(0u, 0u);
            sf_tile[(kb >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = 0x01;
            continue;
        }
        const uint4 g4[2] = {__ldg(gp), __ldg(gp + 1)}, u4[2] = {__ldg(up), __ldg(up + 1)};
        const uint32_t* gw = reinterpret_cast<const uint32_t*>(g4);
        const uint32_t* uw = reinterpret_cast<const uint32_t*>(u4);
        uint32_t act[8];                                       // bf16 pairs of the rounded activation
        #pragma unroll
        for (int i = 0; i < 8; ++i) {
            float a2[2];
            #pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t gbits = h ? (gw[i] & 0xFFFF0000u) : (gw[i] << 16);
                const uint32_t ubits = h ? (uw[i] & 0xFFFF0000u) : (uw[i] << 16);
                const float gate = fminf(__uint_as_float(gbits), clamp);
                const float upv = fminf(fmaxf(__uint_as_float(ubits), -clamp), clamp);
                a2[h] = silu_fast(gate) * upv * w;
            }
            const __nv_bfloat162 p = __floats2bfloat162_rn(a2[0], a2[1]);
            act[i] = *reinterpret_cast<const uint32_t*>(&p);
        }
        uint2 out;
        const uint32_t sbyte = quantise_block_pairs<Bf16Pairs>(act, out);
        *reinterpret_cast<uint2*>(act_packed + row * (inter / 2) + k / 2) = out;
        sf_tile[(kb >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = static_cast<uint8_t>(sbyte);
    }
    __syncthreads();
    if (threadIdx.x < 128) {
        const size_t first_atom = size_t(blockIdx.y) * (inter / 64) + size_t(blockIdx.x) * 4;
        reinterpret_cast<uint4*>(act_scales + first_atom * 512)[threadIdx.x] =
            reinterpret_cast<const uint4*>(sf_tile)[threadIdx.x];
    }
}

__global__ void return_rows_kernel(const uint4* __restrict__ out_pool, const int* __restrict__ pool_of_recv,
                                   const int* __restrict__ totals, int row_vec, uint4* __restrict__ ret) {
    chain_point();
    const int p = blockIdx.x;
    if (p >= totals[0] || totals[2]) return;
    const uint4* src = out_pool + size_t(pool_of_recv[p]) * row_vec;
    uint4* dst = ret + size_t(p) * row_vec;
    for (int i = threadIdx.x; i < row_vec; i += blockDim.x) dst[i] = __ldg(src + i);
}

// y[t] = bf16(sum over j of fp32(row of route (t, j))), j ascending: the order of the reference's
// reduce kernel (kernels/moe/fused/sm90.cu:125-133). A dropped route (expert id outside [0, experts), or a
// negative row index) adds nothing. TOPK > 0: the route count as a compile-time constant, so that a thread has
// all of a column's loads in flight before it adds them up (the kernel only moves bytes: 16 bytes x TOPK in
// flight per thread is what brings it near the memory's speed); TOPK = 0: any count, one load at a time.
template <int TOPK>
__global__ void __launch_bounds__(256)
reduce_kernel(const uint4* __restrict__ returned, const int* __restrict__ send_pos, int topk,
              int row_vec, uint4* __restrict__ y, const long long* __restrict__ ids, int experts) {
    chain_point();
    const int t = blockIdx.x;
    constexpr int SLOTS = TOPK > 0 ? TOPK : 1;
    const int count = TOPK > 0 ? TOPK : topk;
    __shared__ int rows[64];                                     // row of every route of this token, -1 = skip
    for (int j = threadIdx.x; j < count && j < 64; j += blockDim.x) {
        int pos = send_pos[t * count + j];
        if (ids) {
            const long long id = ids[t * count + j];
            if (id < 0 || id >= experts) pos = -1;
        }
        rows[j] = pos;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < row_vec; i += blockDim.x) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        auto add = [&](const uint4& v) {
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            #pragma unroll
            for (int q = 0; q < 4; ++q) {
                acc[2 * q] += __uint_as_float(w[q] << 16);
                acc[2 * q + 1] += __uint_as_float(w[q] & 0xFFFF0000u);
            }
        };
        if constexpr (TOPK > 0) {
            uint4 v[SLOTS];
            #pragma unroll
            for (int j = 0; j < SLOTS; ++j)
                v[j] = rows[j] >= 0 ? __ldg(returned + size_t(rows[j]) * row_vec + i) : make_uint4(0u, 0u, 0u, 0u);
            #pragma unroll
            for (int j = 0; j < SLOTS; ++j)
                if (rows[j] >= 0) add(v[j]);                     // a skipped route adds nothing, not even +0
        } else {
            for (int j = 0; j < count; ++j) {
                const int pos = j < 64 ? rows[j] : -1;
                if (pos >= 0) add(__ldg(returned + size_t(pos) * row_vec + i));
            }
        }
        uint32_t o[4];
        #pragma unroll
        for (int q = 0; q < 4; ++q) {
            const __nv_bfloat162 p = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
            o[q] = *reinterpret_cast<const uint32_t*>(&p);
        }
        y[size_t(t) * row_vec + i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---- expert parallelism over peer memory ----------------------------------------------------
// Instead of packing into a send buffer and letting a library all-to-all move it, each route's row
// is stored directly into the receive buffer of the rank that owns its expert (NVLink peer store),
// and each expert output row directly into the [T, topk, H] slot buffer of the rank the token came
// from. Every peer write is bounds-checked against the capacity the peers agreed on; a violation is
// recorded in `error` and the write is skipped. The caller separates the phases with a collective
// (a stream-ordered barrier): nothing here waits on another GPU.
struct PeerBuffers {
    void* ptr[8];
};

__global__ void pack_peer_kernel(const uint8_t* __restrict__ xq, const uint8_t* __restrict__ xs,
                                 const long long* __restrict__ ids, const float* __restrict__ weights, int routes,
                                 int topk, int hidden, int local_experts, int experts, const int* __restrict__ peer_offset,
                                 int* __restrict__ cursor, PeerBuffers recv, int recv_capacity, int* __restrict__ error) {
    chain_point();
    const int lane = threadIdx.x & 31;
    const int route = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (route >= routes) return;
    const int token = route / topk;
    const long long id = ids[route];
    if (id < 0 || id >= experts) return;                        // dropped route: no row is sent (see reduce_kernel)
    const int expert = int(id);
    int dst = 0;
    if (lane == 0) dst = peer_offset[expert] + atomicAdd(&cursor[expert], 1);
    dst = __shfl_sync(0xFFFFFFFFu, dst, 0);
    if (dst < 0 || dst >= recv_capacity) {
        if (lane == 0) atomicOr(error, 1);
        return;
    }
    uint8_t* out = static_cast<uint8_t*>(recv.ptr[expert / local_experts]) + size_t(dst) * payload_bytes(hidden);
    const uint4* src = reinterpret_cast<const uint4*>(xq + size_t(token) * (hidden / 2));
    for (int i = lane; i < hidden / 32; i += 32) reinterpret_cast<uint4*>(out)[i] = __ldg(src + i);
    for (int b = lane; b < hidden / 16; b += 32) out[hidden / 2 + b] = xs[scale_byte_offset(token, b, hidden)];
    if (lane == 0) {
        *reinterpret_cast<float*>(out + hidden / 2 + hidden / 16) = weights[route];
        *reinterpret_cast<int*>(out + hidden / 2 + hidden / 16 + 4) = route;       // where the result goes back to
    }
}

// Quantise each token's row once (bf16 -> E2M1 codes + UE4M3 scale bytes, bit for bit what quantise_kernel
// writes), keep it in shared memory as one dispatch row, and deliver it to the token's topk experts: into the
// receive buffers of the ranks that own them (world > 0: peer stores over NVLink, each bounds-checked), or
// straight into this rank's expert-major pool (world == 0). Replaces the stand-alone quantiser, its padded input
// copy and the pack kernel: the quantised tokens never go through global memory.
// A CTA walks tokens blockIdx.x, blockIdx.x + gridDim.x, ... with two row buffers: while token t is quantised
// and sent, the 32 bytes each thread needs of token t + gridDim.x are already in flight, and so is that token's
// chain of dependent accesses (expert id -> pool offset -> arrival counter) that yields its destination rows.
// The bulk copies that carry a row out are only waited for when their buffer (one of four) comes round again. (One token per
// CTA without the prefetch: 39 us for 4096 tokens of 4096 values, top-6; ncu: DRAM 21 % busy, issue slots 39 %,
// warps waiting on the loads and on the barrier behind them in equal parts.)
__global__ void __launch_bounds__(256, 4)
quantise_route_kernel(const __nv_bfloat16* __restrict__ x, const long long* __restrict__ ids,
                      const float* __restrict__ weights, int tokens, int topk, int hidden, int experts,
                      const int* __restrict__ offsets, int* __restrict__ cursor,
                      PeerBuffers recv, PeerBuffers meta, int to_pool, int world, int local_experts, int recv_capacity,
                      int* __restrict__ error,
                      uint8_t* __restrict__ pool_packed, uint8_t* __restrict__ pool_scales,
                      float* __restrict__ pool_weight, int* __restrict__ route_row) {
    chain_point();
    extern __shared__ __align__(16) uint8_t smem_rows[];        // ROUTE_BUFFERS x (codes [hidden/2] | scale bytes [hidden/16] | int dst[topk])
    const int row_bytes = hidden / 2 + hidden / 16;
    const int dst_off = (row_bytes + 15) & ~15;
    const int buf_bytes = (dst_off + topk * int(sizeof(int)) + 15) & ~15;
    const int tid = threadIdx.x, blocks = hidden / 16;
    const bool chooser = tid < topk;                            // thread j owns route j of the token
    auto fetch = [&](int token, uint4& lo, uint4& hi) {
        const uint4* src = reinterpret_cast<const uint4*>(x + size_t(token) * hidden);
        lo = __ldg(src + 2 * tid);
        hi = __ldg(src + 2 * tid + 1);
    };
    // The chain id -> (offset, counter) is split over two iterations, so that no warp waits for the id inside one:
    // the id and weight of the token after next are loaded while the next token's row is claimed with the id
    // that was loaded an iteration ago.
    long long id2 = -1;                                         // expert id of the token after next
    float weight2 = 0.0f;
    int ndst = -1, nexpert = 0;
    float nweight = 0.0f;
    auto look = [&](int token) {
        id2 = ids[size_t(token) * topk + tid];
        weight2 = weights[size_t(token) * topk + tid];
    };
    auto claim = [&]() {                                        // route tid of the token whose id is in id2
        nweight = weight2;
        nexpert = int(id2);
        ndst = (id2 >= 0 && id2 < experts) ? offsets[id2] + atomicAdd(&cursor[id2], 1) : -1;
    };
    int token = blockIdx.x;
    uint4 nlo = make_uint4(0u, 0u, 0u, 0u), nhi = nlo;
    if (token < tokens) {
        if (tid < blocks) fetch(token, nlo, nhi);
        if (chooser) {
            look(token);
            claim();
            if (token + int(gridDim.x) < tokens) look(token + gridDim.x);
        }
    }
    for (int it = 0; token < tokens; token += gridDim.x, ++it) {
        uint8_t* row = smem_rows + (it % ROUTE_BUFFERS) * buf_bytes;
        int* dst = reinterpret_cast<int*>(row + dst_off);
        const uint4 lo = nlo, hi = nhi;
        const int my_dst = ndst, my_expert = nexpert;
        const float my_weight = nweight;
        const int next = token + gridDim.x;
        if (next < tokens) {
            if (tid < blocks) fetch(next, nlo, nhi);
            if (chooser) {
                claim();
                if (next + int(gridDim.x) < tokens) look(next + gridDim.x);
            }
        }
        if (tid < blocks) {
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            uint2 codes;
            const uint32_t sbyte = quantise_block_pairs<Bf16Pairs>(w, codes);
            *reinterpret_cast<uint2*>(row + tid * 8) = codes;
            row[hidden / 2 + tid] = static_cast<uint8_t>(sbyte);
        }
        const uint4* src = reinterpret_cast<const uint4*>(x + size_t(token) * hidden);
        for (int b = tid + blockDim.x; b < blocks; b += blockDim.x) {     // rows wider than 4096 values
            const uint4 l2 = __ldg(src + 2 * b), h2 = __ldg(src + 2 * b + 1);
            const uint32_t w[8] = {l2.x, l2.y, l2.z, l2.w, h2.x, h2.y, h2.z, h2.w};
            uint2 codes;
            const uint32_t sbyte = quantise_block_pairs<Bf16Pairs>(w, codes);
            *reinterpret_cast<uint2*>(row + b * 8) = codes;
            row[hidden / 2 + b] = static_cast<uint8_t>(sbyte);
        }
        if (chooser) {
            // where the row's scale words go in the pool's atoms: word q of row d sits at base(d) + 512 q
            dst[tid] = my_dst < 0 ? -1 : (my_dst / 128) * (hidden / 64) * 512 + (my_dst % 32) * 16 + ((my_dst % 128) / 32) * 4;
            // one group per token and chooser thread (empty for a dropped route): all but the last
            // ROUTE_BUFFERS - 2 have read their rows, so the buffer the next token takes is free
            ptx::tma_store_wait_read<ROUTE_BUFFERS - 2>();
        }
        ptx::fence_async_smem();                                // the row, written above, is read by bulk copies below
        __syncthreads();
        const uint32_t row_smem = ptx::smem_u32(row);
        if (world > 0) {
            // thread j sends route j: one bulk copy of the whole row (codes + scale bytes), then the 8-byte tail
            if (chooser) {
                const int route = token * topk + tid, d = my_dst;
                if (d < 0) {
                    // an expert id outside the range: a dropped route, nothing is sent and the reduce skips it
                } else if (d >= recv_capacity) {
                    atomicOr(error, 1);
                } else {
                    const int owner = my_expert / local_experts;
                    if (to_pool) {
                        // d is a row of the owner's pool: the codes land where FC1 reads them; scale bytes, weight
                        // and route index go to the owner's side buffer (its scale atoms are laid out there)
                        uint8_t* side = static_cast<uint8_t*>(meta.ptr[owner]) + size_t(d) * (hidden / 16 + PAYLOAD_TAIL);
                        ptx::bulk_store(static_cast<uint8_t*>(recv.ptr[owner]) + size_t(d) * (hidden / 2), row_smem, uint32_t(hidden / 2));
                        ptx::bulk_store(side, row_smem + uint32_t(hidden / 2), uint32_t(hidden / 16));
                        *reinterpret_cast<float*>(side + hidden / 16) = my_weight;
                        *reinterpret_cast<int*>(side + hidden / 16 + 4) = route;
                    } else {
                        uint8_t* out = static_cast<uint8_t*>(recv.ptr[owner]) + size_t(d) * payload_bytes(hidden);
                        ptx::bulk_store(out, row_smem, uint32_t(row_bytes));
                        *reinterpret_cast<float*>(out + row_bytes) = my_weight;
                        *reinterpret_cast<int*>(out + row_bytes + 4) = route;       // where the result goes back to
                    }
                }
                ptx::tma_store_commit();
            }
            continue;
        }
        if (chooser) {
            const int route = token * topk + tid, d = my_dst;
            if (d >= 0) {
                ptx::bulk_store(pool_packed + size_t(d) * (hidden / 2), row_smem, uint32_t(hidden / 2));
                pool_weight[d] = my_weight;
            }
            ptx::tma_store_commit();
            route_row[route] = d;                               // -1: an id outside the expert range, dropped (the reduce skips it)
        }
        // four scale bytes (64 K-values) are contiguous in the atom layout
        for (int q = tid; q < hidden / 64; q += blockDim.x) {
            const uint32_t word = *reinterpret_cast<const uint32_t*>(row + hidden / 2 + 4 * q);
            for (int j = 0; j < topk; ++j) {
                const int base = dst[j];
                if (base >= 0) *reinterpret_cast<uint32_t*>(pool_scales + size_t(base) + size_t(q) * 512) = word;
            }
        }
    }
    if (chooser) ptx::tma_store_wait_read<0>();                 // shared memory stays until the last copies have read it
}

// One CTA per received row: expert output -> slot `route` of the source rank's [T*topk, H] buffer.
__global__ void return_peer_kernel(const uint4* __restrict__ out_pool, const uint8_t* __restrict__ recv_rows,
                                   const int* __restrict__ pool_of_recv, const int* __restrict__ totals,
                                   const int* __restrict__ seg_src_offset, int segments, int local_experts, int hidden,
                                   PeerBuffers slots, int slot_capacity, int* __restrict__ error) {
    chain_point();
    const int p = blockIdx.x;
    if (p >= totals[0] || totals[2]) return;
    int lo = 0, hi = segments;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg_src_offset[mid] <= p) lo = mid; else hi = mid;
    }
    const int src_rank = lo / local_experts;
    const int route = *reinterpret_cast<const int*>(recv_rows + size_t(p) * payload_bytes(hidden) + hidden / 2 + hidden / 16 + 4);
    if (route < 0 || route >= slot_capacity) {
        if (threadIdx.x == 0) atomicOr(error, 2);
        return;
    }
    const int row_vec = hidden / 8;
    const uint4* src = out_pool + size_t(pool_of_recv[p]) * row_vec;
    uint4* dst = static_cast<uint4*>(slots.ptr[src_rank]) + size_t(route) * row_vec;
    for (int i = threadIdx.x; i < row_vec; i += blockDim.x) dst[i] = __ldg(src + i);
}

void check_hidden(int hidden, const char* what) {
    if (hidden <= 0 || hidden % 256) throw std::invalid_argument(std::string(what) + ": width must be a positive multiple of 256");
}

}  // namespace

void moe_route_count(const long long* ids, int routes, int experts, int* counts, cudaStream_t stream) {
    if (!ids || !counts || routes < 0 || experts <= 0 || experts > 4096) throw std::invalid_argument("moe route_count: bad argument");
    if (routes == 0) return;
    const int blocks = std::min(64, (routes + 255) / 256);
    launch_chained(route_count_kernel, dim3(blocks), dim3(256), size_t(experts * sizeof(int)), stream, ids, routes, experts, counts);
}

void moe_plan(int* block_valid, int* counts_matrix, int world, int rank, int experts, int pool_capacity_rows, int block_rows,
              int* send_offset, int* seg_src_offset, int* seg_pool_offset, int* block_expert, int* num_blocks,
              int* totals, int* peer_offset, const long long* ids, int routes, int* cursor, int peer_to_pool,
              cudaStream_t stream) {
    if (ids && (world != 1 || routes < 0)) throw std::invalid_argument("moe plan: counting the routes in the plan kernel is for one rank");
    if (world <= 0 || rank < 0 || rank >= world || experts <= 0 || experts % world || experts > 4096)
        throw std::invalid_argument("moe plan: experts must divide over the ranks (and be <= 4096)");
    if (block_rows != 128 && block_rows != 256) throw std::invalid_argument("moe plan: block rows must be 128 or 256");
    if (pool_capacity_rows <= 0 || pool_capacity_rows % block_rows) throw std::invalid_argument("moe plan: pool capacity must be a multiple of the block rows");
    const int local = experts / world;
    launch_chained(plan_kernel, dim3(1), dim3(256), size_t((experts + local + 257) * sizeof(int)), stream, block_valid, counts_matrix, world, rank, experts, pool_capacity_rows, block_rows,
                                                                   send_offset, seg_src_offset, seg_pool_offset,
                                                                   block_expert, num_blocks, totals, peer_offset, ids, routes, cursor, peer_to_pool);
}

void moe_pack(const uint8_t* xq, const uint8_t* xs, const long long* ids, const float* weights, int tokens, int topk,
              int hidden, int experts, const int* send_offset, int* cursor, uint8_t* send_rows, int* send_pos,
              cudaStream_t stream) {
    check_hidden(hidden, "moe pack");
    const int routes = tokens * topk;
    if (routes == 0) return;
    launch_chained(pack_kernel, dim3((routes * 32 + 255) / 256), dim3(256), size_t(0), stream, xq, xs, ids, weights, routes, topk, hidden, experts, send_offset,
                                                               cursor, send_rows, send_pos, nullptr, nullptr, nullptr, nullptr);
}

void moe_pack_to_pool(const uint8_t* xq, const uint8_t* xs, const long long* ids, const float* weights, int tokens,
                      int topk, int hidden, int experts, const int* seg_pool_offset, int* cursor, uint8_t* pool_packed,
                      uint8_t* pool_scales, float* pool_weight, int* route_row, cudaStream_t stream) {
    check_hidden(hidden, "moe pack_to_pool");
    const int routes = tokens * topk;
    if (routes == 0) return;
    if (!pool_packed || !pool_scales || !pool_weight) throw std::invalid_argument("moe pack_to_pool: null pool");
    launch_chained(pack_kernel, dim3((routes * 32 + 255) / 256), dim3(256), size_t(0), stream, xq, xs, ids, weights, routes, topk, hidden, experts, nullptr, cursor,
                                                               nullptr, route_row, seg_pool_offset, pool_packed,
                                                               pool_scales, pool_weight);
}

void moe_unpack(const uint8_t* recv_rows, int recv_count_capacity, const int* totals, int world, int local_experts,
                int hidden, const int* seg_src_offset, const int* seg_pool_offset, uint8_t* pool_packed,
                uint8_t* pool_scales, float* pool_weight, int* pool_of_recv, int* pool_dst, cudaStream_t stream) {
    check_hidden(hidden, "moe unpack");
    if (recv_count_capacity <= 0) return;
    launch_chained(unpack_kernel, dim3((recv_count_capacity * 32 + 255) / 256), dim3(256), size_t(0), stream, 
        recv_rows, totals, world * local_experts, hidden, seg_src_offset, seg_pool_offset, pool_packed, pool_scales,
        pool_weight, pool_of_recv, local_experts, pool_dst);
}

void moe_swiglu_quant(const void* gate_up_bf16, const float* pool_weight, const int* num_blocks, int block_rows, int pool_rows,
                      int intermediate, float clamp, uint8_t* act_packed, uint8_t* act_scales, cudaStream_t stream) {
    check_hidden(intermediate, "moe swiglu_quant");
    if (pool_rows <= 0 || pool_rows % 128) throw std::invalid_argument("moe swiglu_quant: pool rows must be a multiple of 128");
    const dim3 grid(intermediate / 256, pool_rows / 128);
    launch_chained(swiglu_quant_kernel, dim3(grid), dim3(256), size_t(0), stream, static_cast<const __nv_bfloat16*>(gate_up_bf16), pool_weight, num_blocks, block_rows,
                                                  intermediate, clamp, act_packed, act_scales);
}

void moe_return_rows(const void* out_pool_bf16, const int* pool_of_recv, const int* totals, int capacity, int hidden,
                     void* return_rows_bf16, cudaStream_t stream) {
    check_hidden(hidden, "moe return_rows");
    if (capacity <= 0) return;
    launch_chained(return_rows_kernel, dim3(capacity), dim3(128), size_t(0), stream, static_cast<const uint4*>(out_pool_bf16), pool_of_recv, totals,
                                                     hidden / 8, static_cast<uint4*>(return_rows_bf16));
}

void moe_reduce(const void* returned_bf16, const int* send_pos, int tokens, int topk, int hidden, void* y_bf16,
                const long long* ids, int experts, cudaStream_t stream) {
    check_hidden(hidden, "moe reduce");
    if (tokens <= 0) return;
    if (topk < 1 || topk > 64) throw std::invalid_argument("moe reduce: 1..64 routes per token");
    auto go = [&](auto kernel) {
        launch_chained(kernel, dim3(tokens), dim3(256), size_t(0), stream, static_cast<const uint4*>(returned_bf16), send_pos, topk,
                       hidden / 8, static_cast<uint4*>(y_bf16), ids, experts);
    };
    switch (topk) {
        case 1: go(reduce_kernel<1>); break;
        case 2: go(reduce_kernel<2>); break;
        case 4: go(reduce_kernel<4>); break;
        case 6: go(reduce_kernel<6>); break;
        case 8: go(reduce_kernel<8>); break;
        default: go(reduce_kernel<0>); break;
    }
}

void moe_pack_peer(const uint8_t* xq, const uint8_t* xs, const long long* ids, const float* weights, int tokens,
                   int topk, int hidden, int world, int local_experts, const int* peer_offset, int* cursor,
                   void* const* peer_recv, int recv_capacity, int* error, cudaStream_t stream) {
    check_hidden(hidden, "moe pack_peer");
    if (world < 1 || world > 8 || !peer_recv) throw std::invalid_argument("moe pack_peer: 1..8 ranks");
    const int routes = tokens * topk;
    if (routes == 0) return;
    PeerBuffers recv{};
    for (int r = 0; r < world; ++r) {
        if (!peer_recv[r]) throw std::invalid_argument("moe pack_peer: null peer buffer");
        recv.ptr[r] = peer_recv[r];
    }
    launch_chained(pack_peer_kernel, dim3((routes * 32 + 255) / 256), dim3(256), size_t(0), stream, xq, xs, ids, weights, routes, topk, hidden,
                                                                    local_experts, world * local_experts, peer_offset,
                                                                    cursor, recv, recv_capacity, error);
}

void moe_return_peer(const void* out_pool_bf16, const uint8_t* recv_rows, const int* pool_of_recv, const int* totals,
                     const int* seg_src_offset, int world, int local_experts, int hidden, int recv_capacity,
                     void* const* peer_slots, int slot_capacity, int* error, cudaStream_t stream) {
    check_hidden(hidden, "moe return_peer");
    if (world < 1 || world > 8 || !peer_slots) throw std::invalid_argument("moe return_peer: 1..8 ranks");
    if (recv_capacity <= 0) return;
    PeerBuffers slots{};
    for (int r = 0; r < world; ++r) {
        if (!peer_slots[r]) throw std::invalid_argument("moe return_peer: null peer buffer");
        slots.ptr[r] = peer_slots[r];
    }
    launch_chained(return_peer_kernel, dim3(recv_capacity), dim3(128), size_t(0), stream, static_cast<const uint4*>(out_pool_bf16), recv_rows, pool_of_recv,
                                                          totals, seg_src_offset, world * local_experts, local_experts,
                                                          hidden, slots, slot_capacity, error);
}

void moe_quantise_route(const void* x_bf16, const long long* ids, const float* weights, int tokens, int topk, int hidden,
                        int experts, const int* offsets, int* cursor, void* const* peer_recv, void* const* peer_meta, int world,
                        int local_experts, int recv_capacity, int* error, uint8_t* pool_packed, uint8_t* pool_scales,
                        float* pool_weight, int* route_row, cudaStream_t stream) {
    check_hidden(hidden, "moe quantise_route");
    if (tokens <= 0) return;
    if (topk < 1 || topk > 256 || experts < 1 || !x_bf16 || !ids || !weights || !offsets || !cursor)
        throw std::invalid_argument("moe quantise_route: bad argument");
    PeerBuffers recv{}, meta{};
    if (world > 0) {
        if (world > 8 || !peer_recv || !error || local_experts < 1) throw std::invalid_argument("moe quantise_route: 1..8 ranks");
        for (int r = 0; r < world; ++r) {
            if (!peer_recv[r] || (peer_meta && !peer_meta[r])) throw std::invalid_argument("moe quantise_route: null peer buffer");
            recv.ptr[r] = peer_recv[r];
            if (peer_meta) meta.ptr[r] = peer_meta[r];
        }
    } else if (!pool_packed || !pool_scales || !pool_weight || !route_row) {
        throw std::invalid_argument("moe quantise_route: null pool");
    }
    const size_t row = (size_t(hidden) / 2 + hidden / 16 + 15) & ~size_t(15);
    const size_t smem = ROUTE_BUFFERS * ((row + size_t(topk) * sizeof(int) + 15) & ~size_t(15));
    // four resident CTAs per SM walk the tokens
    static int sms = 0;
    if (!sms) {
        int device = 0;
        cuda_check(cudaGetDevice(&device));
        cuda_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    }
    const int grid = std::min(tokens, 4 * sms);
    if (smem > 48 * 1024) throw std::invalid_argument("moe quantise_route: hidden too wide for the row buffers");
    launch_chained(quantise_route_kernel, dim3(grid), dim3(256), size_t(smem), stream, static_cast<const __nv_bfloat16*>(x_bf16), ids, weights, tokens, topk, hidden,
                                                        experts, offsets, cursor, recv, meta, peer_meta ? 1 : 0, world,
                                                        local_experts, recv_capacity, error, pool_packed, pool_scales,
                                                        pool_weight, route_row);
}

// One CTA per 128 pool rows: if the rows belong to a live block, clear their scale bytes (whole atoms, one
// contiguous run), route weights and destination codes, so that the padding rows of every expert's last block
// contribute nothing. Only the blocks of this forward are touched: the pool is sized for the worst case and
// clearing all of it every call costs more than the small-batch kernels themselves.
__global__ void __launch_bounds__(256)
clear_live_kernel(const int* __restrict__ num_blocks, int block_rows, int hidden, uint8_t* __restrict__ pool_scales,
                  float* __restrict__ pool_weight, int* __restrict__ pool_dst) {
    chain_point();
    const int row0 = blockIdx.x * 128;
    if (row0 >= *num_blocks * block_rows) return;
    const size_t bytes = size_t(hidden / 64) * 512;            // the scale atoms of 128 rows
    uint4* scales = reinterpret_cast<uint4*>(pool_scales + size_t(blockIdx.x) * bytes);
    for (size_t i = threadIdx.x; i < bytes / 16; i += blockDim.x) scales[i] = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x < 128) {
        pool_weight[row0 + threadIdx.x] = 0.0f;
        if (pool_dst) pool_dst[row0 + threadIdx.x] = 0;
    }
}

void moe_unpack_meta(const uint8_t* side, int recv_count_capacity, const int* totals, int world, int local_experts, int hidden,
                     const int* seg_src_offset, const int* seg_pool_offset, uint8_t* pool_scales, float* pool_weight,
                     int* pool_dst, cudaStream_t stream) {
    check_hidden(hidden, "moe unpack_meta");
    if (recv_count_capacity <= 0) return;
    if (!side || !pool_scales || !pool_weight || !pool_dst) throw std::invalid_argument("moe unpack_meta: null pointer");
    launch_chained(unpack_meta_kernel, dim3((size_t(recv_count_capacity) * 32 + 255) / 256), dim3(256), size_t(0), stream, 
        side, totals, world * local_experts, hidden, seg_src_offset, seg_pool_offset, pool_scales, pool_weight, pool_dst,
        local_experts);
}

void moe_clear_live(const int* num_blocks, int block_rows, int pool_rows, int hidden, uint8_t* pool_scales,
                    float* pool_weight, int* pool_dst, cudaStream_t stream) {
    check_hidden(hidden, "moe clear_live");
    if (!num_blocks || !pool_scales || !pool_weight || pool_rows <= 0 || pool_rows % 128 || (block_rows != 128 && block_rows != 256))
        throw std::invalid_argument("moe clear_live: bad argument");
    launch_chained(clear_live_kernel, dim3(pool_rows / 128), dim3(256), size_t(0), stream, num_blocks, block_rows, hidden, pool_scales, pool_weight, pool_dst);
}

int moe_payload_bytes(int hidden) { return payload_bytes(hidden); }

// ---- barrier (+ small all-gather) between the GPUs of one node over peer memory --------------------------
//
// Every rank owns one PeerState in memory that all the others map. An exchange with sequence number e (one
// more than this rank's last): write this rank's payload into row `rank` of slot e & 1 of every rank's
// payload area, fence, store e into arrived[rank] of every rank, wait until all of this rank's own arrived[]
// words have reached e, copy the gathered rows out. One CTA per GPU; the kernels of one exchange run on
// different GPUs, never two on the same one. The wait is bounded: after WAIT_LIMIT_NS the kernel sets
// STATUS_TIMEOUT_PEER, leaves its sequence number unchanged (the next call repeats the same exchange) and
// returns. The payload slots alternate so that a rank already at exchange e + 1
// cannot overwrite rows a slower rank is still copying out of exchange e; it cannot get to e + 2 before that
// rank has arrived at e + 1.
using ptx::globaltimer_ns;
using ptx::WAIT_LIMIT_NS;
using ptx::STATUS_TIMEOUT_PEER;

struct PeerState {
    uint32_t epoch;
    uint32_t pad0[31];
    uint32_t arrived[64];
    uint32_t pad1[32];
    int payload[1];                 // [2][world][max_ints]
};
constexpr size_t PEER_STATE_HEADER = offsetof(PeerState, payload);

__global__ void peer_exchange_kernel(PeerState* own, PeerState* const* peers, int world, int rank,
                                     const int* __restrict__ payload, int ints, int max_ints, int* __restrict__ out,
                                     uint32_t* status, const long long* __restrict__ ids, int routes) {
    // No chain_point() here, and an ordinary launch: the kernels in front of a barrier store into other GPUs'
    // memory, and only the ordinary end of a kernel (not the early start of its dependent) is what makes those
    // stores complete before this kernel tells the peers so.
    extern __shared__ int histogram[];                          // [ints], only when ids are given
    __shared__ uint32_t next_epoch;
    __shared__ int failed;
    if (threadIdx.x == 0) { next_epoch = own->epoch + 1u; failed = 0; }
    if (ids) {
        // the payload is the histogram of this rank's routes over the experts, taken here (small batches):
        // saves the memset and the counting kernel in front of the exchange
        for (int e = threadIdx.x; e < ints; e += blockDim.x) histogram[e] = 0;
        __syncthreads();
        for (int i = threadIdx.x; i < routes; i += blockDim.x) {
            const long long e = ids[i];
            if (e >= 0 && e < ints) atomicAdd(&histogram[int(e)], 1);
        }
        payload = histogram;
    }
    __syncthreads();
    const uint32_t e = next_epoch;
    const size_t slot = size_t(e & 1u) * world;
    for (int r = 0; r < world && ints > 0; ++r) {
        int* dst = peers[r]->payload + (slot + rank) * max_ints;
        for (int i = threadIdx.x; i < ints; i += blockDim.x) dst[i] = payload[i];
    }
    __threadfence_system();
    __syncthreads();
    if (int(threadIdx.x) < world) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(&peers[threadIdx.x]->arrived[rank]), "r"(e) : "memory");
        const uint64_t start = globaltimer_ns();
        while (true) {
            uint32_t seen;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(&own->arrived[threadIdx.x]) : "memory");
            if (int32_t(seen - e) >= 0) break;
            if (globaltimer_ns() - start > WAIT_LIMIT_NS) {
                atomicOr(status, uint32_t(STATUS_TIMEOUT_PEER));
                atomicCAS(status + 1, 0u, 0x40000000u | (uint32_t(threadIdx.x) << 16) | (e & 0xFFFFu));
                failed = 1;
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    if (!failed && ints > 0) {
        const int* src = own->payload + slot * max_ints;
        for (int r = 0; r < world; ++r)
            for (int i = threadIdx.x; i < ints; i += blockDim.x) out[r * ints + i] = __ldcg(src + size_t(r) * max_ints + i);
    }
    // After a wait that ran out the sequence number stays where it was: the next exchange repeats number e, so a
    // rank whose partner had not launched yet (and will start from e as well) falls back into step with it.
    if (threadIdx.x == 0 && !failed) own->epoch = e;
}

size_t peer_state_bytes(int world, int max_ints) {
    if (world < 1 || world > 64 || max_ints < 0) throw std::invalid_argument("peer state: 1..64 ranks");
    return PEER_STATE_HEADER + size_t(2) * world * std::max(max_ints, 1) * sizeof(int);
}

void peer_exchange(void* own, void* const* peers_device, int world, int rank, const int* payload, int ints, int max_ints,
                   int* out, const long long* ids, int routes, cudaStream_t stream) {
    if (!own || !peers_device || world < 1 || world > 64 || rank < 0 || rank >= world)
        throw std::invalid_argument("peer exchange: bad state, table or rank");
    if (ints < 0 || ints > max_ints || (ints > 0 && ((!payload && !ids) || !out))) throw std::invalid_argument("peer exchange: bad payload");
    if (ids && (ints < 1 || ints > 4096 || routes < 0)) throw std::invalid_argument("peer exchange: a histogram needs 1..4096 bins");
    int device = 0;
    cuda_check(cudaGetDevice(&device));
    peer_exchange_kernel<<<1, 256, ids ? size_t(ints) * sizeof(int) : 0, stream>>>(static_cast<PeerState*>(own), reinterpret_cast<PeerState* const*>(peers_device), world, rank, payload, ints, max_ints, out,
        device_status_word(device), ids, routes);
    cuda_check(cudaGetLastError());
}

}  // namespace nvfp4_b200
