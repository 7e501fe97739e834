// NVFP4 block-scaled GEMM for B200 (sm_100a): C[M,N] fp16 = alpha * (A sfA)(B sfB)^T.
//
// One persistent kernel, three roles per CTA (192 or 320 threads):
//   warps 0-3  epilogue: TMEM -> registers -> FP16 -> swizzled shared memory -> TMA store, or straight to
//              global memory (then warps 6-9 are a second set, two warps per Tensor Memory lane quarter)
//   warp  4    MMA issuer (one elected lane): scale copies into TMEM + tcgen05 block-scaled MMAs
//   warp  5    producer  (one elected lane): TMA tile loads of packed operands and scale atoms
// A ring stage carries K = 256 of everything one MMA group needs (A rows, B rows,
// SFA atoms, SFB atoms) behind a single "full" barrier, so the issuer waits once
// per four MMAs. Accumulators are double-buffered in Tensor Memory; for 256-wide
// tiles the two buffers overlap by the width of the scale columns and the
// epilogue drains the shared columns first. Tiles are visited in bands of
// `group_m` tile rows, serpentine along N, computed arithmetically per tile (no
// table, no global state) so that the tiles in flight share A and B panels in L2.
// With CTA pairs (cta_group::2) each CTA loads its own half of A and B and both
// scale halves of B itself: no load in this file is multicast.
//
// Replaces the reference's kernels/gemm/matmul/sm100.cu (prepare/launch/validate
// at :701-737, kernel at :393-529) behind the same C++ interface.
#include "nvfp4.h"
#include "nvfp4_internal.h"
#include "ptx.cuh"
#include "quant_device.cuh"

#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

namespace nvfp4_b200 {

std::atomic<unsigned long long> g_launches{0};

namespace {

using namespace ptx;

constexpr int BLOCK_M = 128;        // rows of C per CTA (= TMEM lanes)
constexpr int STAGE_K = 256;        // K values per ring stage: 128 bytes of packed FP4 per row
constexpr int MMA_K = 64;           // K values per tcgen05.mma of this kind
constexpr int ROW_BYTES = STAGE_K / 2;
constexpr int SF_ATOM_BYTES = 512;  // 128 rows x 4 scale bytes (K = 64)
constexpr int EPI_COLS = 64;        // FP16 columns per epilogue chunk: one 128-byte line per row
constexpr int TMEM_COLS = 512;
constexpr int SMEM_LIMIT = 232448;  // 227 KiB opt-in maximum per CTA

// Device-side status, four words per slot: [0] OR of StatusBits, [1] tag of the first wait that gave up,
// [2] (slot 0 only) SM cycles the first CTA of the most recent GEMM launch was resident (diagnostic),
// [3] launches-times-clusters that found themselves on the other L2 side than their tile route assumed.
// Slot 0 is the device's own (grouped launches, the expert-path kernels, the barrier kernel); every dense
// plan gets one of the other slots, so that validating one plan neither reports nor clears another's error
// (more than STATUS_SLOTS - 1 live plans share slots, which only merges their reports).
constexpr int STATUS_SLOTS = 1024;
__device__ uint32_t g_status[STATUS_SLOTS][4];

// Epilogue routes, one kernel instance each (the route is a template parameter, so an instance carries
// only its own epilogue).
enum Epi : int {
    EPI_TMA = 0,           // rows staged in swizzled shared memory, C written by TMA stores (CTA pairs)
    EPI_DIRECT = 1,        // C written from registers with 32-byte global stores
    EPI_ACT = 2,           // grouped: clamped SwiGLU + route weight + NVFP4 re-quantisation, no C
    EPI_SCATTER = 3,       // grouped: every row to its own destination buffer, register stores
    EPI_SCATTER_ROWS = 4,  // grouped, CTA pairs: whole tile rows staged, one bulk copy per row
    EPI_GATHER_TMA = 5,    // the slab to every rank's full C by TMA stores
    EPI_GATHER_DIRECT = 6, // the same with register stores
    EPI_SPLIT_K = 7,       // FP32 partial sums + finish (to C or to every rank's full C)
    EPI_DIRECT_RAGGED = 8, // EPI_DIRECT on single-CTA tiles of unequal width (see GemmArgs::ragged_base)
    EPI_DIRECT_EDGE = 9,   // EPI_DIRECT with rows >= M and columns >= N masked (M, N not multiples of the tile), 16-byte stores
};

// MX: the MXFP4 flavour of the same instruction: one UE8M0 (power-of-two) scale per 32 values, so a 512-byte
// scale atom (128 rows x 4 scales) covers K = 128 and each MMA (K = 64) uses two of its four scale bytes.
template <int CG, int UN, int EPI, bool MX = false>
struct Config {
    static_assert(CG == 1 || CG == 2, "cta group");
    static_assert(UN == 128 || UN == 256, "tile width");
    static constexpr int TILE_M = BLOCK_M * CG;
    static constexpr int B_ROWS = UN / CG;                       // B rows staged by each CTA
    static constexpr int A_BYTES = BLOCK_M * ROW_BYTES;
    static constexpr int B_BYTES = B_ROWS * ROW_BYTES;
    static constexpr int SF_SLOTS = MX ? STAGE_K / 128 : STAGE_K / MMA_K;      // scale atoms per 128 rows and ring stage
    static constexpr int SFA_BYTES = SF_SLOTS * SF_ATOM_BYTES;
    static constexpr int SFB_BLOCKS = UN / 128;                  // 128-row scale blocks across the tile width
    static constexpr int SFB_BLOCK_BYTES = SF_SLOTS * SF_ATOM_BYTES;
    static constexpr int SFB_BYTES = SFB_BLOCKS * SFB_BLOCK_BYTES;
    static constexpr int OFF_B = A_BYTES;
    static constexpr int OFF_SFA = OFF_B + B_BYTES;
    static constexpr int OFF_SFB = OFF_SFA + SFA_BYTES;
    static constexpr int STAGE_BYTES = OFF_SFB + SFB_BYTES;
    static constexpr int EPI_WARP_BYTES = 32 * EPI_COLS * 2;     // 32 rows x 128 B
    // Routes that write from registers keep no staging and get a deeper ring where it fits (their
    // workloads stream weights from HBM and live on bytes in flight).
    static constexpr bool STAGED_EPILOGUE = EPI == EPI_TMA || EPI == EPI_GATHER_TMA;
    // Row staging (the scatter epilogue of the second expert GEMM on CTA pairs): instead of two 32 x 64
    // chunk buffers per warp, every epilogue warp keeps its 32 whole rows of the tile (UN columns, 16 bytes
    // of padding per row so that a quarter-warp's 16-byte stores cover all banks); the ring gives up a
    // stage for it.
    static constexpr bool ROW_STAGING = EPI == EPI_SCATTER_ROWS;
    // Epilogue warps. A warp reaches only the Tensor Memory lanes of its quarter (warp % 4), so the routes that
    // write from registers run two warps per quarter, each with every other 64-column chunk: a 128 x 256
    // accumulator leaves in half the time, which is what bounds tiles with a short K loop and the tail of a
    // launch with one tile per CTA. The routes that stage in shared memory keep one warp per quarter (a second
    // set of staging buffers would cost a ring stage), as does split-K.
    static constexpr int EPI_WARPS = (EPI == EPI_DIRECT || EPI == EPI_ACT || EPI == EPI_SCATTER || EPI == EPI_GATHER_DIRECT ||
                                      EPI == EPI_DIRECT_RAGGED || EPI == EPI_DIRECT_EDGE) ? 8 : 4;
    static constexpr bool RAGGED = EPI == EPI_DIRECT_RAGGED;
    static_assert(!RAGGED || (CG == 1 && UN == 256), "ragged tiles are single-CTA tiles of up to 256 columns");
    static constexpr int THREADS = (2 + EPI_WARPS) * 32;        // warps 0-3 epilogue, 4 MMA, 5 producer, 6-9 epilogue
    static constexpr int ROW_PITCH = UN * 2 + 16;
    static constexpr int EPI_BYTES = ROW_STAGING ? 4 * 32 * ROW_PITCH : STAGED_EPILOGUE ? 4 * 2 * EPI_WARP_BYTES : 0;
    static constexpr int CTRL_BYTES = 1024;
    static constexpr int STAGES = (SMEM_LIMIT - 1024 - CTRL_BYTES - EPI_BYTES) / STAGE_BYTES;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + EPI_BYTES + CTRL_BYTES;
    // Tensor Memory columns: scale columns for the four MMAs of a stage at the top,
    // two accumulators below them (overlapping when they cannot both fit).
    static constexpr int SF_COLS_PER_MMA = 4 + UN / 32;          // columns of one atom of SFA and the tile's atoms of SFB
    static constexpr int SF_COLS = SF_SLOTS * SF_COLS_PER_MMA;
    static constexpr int SF_BASE = TMEM_COLS - SF_COLS;
    static constexpr int ACC_STRIDE = (2 * UN <= SF_BASE) ? UN : SF_BASE - UN;
    static constexpr int OVERLAP = UN - ACC_STRIDE;              // columns shared by the two accumulators
    static_assert(OVERLAP <= EPI_COLS, "the first epilogue chunk must cover the overlap");
    static_assert(STAGE_BYTES % 1024 == 0, "stages keep the 1024-byte swizzle alignment");
    static_assert(STAGES >= 3 && STAGES <= 8, "ring depth");
    static_assert(!STAGED_EPILOGUE || CG == 2, "single CTAs write C from registers");
    // Instruction descriptor of kind::mxf4nvf4: A and B E2M1 (format 1) at bits 7 and 10,
    // both K-major, N >> 3 at bit 17, UE4M3 scales (bit 23 = 0), M >> 4 at bit 24,
    // scale-factor ids 0 (each MMA reads whole 32-bit scale columns).
    // MX: scale format UE8M0 (bit 23); the scale-factor ids (bits 29-30 for A, 4-5 for B) are set per MMA.
    static constexpr uint32_t IDESC = (1u << 7) | (1u << 10) | (uint32_t(UN >> 3) << 17) |
                                      (uint32_t(TILE_M >> 4) << 24) | (MX ? (1u << 23) : 0u);
};

struct Control {
    uint64_t full[8], empty[8];
    uint64_t acc_full, acc_free;
    uint32_t tmem_base;
    WaitCtl wait;
};
static_assert(sizeof(Control) <= 1024, "control block");

struct GemmArgs {
    int M, N, K;
    int ksteps;                     // ring steps per tile: ceil(K / 256); a last partial step reads zero fill
    int tiles_m, tiles_n, group_m;
    float alpha;
    uint32_t* status;               // this plan's four status words ([0] StatusBits, [1] first tag, [3] placement misses)
    uint32_t* cycles;               // where CTA 0 leaves the SM cycles it was resident (diagnostic)
    unsigned long long* prof;       // PROF instances only: per-unit wait/role cycle counters (16 words per CTA)
    int c_evict_first;              // store C with the evict-first L2 policy
    int out_bf16;                   // 1: C is bfloat16 instead of float16
    // Grouped mode (routed-MoE experts): A is a pool of 128-row blocks, block i belongs to expert
    // block_expert[i] and multiplies rows [expert * b_rows_per_expert, +N) of the stacked B. The
    // number of live blocks is only known on the device. Null block_expert = one dense GEMM.
    const int* block_expert;
    const int* num_blocks;
    int b_rows_per_expert;
    // Grouped mode, EPI_DIRECT_EDGE: block i holds block_valid[i] real rows followed by padding, and only the real
    // rows of C are written (a pool of 128-row blocks with a few routes per expert is mostly padding: at 1024
    // tokens, 256 experts, top-6 the second expert GEMM wrote 248 MB where 50 MB are rows anyone reads).
    const int* block_valid;
    void* c;                        // C base and leading dimension (elements), used by the register-store routes
    int ldc;
    // EPI_ACT (grouped mode only): the weight rows arrive interleaved as 16 gate rows, 16 up rows, ..., so a
    // lane's 64 accumulator columns are two (gate, up) block pairs; the epilogue rounds them to bf16, applies
    // the clamped SwiGLU and the row's route weight, rounds to bf16, quantises each 16-value block to NVFP4
    // and writes packed codes and scale bytes for the second GEMM.
    uint8_t* act_packed;            // [pool_rows, N/4] (N/2 activation columns, two per byte)
    uint8_t* act_scales;            // VEC16 layout of [pool_rows, N/2]
    const float* row_weight;        // [pool_rows]
    float swiglu_clamp;
    // EPI_SCATTER / EPI_SCATTER_ROWS (second expert GEMM + combine): row r of the pool is not written to C but
    // to row (row_dst[r] & 0xFFFFFF) - 1 of the [slot_rows, N] buffer of rank row_dst[r] >> 24 (peer memory
    // over NVLink, or this rank's own buffer); row_dst[r] == 0 marks a padding row.
    const int* row_dst;
    void* const* slots;             // device array of `world` buffer addresses
    int world;
    int slot_rows;
    // Tile t walks K starting at step (t * k_skew) % ksteps and wraps: the CTAs then do not all ask HBM for
    // the same 128-byte column of their rows at the same time. 0 = every tile starts at K = 0.
    int k_skew;
    // EPI_SPLIT_K (dense mode, shapes with far fewer tiles than SMs): unit u works on K steps
    // [slice * steps / S, (slice + 1) * steps / S) of tile u / S, slice = u % S, and writes FP32 partial sums
    // to its slot of sk_partials. When the S slices of a tile are there (flags), slice j adds them up, in
    // slice order, for the column chunks c with c % S == j and writes those columns of C. One item per
    // unit: the grid is tiles * S CTAs (or pairs), all resident at once.
    int split_k;                    // S; 0 or 1 = off
    float* sk_partials;             // [units][CG][4 warps][UN/64 chunks][16][32 lanes] float4
    uint32_t* sk_flags;             // [units][CG][4 warps]: partial sums published
    uint32_t* sk_done;              // [tiles][CG][4 warps]: readers finished (the last one lowers the flags)
    // GEMM fused with the all-gather of C (dense mode, N sharded over ranks): this rank's column slab is
    // written into the full [M, gather_ldc] C of EVERY rank, its own and its peers' (NVLink), from the
    // epilogue: TMA stores through one tensor map per destination (EPI_GATHER_TMA) or register stores
    // (EPI_GATHER_DIRECT, and the finish of EPI_SPLIT_K).
    int gather_world;
    int gather_col0;                // first column of this rank's slab in the full C
    int gather_ldc;                 // columns of the full C
    const CUtensorMap* gather_maps; // [gather_world] in device memory, written by the host before any launch
    void* const* gather_ptrs;       // [gather_world] bases of the full C buffers
    // L2-side-aware order (dense mode): work item w (= unit + trip * units) is tile route[w] of the band order
    // instead of tile w. The table keeps the clusters that sit on one side of the L2 on one contiguous part
    // of the band sequence. sm_side[smid] and unit_side[unit] are what the census saw; a cluster that finds
    // itself on the other side than the table assumed only counts a placement miss (results do not depend on it).
    const uint32_t* route;
    const uint8_t* sm_side;
    const uint8_t* unit_side;
    // What the launch in front of this one in the stream may still be writing when this kernel starts (it can
    // start early under programmatic dependent launch): 0 = anything, so every thread waits for that grid before
    // it touches global memory; 1 = not B and its scales (weights that were there long before): the first ring
    // stages of B are requested before the wait; 2 = none of the operands: only the epilogue waits, before its
    // first store, so the tiles of this launch run while the tail of the previous one drains.
    int static_operands;
    // EPI_DIRECT_RAGGED (one tile row, M = 128): the N columns are dealt to exactly as many tiles as there are
    // SMs, in units of 64 columns: the first ragged_extra tiles are ragged_base + 1 units wide, the others
    // ragged_base (2 or 3), so that no SM is left without a tile when N / 256 is smaller than the SM count. B is
    // fetched in 64-row boxes; a tile's scale atoms are the two 128-row blocks its columns lie in, and the MMA
    // reads them from the column (n0 % 128) / 32 on.
    int ragged_base, ragged_extra;
};

// First column and width of tile tn of a ragged row of tiles.
__device__ __forceinline__ void ragged_span(const GemmArgs& g, int tn, int& n0, int& width) {
    const int wide = g.ragged_base + 1;
    if (tn < g.ragged_extra) {
        n0 = tn * wide * 64;
        width = wide * 64;
    } else {
        n0 = (g.ragged_extra * wide + (tn - g.ragged_extra) * g.ragged_base) * 64;
        width = g.ragged_base * 64;
    }
}

struct Segment {
    uint32_t tile, item;            // item = position in the work sequence (tile * S + slice)
    int k0, k1;                     // ring steps [k0, k1) of the tile
};
// The sequence of segments one unit works through; every role of the unit builds the same one.
struct Walk {
    uint32_t next, stride, tiles;
    int ksteps, split;
    const uint32_t* route;
    __device__ Walk(const GemmArgs& g, uint32_t unit, uint32_t units, uint32_t tiles_, int ksteps_)
        : next(unit), stride(units), tiles(tiles_), ksteps(ksteps_), split(g.split_k > 1 ? g.split_k : 1), route(g.route) {}
    __device__ bool get(Segment& s) {
        if (next >= tiles * uint32_t(split)) return false;
        s.item = next;
        const uint32_t whole = next / uint32_t(split);           // the route table is only used with whole tiles
        s.tile = route ? __ldg(route + next) : whole;
        const int slice = int(next - whole * uint32_t(split)), len = ksteps / split;
        s.k0 = slice * len;
        s.k1 = s.k0 + len;
        next += stride;
        return true;
    }
};

enum ProfSlot { PROF_PROD_WAIT = 0, PROF_PROD_TOTAL, PROF_MMA_WAIT_FULL, PROF_MMA_WAIT_ACC, PROF_MMA_TOTAL,
                PROF_EPI_WAIT_ACC, PROF_EPI_WAIT_STORE, PROF_EPI_TOTAL, PROF_SMID,
                // %globaltimer (ns) when the CTA entered, when its issuer saw the first stage land, when the issuer
                // had issued its last step, when epilogue warp 0 had written its last row
                PROF_T_ENTER, PROF_T_FIRST_DATA, PROF_T_LAST_ISSUE, PROF_T_EPI_DONE, PROF_WORDS = 16 };
// After the per-CTA counters: for the first TR_TILES tiles of unit 0, eight clock64 stamps around the
// tile hand-over {0 issuer: last step issued, 1 issuer: acc_free seen, 2 issuer: first step of the
// next tile issued, 3 leader epilogue warp 0: acc_full seen, 4 same: first chunk loaded,
// 5 same: acc_free arrival sent, 6 peer CTA epilogue warp 0: acc_full seen, 7 peer: arrival sent}.
constexpr int TR_TILES = 16;
constexpr size_t SPLIT_K_FLAG_BYTES = 8192;    // [0, 4096): 4 flags per CTA, up to 256 CTAs; [4096, 8192): readers' counters per tile


// Shared-memory matrix descriptors (built in Roles::issue from two 32-bit halves):
//   operands: K-major rows of 128 bytes under the 128-byte swizzle: start address >> 4, stride
//             between 8-row groups 1024 B (>> 4) at bit 32, version 1 at bit 46, swizzle mode 2
//             (128 B) at bit 61; K advances by adding 32 B to the start address inside the row;
//   scale atoms: 32 rows of 16 bytes, no swizzle: 8-row groups 128 B apart (bit 32), 16 B leading
//             offset (bit 16), version 1.

// Tile t of the persistent sequence -> tile coordinates. Bands of `group_m` tile
// rows, column-major inside a band, bands alternate direction along N.
__device__ __forceinline__ void tile_coords(int t, const GemmArgs& g, int& tm, int& tn, int& b_base) {
    if (g.block_expert) {
        // grouped: all N tiles of one row block are consecutive, so an expert's weights are streamed once
        tm = t / g.tiles_n;
        tn = t - tm * g.tiles_n;
        b_base = __ldg(g.block_expert + tm) * g.b_rows_per_expert;
        return;
    }
    b_base = 0;
    const int per_band = g.group_m * g.tiles_n;
    const int band = t / per_band;
    const int first = band * g.group_m;
    const int rows = min(g.group_m, g.tiles_m - first);
    const int r = t - band * per_band;
    const int c = r / rows;
    tm = first + r - c * rows;
    tn = (band & 1) ? g.tiles_n - 1 - c : c;
}

template <int CG, int UN, int EPI, bool PROF, bool MX = false>
struct Roles {
    using Cfg = Config<CG, UN, EPI, MX>;

    uint32_t smem;            // 1024-aligned shared-window address of stage 0
    Control* ctrl;
    uint32_t rank, unit, units, tiles, peer_abort;
    const GemmArgs& g;

    __device__ __forceinline__ uint32_t bar(const uint64_t* b) const { return smem_u32(b); }
    __device__ __forceinline__ bool wait(const uint64_t* b, uint32_t parity, uint32_t who, uint32_t tag) const {
        if (mbar_wait(bar(b), parity, &ctrl->wait, g.status, who, peer_abort)) return true;
        if (who) atomicCAS(g.status + 1, 0u, tag);
        return false;
    }
    static __device__ __forceinline__ long long now() { return PROF ? clock64() : 0; }

    // Both single-issuer roles below run their loops with the WHOLE warp in uniform control
    // flow and let one elected lane execute the asynchronous instructions. Addresses,
    // descriptors and coordinates are then warp-uniform values the compiler can keep in
    // uniform registers, which is what TMA and tcgen05 instructions take; computing them
    // inside a one-lane branch costs a register-to-uniform move chain per instruction.

    // ---- warp 5: stream operand and scale tiles into the ring ----------------------
    // The scale maps are three-dimensional {128 bytes, 4 * K/64 rows, row blocks}: one 16-row box is the four
    // atoms of a K = 256 step, and a last partial step reads zeros beyond the block's own atoms (as the
    // operand maps do beyond K/2 bytes), so K only has to be a multiple of 64.
    __device__ void produce(const CUtensorMap* tmA, const CUtensorMap* tmB,
                            const CUtensorMap* tmSFA, const CUtensorMap* tmSFB, int lane) const {
        int stage = 0;
        uint32_t phase = 0;
        const int ksteps = g.ksteps;
        long long waited = 0;
        const long long born = now();
        // static_operands == 1: the A halves of the first ring fill wait for the grid in front of this launch
        const bool early_b = g.static_operands == 1;
        Held held[Cfg::STAGES];
        int issued = 0;
        Walk walk(g, unit, units, tiles, ksteps);
        Segment seg;
        while (walk.get(seg)) {
            const uint32_t t = seg.tile;
            int tm, tn, b_base;
            tile_coords(int(t), g, tm, tn, b_base);
            const int a_row = tm * Cfg::TILE_M + int(rank) * BLOCK_M;
            int b_row = b_base + tn * UN + int(rank) * Cfg::B_ROWS;
            const int sfa_block = a_row / 128;
            int sfb_block = (b_base + tn * UN) / 128;
            int b_boxes = 1;                                    // 64-row boxes of B per stage (ragged tiles only)
            uint32_t stage_bytes = Cfg::STAGE_BYTES;
            if constexpr (Cfg::RAGGED) {
                int n0, width;
                ragged_span(g, tn, n0, width);
                b_row = n0;
                sfb_block = n0 / 128;
                b_boxes = width / 64;
                stage_bytes = Cfg::A_BYTES + uint32_t(width) * ROW_BYTES + Cfg::SFA_BYTES + Cfg::SFB_BYTES;
            }
            // whole tiles may start anywhere in K and wrap; slices of a tile are walked in order
            const int k_first = (g.k_skew && g.split_k <= 1) ? int((t * uint32_t(g.k_skew)) % uint32_t(ksteps)) : 0;
            for (int step = seg.k0; step < seg.k1; ++step) {
                const int ks = step + k_first < ksteps ? step + k_first : step + k_first - ksteps;
                const long long w0 = now();
                const bool ok = wait(&ctrl->empty[stage], phase ^ 1u, lane == 0 ? STATUS_TIMEOUT_PRODUCER : 0u,
                                     0x10000000u | (stage << 16) | ks);
                if (!__all_sync(0xFFFFFFFFu, ok)) return;
                if (PROF) waited += now() - w0;
                const uint32_t base = smem + stage * Cfg::STAGE_BYTES;
                const uint32_t own_full = bar(&ctrl->full[stage]);
                // The first ring fill of a launch whose B is static goes out in two halves: B and its scales at
                // once, A and its scales after the grid in front of this launch has finished (see below).
                const bool split_issue = early_b && issued < Cfg::STAGES;
                if (split_issue) held[issued] = {ks, a_row, sfa_block};
                if constexpr (CG == 1) {
                    if (elect_one()) {
                        mbar_arrive_expect_tx(own_full, stage_bytes);
                        if (!split_issue) {
                            tma_load_2d(base, tmA, ks * ROW_BYTES, a_row, own_full);
                            tma_load_3d(base + Cfg::OFF_SFA, tmSFA, 0, ks * (Cfg::SF_SLOTS * 4), sfa_block, own_full);
                        }
                        if constexpr (Cfg::RAGGED) {
                            for (int u = 0; u < b_boxes; ++u)
                                tma_load_2d(base + Cfg::OFF_B + u * (64 * ROW_BYTES), tmB, ks * ROW_BYTES, b_row + 64 * u, own_full);
                        } else {
                            tma_load_2d(base + Cfg::OFF_B, tmB, ks * ROW_BYTES, b_row, own_full);
                        }
                        #pragma unroll
                        for (int b = 0; b < Cfg::SFB_BLOCKS; ++b)
                            tma_load_3d(base + Cfg::OFF_SFB + b * Cfg::SFB_BLOCK_BYTES, tmSFB, 0, ks * (Cfg::SF_SLOTS * 4),
                                        sfb_block + b, own_full);
                    }
                } else {
                    // Both CTAs of the pair report their bytes to the leader's barrier.
                    const uint32_t full = map_to_cta(own_full, 0);
                    if (elect_one()) {
                        if (rank == 0) mbar_arrive_expect_tx(own_full, 2 * Cfg::STAGE_BYTES);
                        if (!split_issue) {
                            tma_load_2d_pair(base, tmA, ks * ROW_BYTES, a_row, full);
                            tma_load_3d_pair(base + Cfg::OFF_SFA, tmSFA, 0, ks * (Cfg::SF_SLOTS * 4), sfa_block, full);
                        }
                        tma_load_2d_pair(base + Cfg::OFF_B, tmB, ks * ROW_BYTES, b_row, full);
                        #pragma unroll
                        for (int b = 0; b < Cfg::SFB_BLOCKS; ++b)
                            tma_load_3d_pair(base + Cfg::OFF_SFB + b * Cfg::SFB_BLOCK_BYTES, tmSFB, 0, ks * (Cfg::SF_SLOTS * 4),
                                             sfb_block + b, full);
                    }
                }
                ++issued;
                if (early_b && issued == Cfg::STAGES) release_held(tmA, tmSFA, held, Cfg::STAGES);
                if (++stage == Cfg::STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (early_b && issued < Cfg::STAGES) release_held(tmA, tmSFA, held, issued);   // fewer steps than ring stages
        if (PROF && lane == 0) {
            unsigned long long* out = g.prof + (size_t(unit) * CG + rank) * PROF_WORDS;
            out[PROF_PROD_WAIT] = waited;
            out[PROF_PROD_TOTAL] = now() - born;
        }
    }

    // The A halves (rows of A and their scale atoms) of the first `count` ring stages, once the grid this launch
    // depends on has finished: stage i of the ring, in issue order.
    struct Held { int ks, a_row, sfa_block; };
    __device__ void release_held(const CUtensorMap* tmA, const CUtensorMap* tmSFA, const Held* held, int count) const {
        grid_dependency_wait();
        if (elect_one()) {
            for (int i = 0; i < count; ++i) {
                const uint32_t base = smem + i * Cfg::STAGE_BYTES;
                const uint32_t own_full = bar(&ctrl->full[i]);
                if constexpr (CG == 1) {
                    tma_load_2d(base, tmA, held[i].ks * ROW_BYTES, held[i].a_row, own_full);
                    tma_load_3d(base + Cfg::OFF_SFA, tmSFA, 0, held[i].ks * (Cfg::SF_SLOTS * 4), held[i].sfa_block, own_full);
                } else {
                    const uint32_t full = map_to_cta(own_full, 0);
                    tma_load_2d_pair(base, tmA, held[i].ks * ROW_BYTES, held[i].a_row, full);
                    tma_load_3d_pair(base + Cfg::OFF_SFA, tmSFA, 0, held[i].ks * (Cfg::SF_SLOTS * 4), held[i].sfa_block, full);
                }
            }
        }
    }

    // ---- warp 4 of the leader CTA: scale copies and MMAs ------------------------------
    // Per ring step the warp spends its time on: noticing that the stage has landed, the 12
    // scale copies + 4 MMAs + commit, and loop control. The tensor pipe needs 4 x 128 cycles per
    // step, so the thread side has to stay clearly below that or the pipe runs dry at every
    // step. Two things keep it there: the barrier of the NEXT stage is probed (non-blocking)
    // before this stage's instructions are issued, so its latency hides behind them and the
    // blocking wait is skipped when the probe succeeded; and every descriptor is a uniform
    // 32-bit add on values computed outside the one-lane block.
    __device__ void issue(uint32_t tmem, int lane) const {
        int stage = 0;
        uint32_t phase = 0, iter = 0;
        const int ksteps = g.ksteps;
        long long wait_full = 0, wait_acc = 0;
        const long long born = now();
        // Descriptor words. Low word: start address >> 4 (bits 0-13), leading offset >> 4 (bits 16-29).
        // High word: stride >> 4 (bits 0-13), version 1 (bit 14), swizzle mode (bits 29-31).
        constexpr uint32_t OPERAND_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
        constexpr uint32_t SCALE_HI = (128u >> 4) | (1u << 14);
        constexpr uint32_t SCALE_LBO = (16u >> 4) << 16;
        const uint32_t ring_lo = (smem & 0x3FFFFu) >> 4;
        const uint32_t sf_tmem = tmem + Cfg::SF_BASE;
        bool landed = false;                                    // the probe of this step's barrier succeeded
        Walk walk(g, unit, units, tiles, ksteps);
        Segment seg;
        for (; walk.get(seg); ++iter) {
            const uint32_t acc = tmem + (iter & 1u) * Cfg::ACC_STRIDE;
            uint32_t idesc = Cfg::IDESC, sfb_shift = 0;
            if constexpr (Cfg::RAGGED) {
                int tm, tn, b_base, n0, width;
                tile_coords(int(seg.tile), g, tm, tn, b_base);
                ragged_span(g, tn, n0, width);
                idesc = (1u << 7) | (1u << 10) | (uint32_t(width >> 3) << 17) | (uint32_t(Cfg::TILE_M >> 4) << 24);
                sfb_shift = uint32_t(n0 % 128) / 32u;           // the tile's first row inside its first scale atom
            }
            unsigned long long* tr = nullptr;
            if (PROF && unit == 0 && lane == 0 && iter > 0 && iter <= TR_TILES)
                tr = g.prof + size_t(units) * CG * PROF_WORDS + size_t(iter - 1) * 8;
            for (int ks = seg.k0; ks < seg.k1; ++ks) {
                if (!landed) {
                    const long long w0 = now();
                    const bool ok = wait(&ctrl->full[stage], phase, lane == 0 ? STATUS_TIMEOUT_MMA : 0u,
                                         0x21000000u | (stage << 16) | ks);
                    if (!__all_sync(0xFFFFFFFFu, ok)) return;
                    if (PROF) wait_full += now() - w0;
                }
                if (PROF && iter == 0 && ks == seg.k0 && lane == 0)
                    g.prof[size_t(unit) * CG * PROF_WORDS + PROF_T_FIRST_DATA] = globaltimer_ns();
                tc_fence_after_sync();
                const int next_stage = stage + 1 == Cfg::STAGES ? 0 : stage + 1;
                const uint32_t next_phase = stage + 1 == Cfg::STAGES ? phase ^ 1u : phase;
                const bool probe = mbar_test_wait(bar(&ctrl->full[next_stage]), next_phase);
                const uint32_t lo = ring_lo + uint32_t(stage) * (Cfg::STAGE_BYTES >> 4);
                const uint32_t empty = bar(&ctrl->empty[stage]);
                const uint32_t first = ks != seg.k0 ? 1u : 0u;   // 0: the first MMA of the segment overwrites the accumulator
                // j: the MMA (K = 64) inside the stage. NVFP4: MMA j has its own scale atom j. MXFP4: MMAs 2a and 2a+1
                // share atom a (copied before the first of them) and read its bytes 0-1 and 2-3.
                auto copies = [&](int j) {
                    if (MX && (j & 1)) return;
                    const int slot = MX ? j / 2 : j;
                    const uint32_t sf = sf_tmem + slot * Cfg::SF_COLS_PER_MMA;
                    tmem_copy_scales<CG>(sf, (lo + ((Cfg::OFF_SFA + slot * SF_ATOM_BYTES) >> 4)) | SCALE_LBO, SCALE_HI);
                    #pragma unroll
                    for (int b = 0; b < Cfg::SFB_BLOCKS; ++b)
                        tmem_copy_scales<CG>(sf + 4 + 4 * b,
                                             (lo + ((Cfg::OFF_SFB + b * Cfg::SFB_BLOCK_BYTES + slot * SF_ATOM_BYTES) >> 4)) | SCALE_LBO,
                                             SCALE_HI);
                };
                auto mma = [&](int j) {
                    // K advances 32 bytes inside the 128-byte swizzled row per MMA.
                    const int slot = MX ? j / 2 : j;
                    const uint32_t sf = sf_tmem + slot * Cfg::SF_COLS_PER_MMA;
                    const uint32_t sf_id = MX ? uint32_t(j & 1) * 2u : 0u;
                    mma_block_scaled<CG, MX>(acc, lo + ((j * (MMA_K / 2)) >> 4), lo + ((Cfg::OFF_B + j * (MMA_K / 2)) >> 4),
                                             OPERAND_HI, idesc | (sf_id << 29) | (sf_id << 4), sf, sf + 4 + sfb_shift,
                                             j != 0 ? 1u : first);
                };
                const bool handover = ks == seg.k0 && iter > 0;
                if (handover) {
                    // First step of a tile: the scale copies do not touch the accumulators, so they go out
                    // before the wait for the epilogue to pull the columns this tile shares with the last one.
                    if (elect_one()) {
                        #pragma unroll
                        for (int j = 0; j < STAGE_K / MMA_K; ++j) copies(j);
                    }
                    const long long w0 = now();
                    if (tr) tr[0] = w0;
                    const bool ok = wait(&ctrl->acc_free, (iter - 1u) & 1u, lane == 0 ? STATUS_TIMEOUT_MMA : 0u, 0x20000000u | iter);
                    if (!__all_sync(0xFFFFFFFFu, ok)) return;
                    if (PROF) wait_acc += now() - w0;
                    if (tr) tr[1] = now();
                    tc_fence_after_sync();
                }
                if (elect_one()) {
                    #pragma unroll
                    for (int j = 0; j < STAGE_K / MMA_K; ++j) {
                        if (!handover) copies(j);
                        mma(j);
                    }
                    mma_commit<CG>(empty);                      // stage reusable once these MMAs retire
                    if (ks == seg.k1 - 1) mma_commit<CG>(bar(&ctrl->acc_full));
                }
                if (tr && ks == seg.k0) tr[2] = now();
                landed = __all_sync(0xFFFFFFFFu, probe);
                stage = next_stage;
                phase = next_phase;
            }
        }
        if (PROF && lane == 0) {
            unsigned long long* out = g.prof + size_t(unit) * CG * PROF_WORDS;
            out[PROF_MMA_WAIT_FULL] = wait_full;
            out[PROF_MMA_WAIT_ACC] = wait_acc;
            out[PROF_MMA_TOTAL] = now() - born;
            out[PROF_T_LAST_ISSUE] = globaltimer_ns();
        }
    }

    // Two accumulator values x alpha -> one packed FP16 (or BF16) pair.
    __device__ __forceinline__ uint32_t pack_pair(uint32_t lo_bits, uint32_t hi_bits, float alpha) const {
        const float lo = __uint_as_float(lo_bits) * alpha, hi = __uint_as_float(hi_bits) * alpha;
        if (g.out_bf16) {
            const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
            return *reinterpret_cast<const uint32_t*>(&p);
        }
        const __half2 p = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&p);
    }

    // 64 accumulator columns of this lane's row: x alpha, to FP16/BF16, 128 bytes in four 32-byte stores.
    __device__ __forceinline__ void store_row_chunk(uint16_t* dst, const uint32_t (&v)[EPI_COLS], float alpha, bool deliver) const {
        #pragma unroll
        for (int q = 0; q < EPI_COLS / 16; ++q) {
            uint32_t h[8];
            #pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = pack_pair(v[q * 16 + 2 * i], v[q * 16 + 2 * i + 1], alpha);
            if (deliver)
                asm volatile("st.global.L1::no_allocate.L2::evict_first.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                             :: "l"(dst + q * 16), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]),
                                "r"(h[4]), "r"(h[5]), "r"(h[6]), "r"(h[7]) : "memory");
        }
    }

    // The same for a tile that reaches beyond C: nothing leaves for a row >= M, and of the chunk's 64 columns only
    // the first cols_left (a multiple of 8: N is) are written, in 16-byte stores (a row of C starts on a 16-byte
    // boundary, not on a 32-byte one).
    __device__ __forceinline__ void store_row_chunk_edge(uint16_t* dst, const uint32_t (&v)[EPI_COLS], float alpha, bool row_ok,
                                                         int cols_left) const {
        #pragma unroll
        for (int q = 0; q < EPI_COLS / 8; ++q) {
            uint32_t h[4];
            #pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = pack_pair(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1], alpha);
            if (row_ok && q * 8 < cols_left)
                asm volatile("st.global.L1::no_allocate.v4.b32 [%0], {%1, %2, %3, %4};"
                             :: "l"(dst + q * 8), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
        }
    }

    // Destination of pool row `row` on the scatter routes: false = nothing to deliver (a padding row, or a
    // code outside the agreed buffers, which is reported through the status word).
    __device__ __forceinline__ bool scatter_target(int row, uint16_t*& base) const {
        const uint32_t code = uint32_t(__ldg(g.row_dst + row));
        if (code == 0u) return false;
        const uint32_t slot = (code & 0xFFFFFFu) - 1u, owner = code >> 24;
        if (slot >= uint32_t(g.slot_rows) || owner >= uint32_t(g.world)) {
            atomicOr(g.status, uint32_t(STATUS_BAD_ARGUMENT));
            return false;
        }
        base = reinterpret_cast<uint16_t*>(__ldg(reinterpret_cast<const unsigned long long*>(g.slots) + owner)) + size_t(slot) * g.ldc;
        return true;
    }

    // Split-K, once a unit's partial sums are stored: publish them, wait for the other slices of the tile, add
    // up, in slice order, this slice's share of the column chunks and write those columns of C. (Measured:
    // reading the slices with plain L2 loads, sixteen in flight per lane, takes 3.7k cycles per chunk of four
    // slices; staging them in shared memory with bulk copies took 11.6k.)
    __device__ bool split_k_finish(const Segment& seg, int warp, int lane, int row0, int col0, float alpha) const {
        const uint32_t S = uint32_t(g.split_k), first = seg.tile * S, slice = seg.item - first;
        __threadfence();
        __syncwarp();
        bool ok = true;
        if (lane == 0) {
            flag_publish(g.sk_flags + (seg.item * CG + rank) * 4 + warp, 1u);
            for (uint32_t i = 0; i < S && ok; ++i)
                ok = flag_wait(g.sk_flags + ((first + i) * CG + rank) * 4 + warp, &ctrl->wait, g.status,
                               STATUS_TIMEOUT_EPILOGUE, peer_abort);
            if (!ok) atomicCAS(g.status + 1, 0u, 0x31000000u | seg.item);
        }
        if (!__all_sync(0xFFFFFFFFu, ok)) return false;
        constexpr uint32_t CHUNK_FLOAT4 = 32 * EPI_COLS / 4;   // one warp's 32 rows x 64 columns of FP32
        constexpr uint32_t WARP_FLOATS = UN * 32;
        #pragma unroll 1
        for (uint32_t chunk = slice; chunk < UN / EPI_COLS; chunk += S) {
            uint32_t v[EPI_COLS];
            #pragma unroll 1
            for (uint32_t i = 0; i < S; ++i) {
                const float4* in = reinterpret_cast<const float4*>(g.sk_partials + ((size_t(first + i) * CG + rank) * 4 + warp) * WARP_FLOATS) +
                                   size_t(chunk) * CHUNK_FLOAT4 + lane;
                float4 part[EPI_COLS / 4];
                #pragma unroll
                for (int q = 0; q < EPI_COLS / 4; ++q) part[q] = __ldcg(in + q * 32);      // sixteen loads in flight per lane
                #pragma unroll
                for (int q = 0; q < EPI_COLS / 4; ++q) {
                    if (i == 0) {
                        v[4 * q] = __float_as_uint(part[q].x); v[4 * q + 1] = __float_as_uint(part[q].y);
                        v[4 * q + 2] = __float_as_uint(part[q].z); v[4 * q + 3] = __float_as_uint(part[q].w);
                    } else {
                        v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + part[q].x);
                        v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + part[q].y);
                        v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + part[q].z);
                        v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + part[q].w);
                    }
                }
            }
            if (g.gather_world) {
                const size_t at = size_t(row0 + lane) * g.gather_ldc + g.gather_col0 + col0 + chunk * EPI_COLS;
                for (int r = 0; r < g.gather_world; ++r)
                    store_row_chunk(reinterpret_cast<uint16_t*>(__ldg(reinterpret_cast<const unsigned long long*>(g.gather_ptrs) + r)) + at,
                                    v, alpha, true);
            } else {
                store_row_chunk(static_cast<uint16_t*>(g.c) + size_t(row0 + lane) * g.ldc + col0 + chunk * EPI_COLS, v, alpha, true);
            }
        }
        if (lane == 0) {
            uint32_t* done = g.sk_done + (seg.tile * CG + rank) * 4 + warp;
            if (atomicAdd(done, 1u) == S - 1) {                 // the last reader of this warp's rows lowers the flags
                for (uint32_t i = 0; i < S; ++i) g.sk_flags[((first + i) * CG + rank) * 4 + warp] = 0u;
                *done = 0u;
            }
        }
        return true;
    }

    // ---- warps 0-3: drain accumulators to C ---------------------------------------
    // warp: the Tensor Memory lane quarter this warp drains (rows warp * 32 .. + 31 of the CTA's 128);
    // half: with two warps per quarter, which of the alternating 64-column chunks are this warp's.
    __device__ void drain(uint32_t tmem, const CUtensorMap* tmC, int warp, int half, int lane) const {
        const uint32_t stage_base = smem + Cfg::STAGES * Cfg::STAGE_BYTES + warp * 2 * Cfg::EPI_WARP_BYTES;
        const uint32_t acc_free_leader = CG == 2 ? map_to_cta(bar(&ctrl->acc_free), 0) : bar(&ctrl->acc_free);
        uint32_t iter = 0, stores = 0;
        const float alpha = g.alpha;
        const uint64_t c_policy = policy_evict_first();
        long long wait_acc = 0, wait_store = 0;
        const long long born = now();
        // with static operands the prologue did not wait for the grid in front: nothing may be stored before it has finished
        if (g.static_operands != 0) grid_dependency_wait();
        Walk walk(g, unit, units, tiles, g.ksteps);
        Segment seg;
        constexpr uint32_t SK_WARP_FLOATS = UN * 32;            // one warp's 32 rows of a tile
        for (; walk.get(seg); ++iter) {
            const uint32_t t = seg.tile;
            int tm, tn, b_base;
            tile_coords(int(t), g, tm, tn, b_base);
            const int row0 = tm * Cfg::TILE_M + int(rank) * BLOCK_M + warp * 32;
            int col0 = tn * UN, chunks = UN / EPI_COLS;
            int row_limit = g.M;                                 // EPI_DIRECT_EDGE: first row that is not written
            if constexpr (EPI == EPI_DIRECT_EDGE || EPI == EPI_ACT) {
                if (g.block_valid) row_limit = tm * Cfg::TILE_M + __ldg(g.block_valid + tm);
            }
            if constexpr (Cfg::RAGGED) {
                int width;
                ragged_span(g, tn, col0, width);
                chunks = width / EPI_COLS;
            }
            // The whole warp leaves together: the Tensor Memory loads below are warp-collective.
            const long long w0 = now();
            const bool ready = wait(&ctrl->acc_full, iter & 1u, lane == 0 ? STATUS_TIMEOUT_EPILOGUE : 0u, 0x30000000u | iter);
            if (!__all_sync(0xFFFFFFFFu, ready)) break;
            if (PROF) wait_acc += now() - w0;
            unsigned long long* tr = nullptr;
            if (PROF && unit == 0 && warp == 0 && half == 0 && lane == 0 && iter < TR_TILES)
                tr = g.prof + size_t(units) * CG * PROF_WORDS + size_t(iter) * 8 + (rank ? 6 : 3);
            if (tr) tr[0] = now();
            tc_fence_after_sync();
            const uint32_t acc = tmem + (iter & 1u) * Cfg::ACC_STRIDE + (uint32_t(warp * 32) << 16);
            if (Cfg::EPI_WARPS == 8 && half == 1) {
                // This warp's chunks never include the columns the two accumulators share (those are chunk 0).
                // Its arrival says that it has left the previous tile, whose buffer the next tile's MMAs reuse.
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(acc_free_leader);
            }
            #pragma unroll 1
            for (int c = 0; c < chunks; ++c) {
                if (Cfg::EPI_WARPS == 8 && (c & 1) != half) continue;
                // Columns shared with the other accumulator go first: top of buffer 0, bottom of buffer 1.
                const int chunk = (iter & 1u) ? c : chunks - 1 - c;
                uint32_t v[EPI_COLS];
                tmem_ld_32x32(acc + chunk * EPI_COLS, v);
                tmem_ld_32x32(acc + chunk * EPI_COLS + 32, v + 32);
                tmem_ld_wait();
                if (c == 0) {
                    if (tr && rank == 0) tr[1] = now();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(acc_free_leader);
                    if (tr) tr[rank ? 1 : 2] = now();
                }
                if constexpr (EPI == EPI_SPLIT_K) {
                    // FP32 partial sums to this unit's slot: 16 bytes per lane, 512 contiguous bytes per store
                    float4* out = reinterpret_cast<float4*>(g.sk_partials + ((size_t(seg.item) * CG + rank) * 4 + warp) * SK_WARP_FLOATS) +
                                  size_t(chunk) * (EPI_COLS / 4) * 32 + lane;
                    #pragma unroll
                    for (int q = 0; q < EPI_COLS / 4; ++q)
                        __stcg(out + q * 32, make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                         __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3])));
                } else if constexpr (EPI == EPI_ACT) {
                    const int inter = g.N / 2;
                    const int row = row0 + lane;
                    const float w = __ldg(g.row_weight + row);
                    const int act_col = tn * (UN / 2) + chunk * (EPI_COLS / 2);        // first activation column of this chunk
                    uint2 codes[2];
                    uint32_t sb[2];
                    if (w == 0.0f) {
                        // padding row of the pool: the activation is zero (smallest scale, zero codes)
                        codes[0] = codes[1] = make_uint2(0u, 0u);
                        sb[0] = sb[1] = 0x01u;
                    } else {
                        const float cl = g.swiglu_clamp;
                        #pragma unroll
                        for (int b = 0; b < 2; ++b) {
                            uint32_t act[8];
                            #pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                float a2[2];
                                #pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    // gate_up is rounded to bf16 first, as the unfused pipeline stores it
                                    const uint32_t gb = v[b * 32 + 2 * i + h], ub = v[b * 32 + 16 + 2 * i + h];
                                    const float gate = fminf(__uint_as_float((gb + 0x7FFFu + ((gb >> 16) & 1u)) & 0xFFFF0000u), cl);
                                    const float up = fminf(fmaxf(__uint_as_float((ub + 0x7FFFu + ((ub >> 16) & 1u)) & 0xFFFF0000u), -cl), cl);
                                    a2[h] = silu_fast(gate) * up * w;
                                }
                                const __nv_bfloat162 p2 = __floats2bfloat162_rn(a2[0], a2[1]);
                                act[i] = *reinterpret_cast<const uint32_t*>(&p2);
                            }
                            sb[b] = quantise_block_pairs<Bf16Pairs>(act, codes[b]);
                        }
                    }
                    if (row < row_limit) {                        // the padding behind a block's real rows is not written: nobody reads it
                        *reinterpret_cast<uint4*>(g.act_packed + size_t(row) * (inter / 2) + act_col / 2) =
                            make_uint4(codes[0].x, codes[0].y, codes[1].x, codes[1].y);
                        *reinterpret_cast<uint16_t*>(g.act_scales + scale_byte_offset(row, act_col / 16, inter)) =
                            static_cast<uint16_t>(sb[0] | (sb[1] << 8));
                    }
                } else if constexpr (EPI == EPI_SCATTER_ROWS) {
                    // Scatter through shared memory: every lane stages its own row of the tile, chunk by chunk,
                    // and after the last chunk sends the UN columns (512 bytes) with ONE bulk copy to the row's
                    // destination. Over NVLink this makes 512-byte writes (register stores make 32-byte ones,
                    // which took 381 us for FC2 at 4096 tokens per GPU on two GPUs; one 128-byte copy per chunk
                    // took 233 us), and the warp does not wait for them. Bulk groups are per thread and each
                    // lane touches only its own row: no warp synchronisation is needed.
                    const uint32_t rowbuf = smem + Cfg::STAGES * Cfg::STAGE_BYTES + uint32_t(warp * 32 + lane) * Cfg::ROW_PITCH;
                    if (c == 0) tma_store_wait_read<0>();         // this lane's copy of the previous tile has read the row
                    #pragma unroll
                    for (int q = 0; q < EPI_COLS / 8; ++q) {
                        uint32_t h[4];
                        #pragma unroll
                        for (int i = 0; i < 4; ++i) h[i] = pack_pair(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1], alpha);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                     :: "r"(rowbuf + chunk * (EPI_COLS * 2) + q * 16), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
                    }
                    if (c == UN / EPI_COLS - 1) {
                        fence_async_smem();
                        uint16_t* dst = nullptr;
                        if (scatter_target(row0 + lane, dst)) {
                            bulk_store(dst + col0, rowbuf, UN * 2);
                            tma_store_commit();
                        }
                    }
                } else if constexpr (EPI == EPI_SCATTER) {
                    uint16_t* dst = nullptr;                      // a lane-wise predicate: the warp stays converged
                    const bool deliver = scatter_target(row0 + lane, dst);
                    store_row_chunk(dst + col0 + chunk * EPI_COLS, v, alpha, deliver);
                } else if constexpr (EPI == EPI_GATHER_DIRECT) {
                    const size_t at = size_t(row0 + lane) * g.gather_ldc + g.gather_col0 + col0 + chunk * EPI_COLS;
                    for (int r = 0; r < g.gather_world; ++r)
                        store_row_chunk(reinterpret_cast<uint16_t*>(__ldg(reinterpret_cast<const unsigned long long*>(g.gather_ptrs) + r)) + at,
                                        v, alpha, true);
                } else if constexpr (EPI == EPI_DIRECT || EPI == EPI_DIRECT_RAGGED) {
                    store_row_chunk(static_cast<uint16_t*>(g.c) + size_t(row0 + lane) * g.ldc + col0 + chunk * EPI_COLS, v, alpha, true);
                } else if constexpr (EPI == EPI_DIRECT_EDGE) {
                    store_row_chunk_edge(static_cast<uint16_t*>(g.c) + size_t(row0 + lane) * g.ldc + col0 + chunk * EPI_COLS, v, alpha,
                                         row0 + lane < row_limit, g.N - (col0 + chunk * EPI_COLS));
                } else {
                    // EPI_TMA / EPI_GATHER_TMA: the chunk goes through one of the warp's two swizzled buffers
                    const uint32_t buf = stage_base + (stores & 1u) * Cfg::EPI_WARP_BYTES;
                    const long long s0 = now();
                    if (lane == 0) tma_store_wait_read<1>();        // the store that last read this buffer is done
                    __syncwarp();
                    if (PROF) wait_store += now() - s0;
                    #pragma unroll
                    for (int q = 0; q < EPI_COLS / 8; ++q) {
                        uint32_t h[4];
                        #pragma unroll
                        for (int i = 0; i < 4; ++i) h[i] = pack_pair(v[q * 8 + 2 * i], v[q * 8 + 2 * i + 1], alpha);
                        // 128-byte swizzle: 16-byte chunk q of row `lane` lands in chunk q ^ (lane % 8).
                        const uint32_t dst = buf + lane * 128 + ((q ^ (lane & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                                     :: "r"(dst), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (EPI == EPI_GATHER_TMA) {
                            // the same staged tile to every rank's full C; one bulk group, so the buffer is reused
                            // only after all of them have read it
                            for (int r = 0; r < g.gather_world; ++r)
                                tma_store_2d(g.gather_maps + r, buf, g.gather_col0 + col0 + chunk * EPI_COLS, row0);
                        } else if (g.c_evict_first) {
                            tma_store_2d_hint(tmC, buf, col0 + chunk * EPI_COLS, row0, c_policy);
                        } else {
                            tma_store_2d(tmC, buf, col0 + chunk * EPI_COLS, row0);
                        }
                        tma_store_commit();
                    }
                    ++stores;
                }
            }
            if constexpr (EPI == EPI_SPLIT_K) {
                if (!split_k_finish(seg, warp, lane, row0, col0, alpha)) break;
            }
        }
        tma_store_wait_all();                                   // lanes without stores in flight fall through
        if (PROF && warp == 0 && half == 0 && lane == 0) {
            unsigned long long* out = g.prof + (size_t(unit) * CG + rank) * PROF_WORDS;
            out[PROF_EPI_WAIT_ACC] = wait_acc;
            out[PROF_EPI_WAIT_STORE] = wait_store;
            out[PROF_EPI_TOTAL] = now() - born;
            uint32_t smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            out[PROF_SMID] = smid;
            out[PROF_T_EPI_DONE] = globaltimer_ns();
        }
    }
};

template <int CG, int UN, int EPI, bool PROF, bool MX = false>
__global__ void __launch_bounds__(Config<CG, UN, EPI>::THREADS, 1)
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmSFA, const __grid_constant__ CUtensorMap tmSFB,
                  const __grid_constant__ CUtensorMap tmC, const GemmArgs g) {
    using Cfg = Config<CG, UN, EPI, MX>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t smem = (raw + 1023u) & ~1023u;
    Control* ctrl = reinterpret_cast<Control*>(smem_raw + (smem - raw) + Cfg::STAGES * Cfg::STAGE_BYTES + Cfg::EPI_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = CG == 2 ? cluster_ctarank() : 0u;
    const long long entered = clock64();

    // Programmatic dependent launch: a kernel launched behind this one with the stream-serialisation attribute
    // may bring its CTAs onto SMs that are free (and set up its barriers and Tensor Memory there) as soon as every
    // CTA of this grid has got here; it then waits in grid_dependency_wait() until this grid has finished.
    if (threadIdx.x == 0) grid_launch_dependents();
    if (PROF && threadIdx.x == 0) g.prof[(size_t(CG == 2 ? blockIdx.x / 2u : blockIdx.x) * CG + rank) * PROF_WORDS + PROF_T_ENTER] = globaltimer_ns();

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(smem_u32(&ctrl->full[s]), 1);
            mbar_init(smem_u32(&ctrl->empty[s]), 1);
        }
        mbar_init(smem_u32(&ctrl->acc_full), 1);
        mbar_init(smem_u32(&ctrl->acc_free), Cfg::EPI_WARPS * CG);   // one arrival per epilogue warp of the pair
        ctrl->wait.abort = 0;
        mbar_init_fence();
    }
    if (warp == 4) {
        tmem_alloc<CG>(smem_u32(&ctrl->tmem_base), TMEM_COLS);
        tmem_relinquish<CG>();
    }
    if (warp == 5 && lane == 0) {
        prefetch_tensormap(&tmA); prefetch_tensormap(&tmB);
        prefetch_tensormap(&tmSFA); prefetch_tensormap(&tmSFB);
        if constexpr (Cfg::STAGED_EPILOGUE) prefetch_tensormap(&tmC);
    }
    const uint32_t unit = CG == 2 ? blockIdx.x / 2u : blockIdx.x;
    if (g.unit_side && threadIdx.x == 32) {
        // the tile route was laid out for the L2 side this unit was seen on when the plan was prepared
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        if (smid < 256u && __ldg(g.sm_side + smid) != __ldg(g.unit_side + unit)) atomicAdd(g.status + 3, 1u);
    }
    tc_fence_before_sync();
    if constexpr (CG == 2) { cluster_arrive(); cluster_wait(); } else { __syncthreads(); }
    tc_fence_after_sync();
    const uint32_t tmem = ctrl->tmem_base;
    // Everything above touched only this CTA's own resources. From here on global memory is read and written:
    // wait for the grid this launch depends on (returns at once when the launch was an ordinary one), unless the
    // caller has declared operands that the grid in front cannot be writing (then the roles wait where they must).
    if (g.static_operands == 0) grid_dependency_wait();

    Roles<CG, UN, EPI, PROF, MX> roles{smem, ctrl, rank, unit, gridDim.x / CG,
                                   uint32_t(g.block_expert ? __ldg(g.num_blocks) : g.tiles_m) * uint32_t(g.tiles_n),
                                   CG == 2 ? map_to_cta(smem_u32(const_cast<uint32_t*>(&ctrl->wait.abort)), rank ^ 1u) : 0u, g};

    if (warp == 5) {
        roles.produce(&tmA, &tmB, &tmSFA, &tmSFB, lane);
    } else if (warp == 4) {
        if (rank == 0) roles.issue(tmem, lane);
    } else {
        roles.drain(tmem, &tmC, warp & 3, warp < 4 ? 0 : 1, lane);
    }
    __syncwarp();

    // Common teardown. After an abandoned wait, give copies still in flight time
    // to land before the CTA's shared memory is released.
    if (ctrl->wait.abort) {
        for (int i = 0; i < 200; ++i) __nanosleep(1000);
    }
    tc_fence_before_sync();
    if constexpr (CG == 2) { cluster_arrive(); cluster_wait(); } else { __syncthreads(); }
    if (warp == 4) {
        tc_fence_after_sync();
        tmem_dealloc<CG>(tmem, TMEM_COLS);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *g.cycles = uint32_t(clock64() - entered);
}


// ---- host side ---------------------------------------------------------------

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime so that the library
// loads (and exports its symbols) on a machine without a CUDA driver.
EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q{};
        cuda_check(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (!p || q != cudaDriverEntryPointSuccess) throw std::runtime_error("cuTensorMapEncodeTiled is unavailable");
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

// rank 2 or 3; shape[0] is the contiguous dimension, strides are those of dimensions 1.. in bytes
CUtensorMap make_map(CUtensorMapDataType type, const void* ptr, int rank, const cuuint64_t* shape,
                     const cuuint64_t* strides, const cuuint32_t* box, CUtensorMapSwizzle swizzle,
                     CUtensorMapL2promotion promo) {
    CUtensorMap map{};
    const cuuint32_t steps[3] = {1, 1, 1};
    const CUresult r = encode_tiled()(&map, type, cuuint32_t(rank), const_cast<void*>(ptr), shape, strides, box, steps,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, promo,
                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(int(r)));
    return map;
}

// Packed operand [rows, K/2] bytes, tiles of `box_rows` rows x 128 bytes, 128-byte swizzle. A box that
// reaches beyond K/2 bytes (the last step of a K that is not a multiple of 256) reads zeros there.
CUtensorMap operand_map(const uint8_t* p, int rows, int K, int box_rows) {
    const cuuint64_t shape[2] = {cuuint64_t(K / 2), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(K / 2)};
    const cuuint32_t box[2] = {ROW_BYTES, cuuint32_t(box_rows)};
    return make_map(CU_TENSOR_MAP_DATA_TYPE_UINT8, p, 2, shape, strides, box, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}
// The scale bytes of one 128-row block are K/64 atoms of 512 bytes = 4 * K/64 rows of 128 bytes; the map is
// {128 bytes, those rows, row blocks}, and one 16-row box is the four atoms of a K = 256 step (zeros beyond
// the block's last atom).
// atom_k: K values one scale atom covers (64 for NVFP4's scale per 16, 128 for MXFP4's scale per 32).
CUtensorMap scale_map(const uint8_t* p, int rows, int K, int atom_k = 64) {
    const cuuint64_t per_block = cuuint64_t(K / atom_k) * 4;
    const cuuint64_t shape[3] = {128, per_block, cuuint64_t((rows + 127) / 128)};       // a last partial row block is a whole atom
    const cuuint64_t strides[2] = {128, per_block * 128};
    const cuuint32_t box[3] = {128, cuuint32_t(STAGE_K / atom_k * 4), 1};
    return make_map(CU_TENSOR_MAP_DATA_TYPE_UINT8, p, 3, shape, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}
CUtensorMap output_map(const void* C, int M, int N, bool bf16) {
    const cuuint64_t shape[2] = {cuuint64_t(N), cuuint64_t(M)};
    const cuuint64_t strides[1] = {cuuint64_t(N) * 2};
    const cuuint32_t box[2] = {EPI_COLS, 32};
    return make_map(bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, C, 2, shape, strides, box,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE);
}

int env_int(const char* name, int fallback) {
    const char* v = std::getenv(name);
    return v && *v ? std::atoi(v) : fallback;
}

std::mutex g_host_state;            // guards the per-device caches below

// One kernel instance: sets its shared-memory limit once per device, then launches.
// pdl: launch with the programmatic stream-serialisation attribute, so that the prologue of this launch overlaps
// the tail of the kernel in front of it in the stream (when that kernel allows it, as this kernel does).
template <int CG, int UN, int EPI, bool PROF = false, bool MX = false>
void launch_instance(int device, int units, const CUtensorMap& A, const CUtensorMap& B, const CUtensorMap& SFA,
                     const CUtensorMap& SFB, const CUtensorMap& tmC, const GemmArgs& g, cudaStream_t stream, bool pdl) {
    using Cfg = Config<CG, UN, EPI, MX>;
    auto kernel = nvfp4_gemm_kernel<CG, UN, EPI, PROF, MX>;
    {
        static bool ready[64] = {};
        std::lock_guard<std::mutex> hold(g_host_state);
        if (device < 0 || device >= 64 || !ready[device]) {
            cuda_check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
            if (device >= 0 && device < 64) ready[device] = true;
        }
    }
    cudaLaunchAttribute attrs[2]{};
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim = {unsigned(CG), 1, 1};
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(units) * CG);
    cfg.blockDim = dim3(Cfg::THREADS);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cfg.attrs = attrs;
    cfg.numAttrs = pdl ? 2 : 1;
    cuda_check(cudaLaunchKernelEx(&cfg, kernel, A, B, SFA, SFB, tmC, g));
    g_launches.fetch_add(1, std::memory_order_relaxed);
}

// Units (CTAs, or CTA pairs) of the persistent grid that fit the device at once. Every instance of a
// variant holds one CTA per SM (its ring fills the shared memory), so the count is taken once per variant.
template <int CG, int UN>
int max_units(int device) {
    constexpr int EPI = CG == 2 ? EPI_TMA : EPI_DIRECT;
    using Cfg = Config<CG, UN, EPI>;
    static int cached[64] = {};
    std::lock_guard<std::mutex> hold(g_host_state);
    if (device >= 0 && device < 64 && cached[device]) return cached[device];
    auto kernel = nvfp4_gemm_kernel<CG, UN, EPI, false>;
    cuda_check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    int sms = 0;
    cuda_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    int units = sms;
    if (CG == 2) {
        cudaLaunchAttribute attr{};
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim = {2, 1, 1};
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(unsigned(sms / 2) * 2);
        cfg.blockDim = dim3(Cfg::THREADS);
        cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        cuda_check(cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg));
        units = clusters;
    }
    if (units < 1) throw std::runtime_error("nvfp4 gemm: the kernel does not fit on this device");
    if (device >= 0 && device < 64) cached[device] = units;
    return units;
}

int fit_units(int device, int cta_group, int tile_n) {
    return cta_group == 2 ? max_units<2, 256>(device) : tile_n == 256 ? max_units<1, 256>(device) : max_units<1, 128>(device);
}

uint32_t* status_base(int device) {
    static uint32_t* cached[64] = {};
    std::lock_guard<std::mutex> hold(g_host_state);
    if (device >= 0 && device < 64 && cached[device]) return cached[device];
    uint32_t* p = nullptr;
    cuda_check(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status));
    if (device >= 0 && device < 64) cached[device] = p;
    return p;
}
uint32_t* status_slot(int device, int slot) { return status_base(device) + size_t(slot) * 4; }

std::atomic<unsigned> g_next_slot{0};

// Ragged tiling of a one-tile-row plan over `tiles` single-CTA tiles (see GemmArgs::ragged_base); tiles = 0
// switches it off. Returns whether the plan now uses it: M = 128, single-CTA 256-column variant, the widths
// come out as 2/3 or 3/4 units of 64 columns, and it is more tiles than the uniform tiling has.
bool set_ragged_tiles(gpu_kernels::Nvfp4Params& p, const uint8_t* B, int tiles) {
    p.ragged_base = p.ragged_extra = p.ragged_units = 0;
    if (tiles <= 0 || !B) return false;
    if (p.mx || p.M != 128 || p.cta_group != 1 || p.tile_n != 256 || p.N % 128) return false;
    const int units = p.N / 64, base = units / tiles, extra = units % tiles;
    if ((base != 2 && base != 3) || tiles <= p.N / 256) return false;
    p.B64 = operand_map(B, p.N, p.K, 64);
    p.ragged_base = base;
    p.ragged_extra = extra;
    p.ragged_units = tiles;
    return true;
}

void prepare_format(gpu_kernels::Nvfp4Params& p, const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                    int M, int N, int K, bool mx) {
    require_sm100();
    if (M <= 0 || N <= 0 || K <= 0) throw std::invalid_argument("nvfp4 gemm: M, N, K must be positive");
    if (N % 8) throw std::invalid_argument("nvfp4 gemm: N must be a multiple of 8 (rows of C start on 16-byte boundaries)");
    if (K % (mx ? 128 : 64)) throw std::invalid_argument(mx ? "mxfp4 gemm: K must be a multiple of 128 (whole scale atoms)"
                                                              : "nvfp4 gemm: K must be a multiple of 64 (whole scale atoms)");
    if (!A || !B || !SFA || !SFB) throw std::invalid_argument("nvfp4 gemm: null operand pointer");
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(SFA) |
         reinterpret_cast<uintptr_t>(SFB)) & 15)
        throw std::invalid_argument("nvfp4 gemm: operand pointers must be 16-byte aligned");
    int device = 0;
    cuda_check(cudaGetDevice(&device));
    p = gpu_kernels::Nvfp4Params{};
    p.M = M; p.N = N; p.K = K;
    p.mx = mx ? 1 : 0;
    p.alpha = 1.0f;
    p.device = device;
    p.c_evict_first = env_int("NVFP4_B200_C_EVICT_FIRST", 1);

    const int force = env_int("NVFP4_B200_VARIANT", 0);        // 0 auto, 2256 / 1256 / 1128 for experiments
    // M and N need not be whole tiles: the scale arrays end in whole 128-row atoms whatever the row count (rows
    // the tensor does not have read as zeros through the tensor maps), and the variant is chosen for the sizes
    // rounded up to 128.
    const int Mp = (M + 127) / 128 * 128, Np = (N + 127) / 128 * 128;
    if ((force == 0 && Mp % 256 == 0 && Np % 256 == 0) || force == 2256) { p.cta_group = 2; p.tile_n = 256; }
    else if ((force == 0 && Np % 256 == 0) || force == 1256) { p.cta_group = 1; p.tile_n = 256; }
    else { p.cta_group = 1; p.tile_n = 128; }
    if (Mp % (128 * p.cta_group) || Np % p.tile_n) throw std::invalid_argument("nvfp4 gemm: forced variant does not divide the shape");
    // Epilogue route. C leaves from registers (32-byte stores, two epilogue warps per Tensor Memory lane
    // quarter) unless the caller asks for the staged route (rows through swizzled shared memory, TMA stores):
    // measured by graph replay under sustained load, registers / staged: 8192^3 222.0 / 227.2 us, 16384^3
    // 1717 / 1753 us, 8192x4096x2048 36.3 / 38.6 us. Single-CTA tiles have no staged route.
    p.direct_store = p.cta_group == 1 ? 1 : env_int("NVFP4_B200_DIRECT_STORE", 1);
    const int box_b = p.tile_n / p.cta_group;
    p.A = operand_map(A, M, K, BLOCK_M);
    p.B = operand_map(B, N, K, box_b);
    p.SFA = scale_map(SFA, M, K, mx ? 128 : 64);
    p.SFB = scale_map(SFB, N, K, mx ? 128 : 64);
    const int tiles = (Mp / (128 * p.cta_group)) * (Np / p.tile_n);
    p.clusters = std::min(fit_units(device, p.cta_group, p.tile_n), tiles);
    // About sqrt(units) tile rows per band keeps the A and B panels of the tiles in flight balanced.
    int gm = 1;
    while ((gm + 1) * (gm + 1) <= p.clusters) ++gm;
    // Measured at 16384^3 (64 x 64 tiles, operands beyond L2): bands of 16 beat 8 by 1.3 %, 32 and 4 lose 10 %;
    // at 8192^3 (everything L2-resident) the band height does not matter.
    if (Mp / (128 * p.cta_group) >= 48) gm = std::max(gm, 16);
    p.group_m = std::max(1, std::min(env_int("NVFP4_B200_GROUP_M", gm), Mp / (128 * p.cta_group)));
    // Measured: 128x28672x8192 30.2 -> 28.9 us, 8192^3 199.8 -> 199.0 us with the tiles' K walks de-phased.
    p.k_skew = env_int("NVFP4_B200_K_SKEW", 11);
    // One tile row whose 256-column tiles would leave SMs idle can deal its columns, in units of 64, to as many
    // tiles as there are SMs (128x28672x8192: 112 tiles of 256 columns become 4 of 256 and 144 of 192): plan
    // option "ragged_tiles". Off unless asked for: measured 27.9 against 28.3 us for dependent launches, but a
    // launch that fills every SM leaves no room for the next launch of a chain to start early (independent
    // launches: 28.5 against 24.7-26.1 us).
    if (!mx && env_int("NVFP4_B200_RAGGED", 0)) set_ragged_tiles(p, B, fit_units(device, 1, 256));
    p.pdl = env_int("NVFP4_B200_PDL", 1);
    p.status_slot = 1 + int(g_next_slot.fetch_add(1, std::memory_order_relaxed) % unsigned(STATUS_SLOTS - 1));
    (void)status_base(device);
}

void prepare(gpu_kernels::Nvfp4Params& p, const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
             int M, int N, int K, cudaStream_t) {
    prepare_format(p, A, B, SFA, SFB, M, N, K, false);
}

// table: device memory of gather_table_bytes(world), filled here (on `stream`) with one tensor map and one
// base pointer per destination; buffers: host array of `world` device pointers to the full [M, n_total] C.
size_t gather_table_bytes(int world) { return size_t(world) * (sizeof(CUtensorMap) + sizeof(void*)); }

void set_gather(gpu_kernels::Nvfp4Params& p, void* const* buffers, int world, int col0, int n_total, void* table,
                cudaStream_t stream) {
    if (world == 0) { p.gather_world = 0; p.gather_maps = nullptr; p.gather_ptrs = nullptr; return; }
    if (!buffers || !table || world < 1 || world > 64) throw std::invalid_argument("nvfp4 gemm gather: 1..64 destination buffers and a table");
    if (p.M % 128 || p.N % 128) throw std::invalid_argument("nvfp4 gemm gather: M and the slab width must be multiples of 128");
    if (col0 < 0 || col0 % 64 || n_total % 8 || col0 + p.N > n_total)
        throw std::invalid_argument("nvfp4 gemm gather: the slab [col0, col0 + N) must lie inside the full C, col0 a multiple of 64");
    if (reinterpret_cast<uintptr_t>(table) & 127) throw std::invalid_argument("nvfp4 gemm gather: table must be 128-byte aligned");
    std::vector<uint8_t> host(gather_table_bytes(world));
    auto* maps = reinterpret_cast<CUtensorMap*>(host.data());
    auto* ptrs = reinterpret_cast<void**>(host.data() + size_t(world) * sizeof(CUtensorMap));
    for (int r = 0; r < world; ++r) {
        if (!buffers[r] || (reinterpret_cast<uintptr_t>(buffers[r]) & 15)) throw std::invalid_argument("nvfp4 gemm gather: null or misaligned buffer");
        maps[r] = output_map(buffers[r], p.M, n_total, p.out_bf16 != 0);
        ptrs[r] = buffers[r];
    }
    cuda_check(cudaMemcpyAsync(table, host.data(), host.size(), cudaMemcpyHostToDevice, stream));
    cuda_check(cudaStreamSynchronize(stream));           // `host` goes out of scope
    p.gather_world = world;
    p.gather_col0 = col0;
    p.gather_ldc = n_total;
    p.gather_maps = table;
    p.gather_ptrs = static_cast<uint8_t*>(table) + size_t(world) * sizeof(CUtensorMap);
}

// Split-K can pay when whole tiles would leave most SMs idle and every tile's K loop is long: four units per
// tile, each with a quarter of the K steps, as long as all tiles * 4 units are resident at once and a slice
// keeps at least four ring steps. Measured (us, split / whole): 128x3584x8192 18.2 / 20.9, 256x256x8192
// 14.6 / 16.3, 128x7168x8192 20.9 / 21.2; two slices per tile lost everywhere (128x14336x8192 26.5 / 22.5,
// 1024x2048x4096 18.1 / 12.9): publishing, waiting for the slowest slice and re-reading the partial sums cost
// about 17k cycles, which is what a quarter of a 32-step K loop saves.
int split_k_factor(const gpu_kernels::Nvfp4Params& p) {
    if (p.M % 128 || p.N % 128) return 0;
    const int tiles = (p.M / (128 * p.cta_group)) * (p.N / p.tile_n);
    const int fit = fit_units(p.device, p.cta_group, p.tile_n);
    const int ksteps = (p.K + STAGE_K - 1) / STAGE_K, chunks = p.tile_n / EPI_COLS;
    for (int s : {4})
        if (!p.mx && p.K % STAGE_K == 0 && s <= chunks && tiles * s <= fit && ksteps % s == 0 && ksteps / s >= 4 &&
            size_t(tiles) * s * p.cta_group * 4 * sizeof(uint32_t) <= SPLIT_K_FLAG_BYTES / 2)
            return s;
    return 0;
}

size_t split_k_workspace_bytes(const gpu_kernels::Nvfp4Params& p) {
    const int s = split_k_factor(p);
    if (!s) return 0;
    const size_t tiles = size_t(p.M / (128 * p.cta_group)) * (p.N / p.tile_n);
    return SPLIT_K_FLAG_BYTES + tiles * s * p.cta_group * 128 * p.tile_n * sizeof(float);
}

void enable_split_k(gpu_kernels::Nvfp4Params& p, void* workspace, size_t bytes, cudaStream_t stream) {
    const int s = split_k_factor(p);
    if (!s) throw std::invalid_argument("nvfp4 gemm: split-K does not apply to this shape");
    if (!workspace || bytes < split_k_workspace_bytes(p) || (reinterpret_cast<uintptr_t>(workspace) & 255))
        throw std::invalid_argument("nvfp4 gemm: split-K workspace missing, too small or not 256-byte aligned");
    // the flags must be zero before the first launch, whatever stream that launch uses
    cuda_check(cudaMemsetAsync(workspace, 0, SPLIT_K_FLAG_BYTES, stream));
    cuda_check(cudaStreamSynchronize(stream));
    p.split_k = s;
    p.split_k_workspace = workspace;
    p.direct_store = 1;
    p.route = nullptr;                                                   // slices are dealt in item order
    p.clusters = (p.M / (128 * p.cta_group)) * (p.N / p.tile_n) * s;     // one (tile, slice) per unit
}

GemmArgs dense_args(const gpu_kernels::Nvfp4Params& p, void* c, unsigned long long* prof) {
    const int tile_m = 128 * p.cta_group;
    GemmArgs g{};
    g.M = p.M; g.N = p.N; g.K = p.K;
    g.ksteps = (p.K + STAGE_K - 1) / STAGE_K;
    g.tiles_m = (p.M + tile_m - 1) / tile_m;
    g.tiles_n = (p.N + p.tile_n - 1) / p.tile_n;
    g.group_m = std::max(1, p.group_m);
    g.alpha = p.alpha;
    g.status = status_slot(p.device, p.status_slot);
    g.cycles = status_slot(p.device, 0) + 2;
    g.prof = prof;
    g.c_evict_first = p.c_evict_first;
    g.out_bf16 = p.out_bf16;
    g.c = c;
    g.ldc = p.N;
    g.k_skew = p.k_skew;
    g.split_k = p.split_k;
    if (p.split_k > 1) {
        auto* ws = static_cast<uint8_t*>(p.split_k_workspace);
        g.sk_flags = reinterpret_cast<uint32_t*>(ws);
        g.sk_done = reinterpret_cast<uint32_t*>(ws) + SPLIT_K_FLAG_BYTES / 8;
        g.sk_partials = reinterpret_cast<float*>(ws + SPLIT_K_FLAG_BYTES);
    }
    g.gather_world = p.gather_world;
    g.gather_col0 = p.gather_col0;
    g.gather_ldc = p.gather_ldc;
    g.gather_maps = static_cast<const CUtensorMap*>(p.gather_maps);
    g.gather_ptrs = static_cast<void* const*>(p.gather_ptrs);
    // split-K launches of one plan share flags and partial sums: they never overlap; profiled launches neither
    g.static_operands = (p.split_k > 1 || prof) ? 0 : p.static_operands;
    if (p.route && p.split_k <= 1) {
        g.route = static_cast<const uint32_t*>(p.route);
        g.sm_side = static_cast<const uint8_t*>(p.sm_side);
        g.unit_side = static_cast<const uint8_t*>(p.unit_side);
    }
    return g;
}

template <int CG, int UN>
void launch_dense(const gpu_kernels::Nvfp4Params& p, const CUtensorMap& tmC, const GemmArgs& g, cudaStream_t stream) {
    const bool staged = CG == 2 && !p.direct_store;
    const bool pdl = p.pdl != 0 && !g.prof;
    const int dev = p.device, units = p.clusters;
    if (p.mx) {
        // MXFP4 plans have the masked register-store route only
        if (p.split_k > 1 || p.gather_world || g.prof) throw std::invalid_argument("mxfp4 gemm: plain launches only");
        launch_instance<CG, UN, EPI_DIRECT_EDGE, false, true>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
    } else if (p.M % 128 || p.N % 128) {
        if (p.split_k > 1 || p.gather_world || g.prof) throw std::invalid_argument("nvfp4 gemm: M or N is no multiple of 128: plain launches only");
        launch_instance<CG, UN, EPI_DIRECT_EDGE>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
    } else if (p.split_k > 1) {
        launch_instance<CG, UN, EPI_SPLIT_K>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
    } else if (p.gather_world) {
        // CTA pairs send the slab with TMA stores of staged 32 x 64 chunks (one per destination): NVLink carries
        // those far better than 32-byte register stores (8192^3 on two GPUs: 141 against 264 us per step).
        if constexpr (CG == 2) return launch_instance<CG, UN, EPI_GATHER_TMA>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
        launch_instance<CG, UN, EPI_GATHER_DIRECT>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
    } else if (CG == 1 && UN == 256 && p.ragged_units > 0 && !g.prof) {
        if constexpr (CG == 1 && UN == 256) {
            GemmArgs r = g;
            r.tiles_m = 1;
            r.tiles_n = p.ragged_units;
            r.ragged_base = p.ragged_base;
            r.ragged_extra = p.ragged_extra;
            launch_instance<1, 256, EPI_DIRECT_RAGGED>(dev, p.ragged_units, p.A, p.B64, p.SFA, p.SFB, tmC, r, stream, pdl);
        }
    } else if (g.prof) {
        if constexpr (CG == 2) {
            if (staged) return launch_instance<CG, UN, EPI_TMA, true>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
        }
        launch_instance<CG, UN, EPI_DIRECT, true>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
    } else {
        if constexpr (CG == 2) {
            if (staged) return launch_instance<CG, UN, EPI_TMA>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
        }
        launch_instance<CG, UN, EPI_DIRECT>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
    }
}

void launch_with(const gpu_kernels::Nvfp4Params& p, void* C, cudaStream_t stream, unsigned long long* prof) {
    if (!C || (reinterpret_cast<uintptr_t>(C) & 15)) throw std::invalid_argument("nvfp4 gemm: C must be 16-byte aligned");
    if (prof && (p.split_k > 1 || p.gather_world)) throw std::invalid_argument("nvfp4 gemm profile: plain plans only");
    const CUtensorMap tmC = output_map(C, p.M, p.N, p.out_bf16 != 0);
    const GemmArgs g = dense_args(p, C, prof);
    if (p.cta_group == 2) launch_dense<2, 256>(p, tmC, g, stream);
    else if (p.tile_n == 256) launch_dense<1, 256>(p, tmC, g, stream);
    else launch_dense<1, 128>(p, tmC, g, stream);
}

void launch(const gpu_kernels::Nvfp4Params& p, __half* C, cudaStream_t stream) { launch_with(p, C, stream, nullptr); }

[[noreturn]] void throw_status(const uint32_t* words) {
    char msg[256];
    std::snprintf(msg, sizeof(msg), "nvfp4 gemm: the kernel reported an error (status 0x%x: 0x10 = bad destination, else a wait gave up; first tag 0x%08x); output is invalid",
                  words[0], words[1]);
    throw std::runtime_error(msg);
}

// Every slot of the current device: any plan's error is reported (and all are cleared).
void validate() {
    cuda_check(cudaDeviceSynchronize());
    static thread_local std::vector<uint32_t> host;
    host.resize(size_t(STATUS_SLOTS) * 4);
    cuda_check(cudaMemcpyFromSymbol(host.data(), g_status, host.size() * sizeof(uint32_t)));
    for (int s = 0; s < STATUS_SLOTS; ++s) {
        if (!host[size_t(s) * 4]) continue;
        const uint32_t words[2] = {host[size_t(s) * 4], host[size_t(s) * 4 + 1]};
        for (int t = 0; t < STATUS_SLOTS; ++t)
            if (host[size_t(t) * 4]) {
                const uint32_t zero[2] = {0u, 0u};
                cuda_check(cudaMemcpyToSymbol(g_status, zero, sizeof(zero), size_t(t) * 16));
            }
        throw_status(words);
    }
}

void validate_slot(int device, int slot) {
    cuda_check(cudaDeviceSynchronize());
    uint32_t host[4] = {};
    uint32_t* where = status_slot(device, slot);
    cuda_check(cudaMemcpy(host, where, sizeof(host), cudaMemcpyDeviceToHost));
    if (host[0]) {
        const uint32_t zero[2] = {0u, 0u};
        cuda_check(cudaMemcpy(where, zero, sizeof(zero), cudaMemcpyHostToDevice));
        throw_status(host);
    }
}

}  // namespace

uint32_t* device_status_word(int device) { return status_slot(device, 0); }

void require_sm100() {
    int device = 0, major = 0;
    cuda_check(cudaGetDevice(&device));
    cuda_check(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) throw std::runtime_error("this library only runs on compute capability 10.x (B200); there is no fallback");
}

// Plain launch through a pointer that may be FP16 or BF16 storage (the plan's out_bf16 decides).
void gemm_launch(const gpu_kernels::Nvfp4Params& p, void* C, cudaStream_t stream) { launch_with(p, C, stream, nullptr); }

// The device-wide slot (grouped launches and the expert-path kernels report there).
void validate_device_slot(int device) { validate_slot(device, 0); }

// One launch with the per-role cycle counters switched on; copies 16 words per CTA to `host`
// (synchronises). Diagnostic: the counters cost a few clock reads per wait.
int gemm_profile(const gpu_kernels::Nvfp4Params& p, __half* C, cudaStream_t stream, unsigned long long* host, int max_words) {
    const int words = p.clusters * p.cta_group * PROF_WORDS + TR_TILES * 8;
    if (words > max_words) throw std::invalid_argument("nvfp4 gemm profile: output buffer too small");
    unsigned long long* dev = nullptr;
    cuda_check(cudaMalloc(&dev, size_t(words) * 8));
    cudaError_t e = cudaMemsetAsync(dev, 0, size_t(words) * 8, stream);
    try {
        cuda_check(e);
        launch_with(p, C, stream, dev);
    } catch (...) {
        cudaFree(dev);
        throw;
    }
    e = cudaMemcpyAsync(host, dev, size_t(words) * 8, cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    cudaFree(dev);
    cuda_check(e);
    return words;
}

// SM cycles the first CTA of the last finished GEMM launch on the current device spent in the kernel.
unsigned last_kernel_cycles() {
    int device = 0;
    cuda_check(cudaGetDevice(&device));
    uint32_t cycles = 0;
    cuda_check(cudaMemcpy(&cycles, status_slot(device, 0) + 2, sizeof(cycles), cudaMemcpyDeviceToHost));
    return cycles;
}

void grouped_prepare(GroupedGemm& p, const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB,
                     int pool_rows, int n, int k, int experts, int block_rows, const int* block_expert,
                     const int* num_blocks) {
    p.block_valid = nullptr;
    require_sm100();
    if (block_rows != 128 && block_rows != 256) throw std::invalid_argument("grouped gemm: block rows must be 128 or 256");
    if (pool_rows <= 0 || pool_rows % block_rows) throw std::invalid_argument("grouped gemm: pool rows must be a positive multiple of the block rows");
    if (n <= 0 || n % 256) throw std::invalid_argument("grouped gemm: N per expert must be a multiple of 256");
    if (k <= 0 || k % 64) throw std::invalid_argument("grouped gemm: K must be a multiple of 64");
    if (experts <= 0 || !A || !B || !SFA || !SFB || !block_expert || !num_blocks)
        throw std::invalid_argument("grouped gemm: null pointer or no experts");
    cuda_check(cudaGetDevice(&p.device));
    p.pool_rows = pool_rows; p.n = n; p.k = k; p.experts = experts; p.tile_n = 256; p.block_rows = block_rows;
    p.block_expert = block_expert; p.num_blocks = num_blocks;
    // 256-row blocks run on CTA pairs (each CTA stages half of the expert's weight tile: half the L2 traffic
    // per FLOP, which is what bounds the single-CTA tiles once an expert has many rows)
    p.A = operand_map(A, pool_rows, k, BLOCK_M);
    p.B = operand_map(B, experts * n, k, block_rows == 256 ? 128 : 256);
    p.SFA = scale_map(SFA, pool_rows, k);
    p.SFB = scale_map(SFB, experts * n, k);
    const int fit = block_rows == 256 ? max_units<2, 256>(p.device) : max_units<1, 256>(p.device);
    p.units = std::min(fit, (pool_rows / block_rows) * (n / 256));
    (void)status_base(p.device);
}

void grouped_launch(const GroupedGemm& p, void* C, int out_bf16, cudaStream_t stream) {
    grouped_launch_fused(p, C, out_bf16, nullptr, nullptr, nullptr, 0.0f, nullptr, nullptr, 0, 0, stream);
}

void grouped_launch_fused(const GroupedGemm& p, void* C, int out_bf16, uint8_t* act_packed, uint8_t* act_scales,
                          const float* row_weight, float clamp, const int* row_dst, void* const* slots, int world,
                          int slot_rows, cudaStream_t stream) {
    const bool fused = act_packed != nullptr;
    if (row_dst) {
        // a destination code is (rank << 24) | (row + 1) in 32 bits
        if (fused || !slots || !C || world < 1 || world > 127 || slot_rows <= 0 || slot_rows >= (1 << 24))
            throw std::invalid_argument("grouped gemm: scatter needs a table of 1..127 slot buffers of fewer than 2^24 rows and "
                                        "this rank's own buffer, and cannot be combined with the fused activation");
    }
    if (fused && (!act_scales || !row_weight)) throw std::invalid_argument("grouped gemm: fused SwiGLU needs scales and row weights");
    if (!fused && (!C || (reinterpret_cast<uintptr_t>(C) & 15))) throw std::invalid_argument("grouped gemm: C must be 16-byte aligned");
    if (fused) C = act_packed;       // only the tensor map needs a valid address; the fused route never stores C
    const CUtensorMap tmC = output_map(C, p.pool_rows, p.n, out_bf16 != 0);
    GemmArgs g{};
    g.M = p.pool_rows; g.N = p.n; g.K = p.k;
    g.ksteps = (p.k + STAGE_K - 1) / STAGE_K;
    g.tiles_m = p.pool_rows / p.block_rows;
    g.tiles_n = p.n / 256;
    g.group_m = 1;
    g.alpha = 1.0f;
    g.status = status_slot(p.device, 0);
    g.cycles = status_slot(p.device, 0) + 2;
    g.c_evict_first = 1;
    g.out_bf16 = out_bf16;
    g.block_expert = p.block_expert;
    g.num_blocks = p.num_blocks;
    g.block_valid = p.block_valid;
    g.b_rows_per_expert = p.n;
    g.c = C;
    g.ldc = p.n;
    g.act_packed = act_packed;
    g.act_scales = act_scales;
    g.row_weight = row_weight;
    g.swiglu_clamp = clamp;
    g.row_dst = row_dst;
    g.slots = slots;
    g.world = world;
    g.slot_rows = slot_rows;
    const int dev = p.device, units = p.units;
    const bool pdl = env_int("NVFP4_B200_PDL", 1) != 0;
    if (p.block_rows == 256) {
        if (fused) launch_instance<2, 256, EPI_ACT>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
        else if (row_dst) launch_instance<2, 256, EPI_SCATTER_ROWS>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
        else if (p.block_valid) launch_instance<2, 256, EPI_DIRECT_EDGE>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
        else launch_instance<2, 256, EPI_DIRECT>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
    } else {
        if (fused) launch_instance<1, 256, EPI_ACT>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
        else if (row_dst) launch_instance<1, 256, EPI_SCATTER>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
        else if (p.block_valid) launch_instance<1, 256, EPI_DIRECT_EDGE>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
        else launch_instance<1, 256, EPI_DIRECT>(dev, units, p.A, p.B, p.SFA, p.SFB, tmC, g, stream, pdl);
    }
}

int gemm_stage_count(int cta_group, int tile_n, int direct_store) {
    if (cta_group == 2) return direct_store ? Config<2, 256, EPI_DIRECT>::STAGES : Config<2, 256, EPI_TMA>::STAGES;
    return tile_n == 256 ? Config<1, 256, EPI_DIRECT>::STAGES : Config<1, 128, EPI_DIRECT>::STAGES;
}

size_t gemm_smem_bytes(int cta_group, int tile_n) {
    if (cta_group == 2) return Config<2, 256, EPI_TMA>::SMEM_BYTES;
    return tile_n == 256 ? Config<1, 256, EPI_DIRECT>::SMEM_BYTES : Config<1, 128, EPI_DIRECT>::SMEM_BYTES;
}

}  // namespace nvfp4_b200

namespace gpu_kernels {

Nvfp4Implementation nvfp4_sm100_implementation() {
    return {nvfp4_b200::prepare, nvfp4_b200::launch, nvfp4_b200::validate};
}

void nvfp4_set_alpha(Nvfp4Params& p, float alpha) { p.alpha = alpha; }

void mxfp4_prepare(Nvfp4Params& p, const uint8_t* A, const uint8_t* B, const uint8_t* SFA, const uint8_t* SFB, int M, int N,
                   int K, cudaStream_t) {
    nvfp4_b200::prepare_format(p, A, B, SFA, SFB, M, N, K, true);
}

void nvfp4_validate_plan(const Nvfp4Params& p) { nvfp4_b200::validate_slot(p.device, p.status_slot); }

size_t nvfp4_split_k_workspace_bytes(const Nvfp4Params& p) { return nvfp4_b200::split_k_workspace_bytes(p); }

void nvfp4_enable_split_k(Nvfp4Params& p, void* workspace, size_t bytes, cudaStream_t stream) {
    nvfp4_b200::enable_split_k(p, workspace, bytes, stream);
}

size_t nvfp4_gather_table_bytes(int world) { return nvfp4_b200::gather_table_bytes(world); }

void nvfp4_set_gather(Nvfp4Params& p, void* const* buffers, int world, int col0, int n_total, void* table,
                      cudaStream_t stream) {
    nvfp4_b200::set_gather(p, buffers, world, col0, n_total, table, stream);
}

bool nvfp4_set_ragged_tiles(Nvfp4Params& p, const uint8_t* B, int tiles) { return nvfp4_b200::set_ragged_tiles(p, B, tiles); }

bool nvfp4_set_l2_side_order(Nvfp4Params& p, int on, cudaStream_t stream) {
    p.route = p.sm_side = p.unit_side = nullptr;
    p.side_units[0] = p.side_units[1] = 0;
    if (!on || p.split_k > 1) return false;
    nvfp4_b200::TileRoute r{};
    const int tile_m = 128 * p.cta_group;
    const int tiles_m = (p.M + tile_m - 1) / tile_m, tiles_n = (p.N + p.tile_n - 1) / p.tile_n;
    if (!nvfp4_b200::l2_side_route(p.device, p.cta_group, p.clusters, tiles_m, tiles_n, p.group_m,
                                   nvfp4_b200::gemm_smem_bytes(p.cta_group, p.tile_n), stream, r))
        return false;
    p.route = r.route; p.sm_side = r.sm_side; p.unit_side = r.unit_side;
    p.side_units[0] = r.side_units[0]; p.side_units[1] = r.side_units[1];
    return true;
}

unsigned nvfp4_placement_misses(const Nvfp4Params& p) {
    uint32_t misses = 0;
    nvfp4_b200::cuda_check(cudaMemcpy(&misses, nvfp4_b200::device_status_word(p.device) + size_t(p.status_slot) * 4 + 3,
                                      sizeof(misses), cudaMemcpyDeviceToHost));
    return misses;
}

}  // namespace gpu_kernels
