// L2-side-aware tile order for the persistent NVFP4 GEMM.
//
// B200's L2 is built from two halves; an SM reaches lines that live in the far half more slowly, and what
// the clusters of one half read is cached in that half. When the clusters of each half work through their
// own contiguous part of the tile sequence, the A and B panels they share stay on their side instead of
// being pulled into both. The reference does this in kernels/gemm/matmul/sm100.cu:545-673 (latency_census,
// cluster_census, prepare_schedule) with one global schedule in __constant__ memory; here the tables are
// per (device, shape) in global memory, several shapes can be live at once, and every wait has a limit.
//
// Steps, all at plan time:
//   1. side census (once per device): one single-thread CTA per SM times a chain of dependent atomic adds
//      on one cache line. The CTAs take turns (so that they do not disturb each other's timing); a CTA
//      whose turn does not come within a time limit goes ahead anyway and flags the census as unusable.
//   2. placement census (per grid shape): a kernel with the GEMM's launch geometry (cluster size, threads,
//      dynamic shared memory) records the SM of every CTA, which gives each unit's side.
//   3. the tile sequence (band order) is cut in two at the share of work of side 0; the units of each side
//      are dealt the tiles of their part in turn.
// The kernel checks at run time that a unit sits on the side the table assumed and counts the misses; a miss
// costs locality, never correctness (the route is a permutation of the tiles whatever the sides are).
#include "nvfp4_internal.h"

#include <algorithm>
#include <map>
#include <mutex>
#include <numeric>
#include <tuple>
#include <vector>

namespace nvfp4_b200 {
namespace {

constexpr unsigned long long CENSUS_TURN_LIMIT_NS = 200000000ull;      // 0.2 s: far beyond the ~10 ms a census takes
constexpr int CENSUS_WARM = 8, CENSUS_TIMED = 64;
constexpr int MAX_SMS = 256;

__global__ void side_census_kernel(unsigned* probe, unsigned* turn, unsigned* cycles_per_op, unsigned* smids,
                                   unsigned* flags) {
    extern __shared__ char pad[];                  // large on purpose: one CTA per SM
    if (threadIdx.x != 0) return;
    pad[0] = 0;
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    while (true) {
        unsigned now_turn;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(now_turn) : "l"(turn) : "memory");
        if (now_turn >= blockIdx.x) break;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        if (t - t0 > CENSUS_TURN_LIMIT_NS) { atomicOr(flags, 1u); break; }
        __nanosleep(200);
    }
    unsigned value = 0;
    for (int i = 0; i < CENSUS_WARM; ++i) value = atomicAdd(probe + (value >> 31), 1u);
    const long long c0 = clock64();
    for (int i = 0; i < CENSUS_TIMED; ++i) value = atomicAdd(probe + (value >> 31), 1u);
    const long long c1 = clock64();
    unsigned sm;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    cycles_per_op[blockIdx.x] = unsigned((c1 - c0) / CENSUS_TIMED) + (value >> 31);
    smids[blockIdx.x] = sm;
    __threadfence();
    atomicMax(turn, blockIdx.x + 1u);
}

__global__ void placement_census_kernel(unsigned* smids) {
    extern __shared__ char pad[];
    if (threadIdx.x == 0) {
        pad[0] = 0;
        unsigned sm;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
        smids[blockIdx.x] = sm;
    }
}

struct DeviceSides {
    bool tried = false, usable = false;
    std::vector<uint8_t> side;                     // by SM id
    uint8_t* device_side = nullptr;                // [MAX_SMS]
    std::vector<unsigned> cycles;                  // by SM id (diagnostic)
};

struct RouteEntry {
    bool usable = false;
    uint32_t* route = nullptr;
    uint8_t* unit_side = nullptr;
    int side_units[2] = {0, 0};
};

std::mutex g_lock;
std::map<int, DeviceSides> g_sides;
std::map<std::tuple<int, int, int, int, int, int>, RouteEntry> g_routes;

// Step 1. Returns the cached labels of `device` (usable = false when the SMs did not fall into two groups).
DeviceSides& census(int device, cudaStream_t stream) {
    DeviceSides& d = g_sides[device];
    if (d.tried) return d;
    d.tried = true;
    int sms = 0;
    cuda_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    if (sms < 4 || sms > MAX_SMS) return d;
    unsigned* scratch = nullptr;
    // words: [0] probe line, [32] turn, [64] flags, [96, 96 + sms) cycles, then sms SM ids
    const size_t words = 96 + 2 * size_t(sms);
    cuda_check(cudaMalloc(&scratch, words * sizeof(unsigned)));
    std::vector<unsigned> host(words);
    try {
        cuda_check(cudaMemsetAsync(scratch, 0, words * sizeof(unsigned), stream));
        constexpr int fat_smem = 120 * 1024;
        cuda_check(cudaFuncSetAttribute(side_census_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fat_smem));
        side_census_kernel<<<sms, 32, fat_smem, stream>>>(scratch, scratch + 32, scratch + 96, scratch + 96 + sms, scratch + 64);
        cuda_check(cudaGetLastError());
        cuda_check(cudaMemcpyAsync(host.data(), scratch, words * sizeof(unsigned), cudaMemcpyDeviceToHost, stream));
        cuda_check(cudaStreamSynchronize(stream));
    } catch (...) {
        cudaFree(scratch);
        throw;
    }
    cudaFree(scratch);
    if (host[64]) return d;                                        // a turn did not come: timings are not clean
    const unsigned* cyc = host.data() + 96;
    const unsigned* ids = host.data() + 96 + sms;
    std::vector<unsigned> by_sm(MAX_SMS, 0);
    std::vector<char> seen(MAX_SMS, 0);
    for (int i = 0; i < sms; ++i) {
        if (ids[i] >= unsigned(MAX_SMS) || seen[ids[i]]) return d; // two CTAs shared an SM: not one per SM
        seen[ids[i]] = 1;
        by_sm[ids[i]] = cyc[i];
    }
    std::vector<unsigned> sorted(cyc, cyc + sms);
    std::sort(sorted.begin(), sorted.end());
    // the widest gap in the middle half of the sorted latencies separates near from far
    int cut = sms / 2 - 1;
    for (int i = sms / 4; i < 3 * sms / 4; ++i)
        if (sorted[i + 1] - sorted[i] > sorted[cut + 1] - sorted[cut]) cut = i;
    const unsigned gap = sorted[cut + 1] - sorted[cut], median = sorted[sms / 2];
    d.cycles = by_sm;
    if (gap * 50 < median) return d;                               // less than 2 % apart: one group
    const unsigned threshold = (sorted[cut] + sorted[cut + 1]) / 2;
    d.side.assign(MAX_SMS, 0);
    for (int s = 0; s < MAX_SMS; ++s) d.side[s] = seen[s] && by_sm[s] > threshold ? 1 : 0;
    cuda_check(cudaMalloc(&d.device_side, MAX_SMS));
    cuda_check(cudaMemcpy(d.device_side, d.side.data(), MAX_SMS, cudaMemcpyHostToDevice));
    d.usable = true;
    return d;
}

}  // namespace

// The work of `units` persistent units over `tiles` items dealt by side. Item w (= unit + trip * units) of the
// kernel's walk becomes tile route[w]. sides[u] in {0, 1}. Pure host arithmetic (tested on the CPU).
std::vector<uint32_t> build_side_route(const std::vector<uint8_t>& sides, int tiles) {
    const int units = int(sides.size());
    std::vector<uint32_t> route(size_t(tiles), 0);
    auto trips = [&](int u) { return u < tiles ? (tiles - 1 - u) / units + 1 : 0; };
    std::vector<int> members[2];
    int work[2] = {0, 0};
    for (int u = 0; u < units; ++u) {
        members[sides[u] ? 1 : 0].push_back(u);
        work[sides[u] ? 1 : 0] += trips(u);
    }
    int first = 0;                                                  // first tile of the side's part of the sequence
    for (int s = 0; s < 2; ++s) {
        auto& m = members[s];
        // units with one more trip go first, so that every trip is a dense run of the part
        std::stable_sort(m.begin(), m.end(), [&](int a, int b) { return trips(a) > trips(b); });
        int at = first;
        const int max_trips = m.empty() ? 0 : trips(m.front());
        for (int trip = 0; trip < max_trips; ++trip)
            for (int u : m)
                if (trip < trips(u)) route[size_t(u) + size_t(trip) * units] = uint32_t(at++);
        first += work[s];
    }
    return route;
}

bool l2_side_route(int device, int cta_group, int units, int tiles_m, int tiles_n, int group_m, size_t smem_bytes,
                   cudaStream_t stream, TileRoute& out) {
    std::lock_guard<std::mutex> hold(g_lock);
    int sms = 0;
    cuda_check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    const int tiles = tiles_m * tiles_n;
    // ownership needs the whole GPU: a grid that leaves SMs free can land anywhere
    if (units * cta_group < sms - sms % cta_group || tiles < 2 * units) return false;
    DeviceSides& d = census(device, stream);
    if (!d.usable) return false;
    const auto key = std::make_tuple(device, cta_group, units, tiles_m, tiles_n, group_m);
    auto found = g_routes.find(key);
    if (found == g_routes.end()) {
        RouteEntry e;
        // Step 2: where does each CTA of a grid of this geometry land?
        const int ctas = units * cta_group;
        unsigned* dev_ids = nullptr;
        cuda_check(cudaMalloc(&dev_ids, size_t(ctas) * sizeof(unsigned)));
        std::vector<unsigned> ids(size_t(ctas), 0);
        try {
            cuda_check(cudaFuncSetAttribute(placement_census_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes)));
            cudaLaunchAttribute attr{};
            attr.id = cudaLaunchAttributeClusterDimension;
            attr.val.clusterDim = {unsigned(cta_group), 1, 1};
            cudaLaunchConfig_t cfg{};
            cfg.gridDim = dim3(unsigned(ctas));
            cfg.blockDim = dim3(192);
            cfg.dynamicSmemBytes = smem_bytes;
            cfg.stream = stream;
            cfg.attrs = &attr;
            cfg.numAttrs = 1;
            cuda_check(cudaStreamSynchronize(stream));              // an idle device, as at the start of a GEMM launch
            cuda_check(cudaLaunchKernelEx(&cfg, placement_census_kernel, dev_ids));
            cuda_check(cudaMemcpyAsync(ids.data(), dev_ids, ids.size() * sizeof(unsigned), cudaMemcpyDeviceToHost, stream));
            cuda_check(cudaStreamSynchronize(stream));
        } catch (...) {
            cudaFree(dev_ids);
            throw;
        }
        cudaFree(dev_ids);
        std::vector<uint8_t> sides(size_t(units), 0);
        bool whole = true;
        for (int u = 0; u < units && whole; ++u) {
            const unsigned a = ids[size_t(u) * cta_group];
            if (a >= unsigned(MAX_SMS)) { whole = false; break; }
            sides[u] = d.side[a];
            for (int r = 1; r < cta_group; ++r) {
                const unsigned b = ids[size_t(u) * cta_group + r];
                if (b >= unsigned(MAX_SMS) || d.side[b] != sides[u]) whole = false;      // a cluster astride both sides
            }
            e.side_units[sides[u]]++;
        }
        if (whole && e.side_units[0] > 0 && e.side_units[1] > 0) {
            const std::vector<uint32_t> route = build_side_route(sides, tiles);
            cuda_check(cudaMalloc(&e.route, route.size() * sizeof(uint32_t)));
            cuda_check(cudaMalloc(&e.unit_side, sides.size()));
            cuda_check(cudaMemcpy(e.route, route.data(), route.size() * sizeof(uint32_t), cudaMemcpyHostToDevice));
            cuda_check(cudaMemcpy(e.unit_side, sides.data(), sides.size(), cudaMemcpyHostToDevice));
            e.usable = true;
        }
        found = g_routes.emplace(key, e).first;
    }
    const RouteEntry& e = found->second;
    if (!e.usable) return false;
    out.route = e.route;
    out.sm_side = d.device_side;
    out.unit_side = e.unit_side;
    out.side_units[0] = e.side_units[0];
    out.side_units[1] = e.side_units[1];
    return true;
}

// Diagnostic: cycles per dependent atomic that each SM of `device` measured in the census (0 = not seen);
// returns how many values were written, 0 when no census has run.
int l2_side_census_cycles(int device, unsigned* out, int capacity) {
    std::lock_guard<std::mutex> hold(g_lock);
    auto it = g_sides.find(device);
    if (it == g_sides.end() || it->second.cycles.empty()) return 0;
    const int n = std::min<int>(capacity, int(it->second.cycles.size()));
    std::copy(it->second.cycles.begin(), it->second.cycles.begin() + n, out);
    return n;
}

}  // namespace nvfp4_b200
