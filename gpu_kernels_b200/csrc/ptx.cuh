// Thin inline-PTX layer for sm_100a: mbarriers with bounded waits, TMA tile
// loads/stores, Tensor Memory management and the tcgen05 block-scaled MMA.
// Every wait in this file gives up after a time limit and reports through a
// status word instead of spinning forever, so a wrong descriptor or a lost
// signal ends the kernel with an error code rather than a hung GPU.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace nvfp4_b200 {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Address of the same shared-memory offset inside CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local_addr), "r"(rank));
    return out;
}

// True in exactly one lane of a fully active warp (the same lane on every call).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- programmatic dependent launch ---------------------------------------------
// launch_dependents: once every CTA of this grid has executed it (or exited), a kernel launched behind it with
// the programmatic stream-serialisation attribute may start. grid_dependency_wait: blocks until the grid this
// launch depends on has completed and its memory is visible; returns at once for an ordinary launch.
__device__ __forceinline__ void grid_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---- mbarrier -------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(arrivals) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
// Arrive on a barrier that may live in another CTA of the cluster (address from map_to_cta).
// Release at CTA scope only: the waiter needs the arrival itself, not this thread's earlier
// memory writes (a cluster-scope release costs on the order of a thousand cycles here).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cta.shared::cluster.b64 _, [%0];" :: "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Non-blocking probe of the same condition (never suspends the warp).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Control block for bounded waits, one per CTA in shared memory.
struct WaitCtl {
    volatile uint32_t abort;   // set once any role of this CTA (or its peer) gave up
};

constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;   // 2 s: far beyond any legitimate wait

// Codes OR-ed into the device status word (bit 0..7 = who gave up).
enum StatusBits : uint32_t {
    STATUS_TIMEOUT_PRODUCER = 1u << 0,
    STATUS_TIMEOUT_MMA = 1u << 1,
    STATUS_TIMEOUT_EPILOGUE = 1u << 2,
    STATUS_TIMEOUT_TEARDOWN = 1u << 3,
    STATUS_BAD_ARGUMENT = 1u << 4,
    STATUS_TIMEOUT_PEER = 1u << 5,       // another GPU of the node did not arrive at a barrier
};

// Same test, but the hardware may park the warp for up to `hint_ns` nanoseconds while the phase
// is incomplete (it is woken at once when the phase completes), so a waiting warp issues no
// instructions and draws no issue power.
__device__ __forceinline__ bool mbar_try_wait_parked(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
    return ok != 0;
}

// Wait for the phase with the given parity. Returns false if the wait was
// abandoned (time limit, or another role already aborted); the caller must then
// leave its loop and go to the common teardown.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, WaitCtl* ctl,
                                          uint32_t* status, uint32_t who, uint32_t peer_abort_addr) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t start = globaltimer_ns();
    #pragma unroll 1
    while (true) {
        // parked in hardware for up to 20 us at a time; the abort flag and the clock are only
        // looked at between parks
        if (mbar_try_wait_parked(bar, parity, 20000u)) return true;
        if (ctl->abort) return false;
        if (globaltimer_ns() - start > WAIT_LIMIT_NS) {
            ctl->abort = 1;
            if (peer_abort_addr)
                asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(peer_abort_addr), "r"(1u) : "memory");
            atomicOr(status, who);
            return false;
        }
    }
}

// Wait (one lane) until a word in global memory that another CTA publishes with flag_publish() is
// non-zero; same limits and abort protocol as mbar_wait.
__device__ __forceinline__ bool flag_wait(const uint32_t* flag, WaitCtl* ctl, uint32_t* status, uint32_t who,
                                          uint32_t peer_abort_addr) {
    const uint64_t start = globaltimer_ns();
    #pragma unroll 1
    while (true) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v) return true;
        if (ctl->abort) return false;
        if (globaltimer_ns() - start > WAIT_LIMIT_NS) {
            ctl->abort = 1;
            if (peer_abort_addr)
                asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(peer_abort_addr), "r"(1u) : "memory");
            atomicOr(status, who);
            return false;
        }
        __nanosleep(200);
    }
}
__device__ __forceinline__ void flag_publish(uint32_t* flag, uint32_t value) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(flag), "r"(value) : "memory");
}

// ---- TMA ------------------------------------------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" :: "l"(m) : "memory");
}

// 2-D tile load into this CTA's shared memory; completion bytes go to `bar`
// (a barrier of this CTA).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// Same, issued by either CTA of a pair; `cluster_bar` may be the partner's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int x, int y,
                                                 uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :: "r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y) : "memory");
}
// The 3-D forms (scale maps: byte, row inside the row block, row block).
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        :: "r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                                 uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        :: "r"(dst), "l"(map), "r"(cluster_bar), "r"(x), "r"(y), "r"(z) : "memory");
}
// L2 policy for data that is written once and not read again by this kernel.
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* map, uint32_t src, int x, int y, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;"
        :: "l"(map), "r"(src), "r"(x), "r"(y), "l"(policy) : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        :: "l"(map), "r"(src), "r"(x), "r"(y) : "memory");
}
// One contiguous run of shared memory to global memory (this GPU's or a peer's); both addresses 16-byte
// aligned, bytes a multiple of 16. Joins the issuing thread's bulk group like the tensor stores.
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 :: "l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
// Make generic-proxy shared-memory writes visible to the async proxy (TMA store source).
__device__ __forceinline__ void fence_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- Tensor Memory ----------------------------------------------------------
template <int CG>
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t columns) {
    if constexpr (CG == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(result_smem), "r"(columns) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(result_smem), "r"(columns) : "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_relinquish() {
    if constexpr (CG == 1)
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CG>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    if constexpr (CG == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(columns) : "memory");
    else
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// 32 lanes x 32 consecutive FP32 columns -> 32 registers per thread.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared memory -> Tensor Memory copy of one 32-row x 16-byte scale atom, replicated into the four
// 32-lane quarters. The 64-bit shared-memory descriptor is passed as its two 32-bit halves: the halves are
// warp-uniform values computed outside the one-lane issue block, and only the cheap pack into a 64-bit
// register happens beside the instruction.
template <int CG>
__device__ __forceinline__ void tmem_copy_scales(uint32_t taddr, uint32_t desc_lo, uint32_t desc_hi) {
    if constexpr (CG == 1)
        asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\t"
                     "tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], d;\n\t}"
                     :: "r"(taddr), "r"(desc_lo), "r"(desc_hi) : "memory");
    else
        asm volatile("{\n\t.reg .b64 d;\n\tmov.b64 d, {%1, %2};\n\t"
                     "tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], d;\n\t}"
                     :: "r"(taddr), "r"(desc_lo), "r"(desc_hi) : "memory");
}
// D[tmem] (+)= (A * sfA) x (B * sfB)^T, E2M1 operands from shared memory, K = 64 per instruction; the 64-bit
// descriptors are passed as halves (as for the scale copies). MX = false: NVFP4, one UE4M3 scale per 16 values (scale_vec::4X);
// MX = true: MXFP4, one UE8M0 scale per 32 values (scale_vec::2X; the instruction descriptor then carries the
// UE8M0 flag and the scale-factor ids that pick two of the four scale bytes).
#define NVFP4_B200_MMA(GROUP, VEC)                                                                                       \
    asm volatile(                                                                                                        \
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"                                                                  \
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\tsetp.ne.b32 p, %7, 0;\n\t"                                   \
        "tcgen05.mma.cta_group::" GROUP ".kind::mxf4nvf4.block_scale.scale_vec::" VEC " [%0], da, db, %4, [%5], [%6], p;\n\t}" \
        :: "r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)   \
        : "memory")
template <int CG, bool MX>
__device__ __forceinline__ void mma_block_scaled(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                                 uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
    if constexpr (CG == 1 && !MX) NVFP4_B200_MMA("1", "4X");
    else if constexpr (CG == 2 && !MX) NVFP4_B200_MMA("2", "4X");
    else if constexpr (CG == 1 && MX) NVFP4_B200_MMA("1", "2X");
    else NVFP4_B200_MMA("2", "2X");
}
#undef NVFP4_B200_MMA

// Arrive on `bar` once all tcgen05 operations issued so far by this thread have
// completed. For a pair the arrival is delivered to the same barrier offset in
// both CTAs.
template <int CG>
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    if constexpr (CG == 1)
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                     :: "r"(bar) : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                     :: "r"(bar), "h"(static_cast<uint16_t>(3)) : "memory");
}

}  // namespace ptx
}  // namespace nvfp4_b200
