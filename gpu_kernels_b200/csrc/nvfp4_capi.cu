// extern "C" surface of libgpu_kernels_nvfp4_bench.so (declared in include/nvfp4_capi.h).
// Every entry point catches all exceptions, stores the message per thread and
// returns 1, the convention of the reference's bridge
// (benchmarks/bindings/nvfp4_bridge.cu:11,88-91).
#include "nvfp4.h"
#include "nvfp4_capi.h"
#include "nvfp4_internal.h"

#include <cublasLt.h>

#include <atomic>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <vector>
#include <string>

namespace nvfp4_b200 {
extern std::atomic<unsigned long long> g_launches;
int gemm_stage_count(int cta_group, int tile_n, int direct_store);
void validate_device_slot(int device);
unsigned last_kernel_cycles();
int gemm_profile(const gpu_kernels::Nvfp4Params& p, __half* C, cudaStream_t stream, unsigned long long* host, int max_words);
}

namespace {

thread_local std::string t_error;

template <typename F>
int guarded(F&& body) {
    try {
        body();
        return 0;
    } catch (const std::exception& e) {
        t_error = e.what();
    } catch (...) {
        t_error = "unknown error";
    }
    return 1;
}

void lt_check(cublasStatus_t s, const char* what) {
    if (s != CUBLAS_STATUS_SUCCESS)
        throw std::runtime_error(std::string("cuBLASLt ") + what + " failed with status " + std::to_string(int(s)));
}

// cuBLASLt's own NVFP4 matmul on the plan's shape: the library bar this kernel is
// compared with, never part of the product path. Built lazily on first use.
class LtMatmul {
public:
    LtMatmul(int M, int N, int K, const void* sfa, const void* sfb, size_t workspace_limit) {
        lt_check(cublasLtCreate(&handle_), "create");
        lt_check(cublasLtMatmulDescCreate(&op_, CUBLAS_COMPUTE_32F, CUDA_R_32F), "desc");
        // cuBLASLt is column-major: C^T[N,M] = B[N,K] * A[M,K]^T, i.e. its "A" operand is our B.
        set(CUBLASLT_MATMUL_DESC_TRANSA, CUBLAS_OP_T);
        set(CUBLASLT_MATMUL_DESC_TRANSB, CUBLAS_OP_N);
        set(CUBLASLT_MATMUL_DESC_A_SCALE_MODE, CUBLASLT_MATMUL_MATRIX_SCALE_VEC16_UE4M3);
        set(CUBLASLT_MATMUL_DESC_B_SCALE_MODE, CUBLASLT_MATMUL_MATRIX_SCALE_VEC16_UE4M3);
        set(CUBLASLT_MATMUL_DESC_A_SCALE_POINTER, sfb);
        set(CUBLASLT_MATMUL_DESC_B_SCALE_POINTER, sfa);
        lt_check(cublasLtMatrixLayoutCreate(&lb_, CUDA_R_4F_E2M1, K, N, K), "layout B");
        lt_check(cublasLtMatrixLayoutCreate(&la_, CUDA_R_4F_E2M1, K, M, K), "layout A");
        lt_check(cublasLtMatrixLayoutCreate(&lc_, CUDA_R_16F, N, M, N), "layout C");
        lt_check(cublasLtMatmulPreferenceCreate(&pref_), "preference");
        lt_check(cublasLtMatmulPreferenceSetAttribute(pref_, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES,
                                                      &workspace_limit, sizeof(workspace_limit)), "workspace");
        cublasLtMatmulHeuristicResult_t found{};
        int n = 0;
        lt_check(cublasLtMatmulAlgoGetHeuristic(handle_, op_, lb_, la_, lc_, lc_, pref_, 1, &found, &n), "heuristic");
        if (n == 0) throw std::runtime_error("cuBLASLt offers no NVFP4 algorithm for this shape on this device");
        algo_ = found.algo;
        workspace_bytes_ = found.workspaceSize;
    }
    ~LtMatmul() {
        if (pref_) cublasLtMatmulPreferenceDestroy(pref_);
        if (lc_) cublasLtMatrixLayoutDestroy(lc_);
        if (la_) cublasLtMatrixLayoutDestroy(la_);
        if (lb_) cublasLtMatrixLayoutDestroy(lb_);
        if (op_) cublasLtMatmulDescDestroy(op_);
        if (handle_) cublasLtDestroy(handle_);
    }
    void run(void* C, const void* A, const void* B, void* workspace, cudaStream_t stream) const {
        const float one = 1.0f, zero = 0.0f;
        lt_check(cublasLtMatmul(handle_, op_, &one, B, lb_, A, la_, &zero, C, lc_, C, lc_, &algo_,
                                workspace, workspace_bytes_, stream), "matmul");
    }

private:
    template <typename T>
    void set(cublasLtMatmulDescAttributes_t attr, T value) {
        lt_check(cublasLtMatmulDescSetAttribute(op_, attr, &value, sizeof(value)), "attribute");
    }
    cublasLtHandle_t handle_ = nullptr;
    cublasLtMatmulDesc_t op_ = nullptr;
    cublasLtMatrixLayout_t la_ = nullptr, lb_ = nullptr, lc_ = nullptr;
    cublasLtMatmulPreference_t pref_ = nullptr;
    cublasLtMatmulAlgo_t algo_{};
    size_t workspace_bytes_ = 0;
};

struct Plan {
    gpu_kernels::Nvfp4Params params{};
    gpu_kernels::Nvfp4Implementation impl{};
    const void* sfa = nullptr;
    const void* sfb = nullptr;
    const void* b = nullptr;
    const void* a = nullptr;
    void* workspace = nullptr;
    size_t workspace_bytes = 0;
    std::unique_ptr<LtMatmul> lt;
    void* gather_table = nullptr;           // owned
    void* split_k_workspace = nullptr;      // owned
    size_t split_k_bytes = 0;
    int whole_tile_units = 0;                // params.clusters and direct_store of the unsplit schedule
    int whole_tile_direct_store = 0;
    Plan() = default;
    Plan(const Plan&) = delete;
    Plan& operator=(const Plan&) = delete;
    ~Plan() {
        if (split_k_workspace) cudaFree(split_k_workspace);
        if (gather_table) cudaFree(gather_table);
    }
};

Plan& as_plan(void* p) {
    if (!p) throw std::invalid_argument("null plan");
    return *static_cast<Plan*>(p);
}

// Device staging for gpu_kernels_nvfp4_gemm_host, kept between calls of one shape.
struct HostGemm {
    int M = 0, N = 0, K = 0;
    uint8_t *A = nullptr, *B = nullptr, *SFA = nullptr, *SFB = nullptr;
    __half* C = nullptr;
    Plan plan;
    // The product in row pieces x column pieces. Copies in and kernels go on the caller's stream in the order
    // A piece 0, B piece 0, block (0,0), B piece 1, block (0,1), ..., A piece 1, block (1,0), ...; every block's
    // result leaves on a second stream as soon as it is computed. So the first bytes of C travel back after one
    // piece of each operand has arrived, and from then on both directions of the host link are busy.
    std::vector<gpu_kernels::Nvfp4Params> pieces;      // [row piece][column piece]
    int piece_rows = 0, piece_cols = 0, row_pieces = 0, col_pieces = 0;
    cudaStream_t out_stream = nullptr;
    std::vector<cudaEvent_t> piece_done;
    void release() {
        for (void* p : {static_cast<void*>(A), static_cast<void*>(B), static_cast<void*>(SFA), static_cast<void*>(SFB),
                        static_cast<void*>(C)})
            if (p) cudaFree(p);
        for (cudaEvent_t e : piece_done) cudaEventDestroy(e);
        if (out_stream) cudaStreamDestroy(out_stream);
        piece_done.clear();
        pieces.clear();
        out_stream = nullptr;
        piece_rows = piece_cols = row_pieces = col_pieces = 0;
        A = B = SFA = SFB = nullptr;
        C = nullptr;
        M = N = K = 0;
    }
};
std::mutex g_host_lock;
std::map<int, HostGemm> g_host;          // one staging set per device: buffers and tensor maps belong to a GPU

// ---- staging for gpu_kernels_nvfp4_gemm_host_static ---------------------------------------
// Some hosts of this library may not allocate device memory while they run: a service that sized
// its memory pool up front and forbids later cudaMalloc calls (they synchronise the device and can
// fail when the pool owns the whole GPU), or code that runs between the capture-time and run-time
// phases of a larger program. For them the device copies of the operands live in this one
// file-scope array. It costs every process that loads the library 2.7 MiB per GPU until exit.
constexpr int STATIC_MAX_M = 512, STATIC_MAX_N = 1024, STATIC_MAX_K = 2048;
constexpr size_t STATIC_OFF_A = 0;
constexpr size_t STATIC_OFF_B = STATIC_OFF_A + size_t(STATIC_MAX_M) * STATIC_MAX_K / 2;
constexpr size_t STATIC_OFF_SFA = STATIC_OFF_B + size_t(STATIC_MAX_N) * STATIC_MAX_K / 2;
constexpr size_t STATIC_OFF_SFB = STATIC_OFF_SFA + size_t(STATIC_MAX_M) * STATIC_MAX_K / 16;
constexpr size_t STATIC_OFF_C = STATIC_OFF_SFB + size_t(STATIC_MAX_N) * STATIC_MAX_K / 16;
constexpr size_t STATIC_BYTES = STATIC_OFF_C + size_t(STATIC_MAX_M) * STATIC_MAX_N * 2;
static_assert(STATIC_OFF_B % 256 == 0 && STATIC_OFF_SFA % 256 == 0 && STATIC_OFF_SFB % 256 == 0 && STATIC_OFF_C % 256 == 0,
              "sub-buffers keep the 256-byte alignment of the array");
static __device__ __align__(256) unsigned char g_static_stage[STATIC_BYTES];

// In host code `g_static_stage` is only a handle for the runtime, not a device address; the
// address a kernel or a tensor map can use comes from cudaGetSymbolAddress, once per device, with
// that device current.
std::mutex g_static_lock;
unsigned char* g_static_base[64] = {};

unsigned char* static_stage_base() {
    int device = 0;
    nvfp4_b200::cuda_check(cudaGetDevice(&device));
    if (device < 0 || device >= 64) throw std::runtime_error("gemm_host_static: device index out of range");
    std::lock_guard<std::mutex> hold(g_static_lock);
    if (!g_static_base[device]) {
        void* p = nullptr;
        nvfp4_b200::cuda_check(cudaGetSymbolAddress(&p, g_static_stage));
        if (!p) throw std::runtime_error("gemm_host_static: the staging array has no address on this device");
        g_static_base[device] = static_cast<unsigned char*>(p);
    }
    return g_static_base[device];
}

}  // namespace

extern "C" {

const char* gpu_kernels_nvfp4_last_error(void) { return t_error.c_str(); }

int gpu_kernels_nvfp4_plan_create(void** out, int M, int N, int K, const void* A, const void* B, const void* SFA,
                                  const void* SFB, void* workspace, size_t workspace_bytes, void* stream) {
    return guarded([&] {
        if (!out) throw std::invalid_argument("plan_create: null result pointer");
        auto plan = std::make_unique<Plan>();
        plan->impl = gpu_kernels::nvfp4_sm100_implementation();
        plan->impl.prepare(plan->params, static_cast<const uint8_t*>(A), static_cast<const uint8_t*>(B),
                           static_cast<const uint8_t*>(SFA), static_cast<const uint8_t*>(SFB), M, N, K,
                           static_cast<cudaStream_t>(stream));
        plan->sfa = SFA;
        plan->sfb = SFB;
        plan->b = B;
        plan->a = A;
        plan->workspace = workspace;
        plan->workspace_bytes = workspace_bytes;
        plan->whole_tile_units = plan->params.clusters;
        plan->whole_tile_direct_store = plan->params.direct_store;
        // off unless asked for: its units wait for each other, which needs the GPU's SMs free of other kernels
        const char* on = std::getenv("NVFP4_B200_SPLIT_K");
        plan->split_k_bytes = gpu_kernels::nvfp4_split_k_workspace_bytes(plan->params);
        if (plan->split_k_bytes && on && on[0] == '1') {
            nvfp4_b200::cuda_check(cudaMalloc(&plan->split_k_workspace, plan->split_k_bytes));
            gpu_kernels::nvfp4_enable_split_k(plan->params, plan->split_k_workspace, plan->split_k_bytes,
                                               static_cast<cudaStream_t>(stream));
        }
        *out = plan.release();
    });
}

int gpu_kernels_nvfp4_plan_create_mx(void** out, int M, int N, int K, const void* A, const void* B, const void* SFA,
                                     const void* SFB, void* stream) {
    return guarded([&] {
        if (!out) throw std::invalid_argument("plan_create_mx: null result pointer");
        auto plan = std::make_unique<Plan>();
        plan->impl = gpu_kernels::nvfp4_sm100_implementation();
        gpu_kernels::mxfp4_prepare(plan->params, static_cast<const uint8_t*>(A), static_cast<const uint8_t*>(B),
                                   static_cast<const uint8_t*>(SFA), static_cast<const uint8_t*>(SFB), M, N, K,
                                   static_cast<cudaStream_t>(stream));
        plan->sfa = SFA;
        plan->sfb = SFB;
        plan->b = B;
        plan->a = A;
        plan->whole_tile_units = plan->params.clusters;
        plan->whole_tile_direct_store = plan->params.direct_store;
        *out = plan.release();
    });
}

void gpu_kernels_nvfp4_plan_destroy(void* plan) { delete static_cast<Plan*>(plan); }

int gpu_kernels_nvfp4_cublas(void* plan, void* C, const void* A, const void* B, void* stream) {
    return guarded([&] {
        Plan& p = as_plan(plan);
        if (p.params.mx) throw std::invalid_argument("cublas: the comparison path is set up for NVFP4 plans only");
        if (!p.lt)
            p.lt = std::make_unique<LtMatmul>(p.params.M, p.params.N, p.params.K, p.sfa, p.sfb,
                                              p.workspace ? p.workspace_bytes : 0);
        p.lt->run(C, A, B, p.workspace, static_cast<cudaStream_t>(stream));
    });
}

int gpu_kernels_nvfp4_custom(void* plan, void* C, void* stream) {
    return guarded([&] {
        Plan& p = as_plan(plan);
        p.impl.launch(p.params, static_cast<__half*>(C), static_cast<cudaStream_t>(stream));
    });
}

int gpu_kernels_nvfp4_linear(void* plan, const void* x, int dtype, void* C, void* stream) {
    return guarded([&] {
        Plan& p = as_plan(plan);
        if (p.params.mx) throw std::invalid_argument("linear: NVFP4 plans only");
        auto s = static_cast<cudaStream_t>(stream);
        // x -> the plan's own A and SFA buffers, then the GEMM. The quantiser lets its dependents start at once
        // and the GEMM is told that the kernel in front of it leaves B alone, so under programmatic dependent
        // launch it sets itself up and requests its first tiles of B while the quantiser runs, and waits for the
        // quantiser's bytes only before its first load of A.
        nvfp4_b200::quantise(x, dtype, static_cast<uint8_t*>(const_cast<void*>(p.a)),
                             static_cast<uint8_t*>(const_cast<void*>(p.sfa)), p.params.M, p.params.K, s);
        gpu_kernels::Nvfp4Params q = p.params;
        if (q.static_operands != 1) q.static_operands = 1;      // 2 would let the GEMM read A before it is written
        p.impl.launch(q, static_cast<__half*>(C), s);
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_validate(void* plan) {
    return guarded([&] {
        // a plan reports to its own status slot; a null plan checks every slot of the current device (this is
        // how grouped launches and the expert-path kernels, which report to the device's own slot, are checked)
        if (!plan) gpu_kernels::nvfp4_sm100_implementation().validate();
        else gpu_kernels::nvfp4_validate_plan(as_plan(plan).params);
    });
}

int gpu_kernels_nvfp4_l2_bytes(void) {
    int device = 0, bytes = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&bytes, cudaDevAttrL2CacheSize, device) != cudaSuccess) return 0;
    return bytes;
}

int gpu_kernels_nvfp4_quantize(const void* x, int dtype, void* packed, void* scales, int rows, int K, void* stream) {
    return guarded([&] {
        nvfp4_b200::require_sm100();
        nvfp4_b200::quantise(x, dtype, static_cast<uint8_t*>(packed), static_cast<uint8_t*>(scales), rows, K,
                             static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_quantize_scaled(const void* x, int dtype, float inv_tensor_scale, void* packed, void* scales, int rows,
                                      int K, void* stream) {
    return guarded([&] {
        nvfp4_b200::require_sm100();
        nvfp4_b200::quantise_scaled(x, dtype, inv_tensor_scale, static_cast<uint8_t*>(packed), static_cast<uint8_t*>(scales),
                                    rows, K, static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_quantize_mx(const void* x, int dtype, void* packed, void* scales, int rows, int K, void* stream) {
    return guarded([&] {
        nvfp4_b200::require_sm100();
        nvfp4_b200::quantise_mx(x, dtype, static_cast<uint8_t*>(packed), static_cast<uint8_t*>(scales), rows, K,
                                static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_dequantize_mx(const void* packed, const void* scales, void* out, int rows, int K, void* stream) {
    return guarded([&] {
        nvfp4_b200::require_sm100();
        nvfp4_b200::dequantise_mx(static_cast<const uint8_t*>(packed), static_cast<const uint8_t*>(scales),
                                  static_cast<float*>(out), rows, K, static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_dequantize(const void* packed, const void* scales, void* out, int rows, int K, void* stream) {
    return guarded([&] {
        nvfp4_b200::require_sm100();
        nvfp4_b200::dequantise(static_cast<const uint8_t*>(packed), static_cast<const uint8_t*>(scales),
                               static_cast<float*>(out), rows, K, static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_plan_set_alpha(void* plan, float alpha) {
    return guarded([&] { gpu_kernels::nvfp4_set_alpha(as_plan(plan).params, alpha); });
}

int gpu_kernels_nvfp4_plan_set_option(void* plan, const char* key, int value) {
    return guarded([&] {
        Plan& p = as_plan(plan);
        if (!key) throw std::invalid_argument("set_option: null key");
        if (std::strcmp(key, "group_m") == 0) {
            const int tiles_m = p.params.M / (128 * p.params.cta_group);
            if (value < 1) throw std::invalid_argument("set_option: group_m must be >= 1");
            p.params.group_m = value < tiles_m ? value : tiles_m;
        } else if (std::strcmp(key, "c_evict_first") == 0) {
            p.params.c_evict_first = value ? 1 : 0;
        } else if (std::strcmp(key, "direct_store") == 0) {
            if (p.params.split_k > 1 && !value) throw std::invalid_argument("set_option: split-K writes C from registers");
            p.params.direct_store = value ? 1 : 0;
            p.whole_tile_direct_store = p.params.direct_store;
        } else if (std::strcmp(key, "k_skew") == 0) {
            if (value < 0) throw std::invalid_argument("set_option: k_skew must be >= 0");
            p.params.k_skew = value;
        } else if (std::strcmp(key, "ragged_tiles") == 0) {
            // value tiles over the plan's one tile row (0 = uniform 256-column tiles); refused where it does not apply
            if (!gpu_kernels::nvfp4_set_ragged_tiles(p.params, static_cast<const uint8_t*>(p.b), value) && value)
                throw std::invalid_argument("set_option: ragged_tiles needs M = 128, N a multiple of 64 and 2 to 4 units of 64 "
                                            "columns per tile, more tiles than N / 256");
        } else if (std::strcmp(key, "pdl") == 0) {
            p.params.pdl = value ? 1 : 0;
        } else if (std::strcmp(key, "static_operands") == 0) {
            if (value < 0 || value > 2) throw std::invalid_argument("set_option: static_operands is 0, 1 or 2");
            p.params.static_operands = value;
        } else if (std::strcmp(key, "out_bf16") == 0) {
            if (p.params.gather_world) throw std::invalid_argument("set_option: choose the output type before set_gather");
            p.params.out_bf16 = value ? 1 : 0;
        } else if (std::strcmp(key, "l2_side") == 0) {
            // value 1: ask for the L2-side-aware order; refused (error) when the census cannot provide it
            if (!gpu_kernels::nvfp4_set_l2_side_order(p.params, value, nullptr) && value)
                throw std::runtime_error("set_option: no L2-side order for this plan (grid smaller than the GPU, too few tiles, "
                                         "or the census did not split the SMs into two sides)");
        } else if (std::strcmp(key, "split_k") == 0) {
            if (!value) {
                p.params.split_k = 0;
                p.params.clusters = p.whole_tile_units;
                p.params.direct_store = p.whole_tile_direct_store;
            } else if (p.params.split_k <= 1) {
                if (!p.split_k_bytes) throw std::invalid_argument("set_option: split_k does not apply to this shape");
                if (!p.split_k_workspace) nvfp4_b200::cuda_check(cudaMalloc(&p.split_k_workspace, p.split_k_bytes));
                gpu_kernels::nvfp4_enable_split_k(p.params, p.split_k_workspace, p.split_k_bytes, nullptr);
            }
        } else {
            throw std::invalid_argument(std::string("set_option: unknown key ") + key);
        }
    });
}

int gpu_kernels_nvfp4_plan_set_gather(void* plan, void* const* buffers, int world, int col0, int n_total) {
    return guarded([&] {
        Plan& p = as_plan(plan);
        if (world > 0 && !p.gather_table) {
            nvfp4_b200::cuda_check(cudaMalloc(&p.gather_table, gpu_kernels::nvfp4_gather_table_bytes(64)));
        }
        gpu_kernels::nvfp4_set_gather(p.params, buffers, world, col0, n_total, p.gather_table, nullptr);
    });
}

int gpu_kernels_nvfp4_plan_info(void* plan, int* info) {
    return guarded([&] {
        Plan& p = as_plan(plan);
        if (!info) throw std::invalid_argument("plan_info: null output");
        const auto& q = p.params;
        const int values[16] = {q.M, q.N, q.K, q.clusters, q.cta_group, q.tile_n, q.group_m,
                                nvfp4_b200::gemm_stage_count(q.cta_group, q.tile_n, q.direct_store), q.split_k, q.k_skew,
                                q.direct_store, q.out_bf16, q.route ? 1 : 0, q.side_units[0], q.side_units[1],
                                q.ragged_units};
        std::memcpy(info, values, sizeof(values));
    });
}

int gpu_kernels_nvfp4_gemm_host(int M, int N, int K, const void* A, const void* B, const void* SFA, const void* SFB,
                                void* C, float alpha, void* stream_) {
    return guarded([&] {
        using nvfp4_b200::cuda_check;
        if (!A || !B || !SFA || !SFB || !C) throw std::invalid_argument("gemm_host: null pointer");
        nvfp4_b200::require_sm100();
        auto stream = static_cast<cudaStream_t>(stream_);
        int device = 0;
        cuda_check(cudaGetDevice(&device));
        std::lock_guard<std::mutex> hold(g_host_lock);
        HostGemm& h = g_host[device];
        const size_t a_bytes = size_t(M) * K / 2, b_bytes = size_t(N) * K / 2;
        const size_t sfa_bytes = size_t(M) * K / 16, sfb_bytes = size_t(N) * K / 16, c_bytes = size_t(M) * N * 2;
        if (h.M != M || h.N != N || h.K != K) {
            h.release();
            if (M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 128 || K % 64)
                throw std::invalid_argument("gemm_host: M, N multiples of 128 and K a multiple of 64 are required");
            cuda_check(cudaMalloc(&h.A, a_bytes));
            cuda_check(cudaMalloc(&h.B, b_bytes));
            cuda_check(cudaMalloc(&h.SFA, sfa_bytes));
            cuda_check(cudaMalloc(&h.SFB, sfb_bytes));
            cuda_check(cudaMalloc(&h.C, c_bytes));
            h.plan.impl = gpu_kernels::nvfp4_sm100_implementation();
            h.plan.impl.prepare(h.plan.params, h.A, h.B, h.SFA, h.SFB, M, N, K, stream);
            // large products go in 4 (or 2) row pieces and as many column pieces, all of whole 256-wide tiles
            auto split = [](int extent) { return (extent >= 2048 && extent % 1024 == 0) ? 4 : (extent >= 1024 && extent % 512 == 0) ? 2 : 1; };
            const int rows_n = split(M), cols_n = rows_n > 1 ? split(N) : 1;
            if (rows_n > 1) {
                h.row_pieces = rows_n;
                h.col_pieces = cols_n;
                h.piece_rows = M / rows_n;
                h.piece_cols = N / cols_n;
                h.pieces.resize(size_t(rows_n) * cols_n);
                h.piece_done.resize(h.pieces.size());
                cuda_check(cudaStreamCreateWithFlags(&h.out_stream, cudaStreamNonBlocking));
                for (int r = 0; r < rows_n; ++r)
                    for (int c = 0; c < cols_n; ++c) {
                        const size_t row0 = size_t(r) * h.piece_rows, col0 = size_t(c) * h.piece_cols;
                        const size_t i = size_t(r) * cols_n + c;
                        h.plan.impl.prepare(h.pieces[i], h.A + row0 * K / 2, h.B + col0 * K / 2, h.SFA + row0 * K / 16,
                                            h.SFB + col0 * K / 16, h.piece_rows, h.piece_cols, K, stream);
                        cuda_check(cudaEventCreateWithFlags(&h.piece_done[i], cudaEventDisableTiming));
                    }
            }
            h.M = M; h.N = N; h.K = K;
        }
        if (h.pieces.empty()) {
            h.plan.params.alpha = alpha;
            cuda_check(cudaMemcpyAsync(h.B, B, b_bytes, cudaMemcpyHostToDevice, stream));
            cuda_check(cudaMemcpyAsync(h.SFB, SFB, sfb_bytes, cudaMemcpyHostToDevice, stream));
            cuda_check(cudaMemcpyAsync(h.SFA, SFA, sfa_bytes, cudaMemcpyHostToDevice, stream));
            cuda_check(cudaMemcpyAsync(h.A, A, a_bytes, cudaMemcpyHostToDevice, stream));
            h.plan.impl.launch(h.plan.params, h.C, stream);
            cuda_check(cudaMemcpyAsync(C, h.C, c_bytes, cudaMemcpyDeviceToHost, stream));
            cuda_check(cudaStreamSynchronize(stream));
            return;
        }
        const size_t a_piece = size_t(h.piece_rows) * K / 2, sfa_piece = size_t(h.piece_rows) * K / 16;
        const size_t b_piece = size_t(h.piece_cols) * K / 2, sfb_piece = size_t(h.piece_cols) * K / 16;
        const size_t block_elems = size_t(h.piece_rows) * h.piece_cols;
        auto in = [&](uint8_t* dst, const void* src, size_t offset, size_t bytes) {
            cuda_check(cudaMemcpyAsync(dst + offset, static_cast<const uint8_t*>(src) + offset, bytes, cudaMemcpyHostToDevice, stream));
        };
        for (int r = 0; r < h.row_pieces; ++r) {
            in(h.A, A, r * a_piece, a_piece);
            in(h.SFA, SFA, r * sfa_piece, sfa_piece);
            for (int c = 0; c < h.col_pieces; ++c) {
                if (r == 0) {
                    in(h.B, B, c * b_piece, b_piece);
                    in(h.SFB, SFB, c * sfb_piece, sfb_piece);
                }
                const size_t i = size_t(r) * h.col_pieces + c;
                h.pieces[i].alpha = alpha;
                // every block has its own compact [piece_rows, piece_cols] area of the staging C
                __half* block = h.C + i * block_elems;
                h.plan.impl.launch(h.pieces[i], block, stream);
                cuda_check(cudaEventRecord(h.piece_done[i], stream));
                cuda_check(cudaStreamWaitEvent(h.out_stream, h.piece_done[i], 0));
                __half* dst = static_cast<__half*>(C) + size_t(r) * h.piece_rows * N + size_t(c) * h.piece_cols;
                cuda_check(cudaMemcpy2DAsync(dst, size_t(N) * 2, block, size_t(h.piece_cols) * 2, size_t(h.piece_cols) * 2,
                                             size_t(h.piece_rows), cudaMemcpyDeviceToHost, h.out_stream));
            }
        }
        cuda_check(cudaStreamSynchronize(h.out_stream));
        cuda_check(cudaStreamSynchronize(stream));
    });
}

int gpu_kernels_nvfp4_plan_profile(void* plan, void* C, void* stream, unsigned long long* counters, int max_words,
                                   int* words_written) {
    return guarded([&] {
        Plan& p = as_plan(plan);
        if (!counters || !words_written) throw std::invalid_argument("plan_profile: null output");
        *words_written = nvfp4_b200::gemm_profile(p.params, static_cast<__half*>(C), static_cast<cudaStream_t>(stream),
                                                  counters, max_words);
    });
}

unsigned gpu_kernels_nvfp4_last_kernel_cycles(void) {
    unsigned cycles = 0;
    guarded([&] { cycles = nvfp4_b200::last_kernel_cycles(); });
    return cycles;
}

/* ---- routed-MoE expert path ---- */

int gpu_kernels_nvfp4_grouped_plan_create(void** out, int pool_rows, int n, int k, int experts, int block_rows,
                                          const void* A, const void* B, const void* SFA, const void* SFB,
                                          const void* block_expert, const void* num_blocks) {
    return guarded([&] {
        if (!out) throw std::invalid_argument("grouped_plan_create: null result pointer");
        auto plan = std::make_unique<nvfp4_b200::GroupedGemm>();
        nvfp4_b200::grouped_prepare(*plan, static_cast<const uint8_t*>(A), static_cast<const uint8_t*>(B),
                                    static_cast<const uint8_t*>(SFA), static_cast<const uint8_t*>(SFB), pool_rows, n, k,
                                    experts, block_rows, static_cast<const int*>(block_expert),
                                    static_cast<const int*>(num_blocks));
        *out = plan.release();
    });
}

void gpu_kernels_nvfp4_grouped_plan_destroy(void* plan) { delete static_cast<nvfp4_b200::GroupedGemm*>(plan); }

int gpu_kernels_nvfp4_grouped_set_valid_rows(void* plan, const void* block_valid) {
    return guarded([&] {
        if (!plan) throw std::invalid_argument("grouped set_valid_rows: null plan");
        static_cast<nvfp4_b200::GroupedGemm*>(plan)->block_valid = static_cast<const int*>(block_valid);
    });
}

int gpu_kernels_nvfp4_grouped_run(void* plan, void* C, int out_bf16, void* stream) {
    return guarded([&] {
        if (!plan) throw std::invalid_argument("null plan");
        nvfp4_b200::grouped_launch(*static_cast<nvfp4_b200::GroupedGemm*>(plan), C, out_bf16,
                                   static_cast<cudaStream_t>(stream));
    });
}

int gpu_kernels_nvfp4_grouped_run_swiglu(void* plan, const void* row_weight, float clamp, void* act_packed,
                                         void* act_scales, void* stream) {
    return guarded([&] {
        if (!plan) throw std::invalid_argument("null plan");
        nvfp4_b200::grouped_launch_fused(*static_cast<nvfp4_b200::GroupedGemm*>(plan), nullptr, 1,
                                         static_cast<uint8_t*>(act_packed), static_cast<uint8_t*>(act_scales),
                                         static_cast<const float*>(row_weight), clamp, nullptr, nullptr, 0, 0,
                                         static_cast<cudaStream_t>(stream));
    });
}

int gpu_kernels_nvfp4_grouped_run_scatter(void* plan, const void* row_dst, const void* slots, void* own_slots, int world,
                                          int slot_rows, int out_bf16, void* stream) {
    return guarded([&] {
        if (!plan) throw std::invalid_argument("null plan");
        if (!row_dst) throw std::invalid_argument("grouped_run_scatter: null row_dst");
        nvfp4_b200::grouped_launch_fused(*static_cast<nvfp4_b200::GroupedGemm*>(plan), own_slots, out_bf16, nullptr, nullptr,
                                         nullptr, 0.0f, static_cast<const int*>(row_dst),
                                         static_cast<void* const*>(slots), world, slot_rows,
                                         static_cast<cudaStream_t>(stream));
    });
}

int gpu_kernels_nvfp4_moe_payload_bytes(int hidden) { return nvfp4_b200::moe_payload_bytes(hidden); }

int gpu_kernels_nvfp4_moe_route_count(const void* ids, int routes, int experts, void* counts, void* stream) {
    return guarded([&] {
        nvfp4_b200::require_sm100();
        nvfp4_b200::moe_route_count(static_cast<const long long*>(ids), routes, experts, static_cast<int*>(counts),
                                    static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_plan(const void* counts_matrix, int world, int rank, int experts, int capacity_rows,
                               int block_rows, void* send_offset, void* seg_src_offset, void* seg_pool_offset, void* block_expert,
                               void* num_blocks, void* totals, void* peer_offset, int peer_to_pool, void* cursor, void* block_valid,
                               void* stream) {
    return guarded([&] {
        nvfp4_b200::require_sm100();
        nvfp4_b200::moe_plan(static_cast<int*>(block_valid), const_cast<int*>(static_cast<const int*>(counts_matrix)), world, rank, experts, capacity_rows,
                             block_rows, static_cast<int*>(send_offset), static_cast<int*>(seg_src_offset),
                             static_cast<int*>(seg_pool_offset), static_cast<int*>(block_expert),
                             static_cast<int*>(num_blocks), static_cast<int*>(totals), static_cast<int*>(peer_offset),
                             nullptr, 0, static_cast<int*>(cursor), peer_to_pool, static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_route_plan(const void* ids, int routes, void* counts, int experts, int capacity_rows, int block_rows,
                                     void* send_offset, void* seg_src_offset, void* seg_pool_offset, void* block_expert,
                                     void* num_blocks, void* totals, void* cursor, void* block_valid, void* stream) {
    return guarded([&] {
        nvfp4_b200::require_sm100();
        if (!ids || !counts || !cursor) throw std::invalid_argument("moe route_plan: null pointer");
        nvfp4_b200::moe_plan(static_cast<int*>(block_valid), static_cast<int*>(counts), 1, 0, experts, capacity_rows, block_rows,
                             static_cast<int*>(send_offset), static_cast<int*>(seg_src_offset),
                             static_cast<int*>(seg_pool_offset), static_cast<int*>(block_expert),
                             static_cast<int*>(num_blocks), static_cast<int*>(totals), nullptr,
                             static_cast<const long long*>(ids), routes, static_cast<int*>(cursor), 0,
                             static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_unpack_meta(const void* side, int recv_capacity, const void* totals, int world, int local_experts,
                                      int hidden, const void* seg_src_offset, const void* seg_pool_offset, void* pool_scales,
                                      void* pool_weight, void* pool_dst, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_unpack_meta(static_cast<const uint8_t*>(side), recv_capacity, static_cast<const int*>(totals), world,
                                    local_experts, hidden, static_cast<const int*>(seg_src_offset),
                                    static_cast<const int*>(seg_pool_offset), static_cast<uint8_t*>(pool_scales),
                                    static_cast<float*>(pool_weight), static_cast<int*>(pool_dst),
                                    static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_clear_live(const void* num_blocks, int block_rows, int pool_rows, int hidden, void* pool_scales,
                                     void* pool_weight, void* pool_dst, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_clear_live(static_cast<const int*>(num_blocks), block_rows, pool_rows, hidden,
                                   static_cast<uint8_t*>(pool_scales), static_cast<float*>(pool_weight),
                                   static_cast<int*>(pool_dst), static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_pack(const void* xq, const void* xs, const void* ids, const void* weights, int tokens,
                               int topk, int hidden, int experts, const void* send_offset, void* cursor, void* send_rows,
                               void* send_pos, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_pack(static_cast<const uint8_t*>(xq), static_cast<const uint8_t*>(xs),
                             static_cast<const long long*>(ids), static_cast<const float*>(weights), tokens, topk, hidden,
                             experts, static_cast<const int*>(send_offset), static_cast<int*>(cursor),
                             static_cast<uint8_t*>(send_rows), static_cast<int*>(send_pos),
                             static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_pack_to_pool(const void* xq, const void* xs, const void* ids, const void* weights, int tokens,
                                       int topk, int hidden, int experts, const void* seg_pool_offset, void* cursor,
                                       void* pool_packed, void* pool_scales, void* pool_weight, void* route_row,
                                       void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_pack_to_pool(static_cast<const uint8_t*>(xq), static_cast<const uint8_t*>(xs),
                                     static_cast<const long long*>(ids), static_cast<const float*>(weights), tokens, topk,
                                     hidden, experts, static_cast<const int*>(seg_pool_offset), static_cast<int*>(cursor),
                                     static_cast<uint8_t*>(pool_packed), static_cast<uint8_t*>(pool_scales),
                                     static_cast<float*>(pool_weight), static_cast<int*>(route_row),
                                     static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_unpack(const void* recv_rows, int recv_capacity, const void* totals, int world,
                                 int local_experts, int hidden, const void* seg_src_offset, const void* seg_pool_offset,
                                 void* pool_packed, void* pool_scales, void* pool_weight, void* pool_of_recv,
                                 void* pool_dst, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_unpack(static_cast<const uint8_t*>(recv_rows), recv_capacity, static_cast<const int*>(totals),
                               world, local_experts, hidden, static_cast<const int*>(seg_src_offset),
                               static_cast<const int*>(seg_pool_offset), static_cast<uint8_t*>(pool_packed),
                               static_cast<uint8_t*>(pool_scales), static_cast<float*>(pool_weight),
                               static_cast<int*>(pool_of_recv), static_cast<int*>(pool_dst),
                               static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_swiglu_quant(const void* gate_up, const void* pool_weight, const void* num_blocks,
                                       int block_rows, int pool_rows, int intermediate, float clamp, void* act_packed,
                                       void* act_scales, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_swiglu_quant(gate_up, static_cast<const float*>(pool_weight), static_cast<const int*>(num_blocks),
                                     block_rows, pool_rows, intermediate, clamp, static_cast<uint8_t*>(act_packed),
                                     static_cast<uint8_t*>(act_scales), static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_return_rows(const void* out_pool, const void* pool_of_recv, const void* totals, int capacity,
                                      int hidden, void* return_rows, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_return_rows(out_pool, static_cast<const int*>(pool_of_recv), static_cast<const int*>(totals),
                                    capacity, hidden, return_rows, static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_reduce(const void* returned, const void* send_pos, int tokens, int topk, int hidden, void* y,
                                 const void* ids, int experts, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_reduce(returned, static_cast<const int*>(send_pos), tokens, topk, hidden, y,
                               static_cast<const long long*>(ids), experts, static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_gemm_host_static(int M, int N, int K, const void* A, const void* B, const void* SFA,
                                       const void* SFB, void* C, float alpha, void* stream_) {
    return guarded([&] {
        using nvfp4_b200::cuda_check;
        if (!A || !B || !SFA || !SFB || !C) throw std::invalid_argument("gemm_host_static: null pointer");
        if (M <= 0 || N <= 0 || K <= 0 || M % 128 || N % 128 || K % 64)
            throw std::invalid_argument("gemm_host_static: M, N multiples of 128 and K a multiple of 64 are required");
        if (M > STATIC_MAX_M || N > STATIC_MAX_N || K > STATIC_MAX_K)
            throw std::invalid_argument("gemm_host_static: shape " + std::to_string(M) + "x" + std::to_string(N) + "x" +
                                        std::to_string(K) + " exceeds the built-in staging (M <= " +
                                        std::to_string(STATIC_MAX_M) + ", N <= " + std::to_string(STATIC_MAX_N) +
                                        ", K <= " + std::to_string(STATIC_MAX_K) + "); use gpu_kernels_nvfp4_gemm_host");
        nvfp4_b200::require_sm100();
        auto stream = static_cast<cudaStream_t>(stream_);
        unsigned char* base = static_stage_base();
        uint8_t* dA = base + STATIC_OFF_A;
        uint8_t* dB = base + STATIC_OFF_B;
        uint8_t* dSFA = base + STATIC_OFF_SFA;
        uint8_t* dSFB = base + STATIC_OFF_SFB;
        __half* dC = reinterpret_cast<__half*>(base + STATIC_OFF_C);
        const size_t a_bytes = size_t(M) * K / 2, b_bytes = size_t(N) * K / 2;
        const size_t sfa_bytes = size_t(M) * K / 16, sfb_bytes = size_t(N) * K / 16, c_bytes = size_t(M) * N * 2;
        // One caller at a time: every call uses the same array, so two calls in flight would overwrite
        // each other's operands. Nothing in the array has to start at zero (operands and C are fully
        // overwritten), so nothing is cleared.
        std::lock_guard<std::mutex> hold(g_host_lock);
        gpu_kernels::Nvfp4Params params{};
        const gpu_kernels::Nvfp4Implementation impl = gpu_kernels::nvfp4_sm100_implementation();
        impl.prepare(params, dA, dB, dSFA, dSFB, M, N, K, stream);
        params.alpha = alpha;
        cuda_check(cudaMemcpyAsync(dA, A, a_bytes, cudaMemcpyHostToDevice, stream));
        cuda_check(cudaMemcpyAsync(dB, B, b_bytes, cudaMemcpyHostToDevice, stream));
        cuda_check(cudaMemcpyAsync(dSFA, SFA, sfa_bytes, cudaMemcpyHostToDevice, stream));
        cuda_check(cudaMemcpyAsync(dSFB, SFB, sfb_bytes, cudaMemcpyHostToDevice, stream));
        impl.launch(params, dC, stream);
        cuda_check(cudaMemcpyAsync(C, dC, c_bytes, cudaMemcpyDeviceToHost, stream));
        cuda_check(cudaStreamSynchronize(stream));
    });
}

int gpu_kernels_nvfp4_moe_pack_peer(const void* xq, const void* xs, const void* ids, const void* weights, int tokens,
                                    int topk, int hidden, int world, int local_experts, const void* peer_offset,
                                    void* cursor, void* const* peer_recv, int recv_capacity, void* error, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_pack_peer(static_cast<const uint8_t*>(xq), static_cast<const uint8_t*>(xs),
                                  static_cast<const long long*>(ids), static_cast<const float*>(weights), tokens, topk,
                                  hidden, world, local_experts, static_cast<const int*>(peer_offset),
                                  static_cast<int*>(cursor), peer_recv, recv_capacity, static_cast<int*>(error),
                                  static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_return_peer(const void* out_pool, const void* recv_rows, const void* pool_of_recv,
                                      const void* totals, const void* seg_src_offset, int world, int local_experts,
                                      int hidden, int recv_capacity, void* const* peer_slots, int slot_capacity,
                                      void* error, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_return_peer(out_pool, static_cast<const uint8_t*>(recv_rows), static_cast<const int*>(pool_of_recv),
                                    static_cast<const int*>(totals), static_cast<const int*>(seg_src_offset), world,
                                    local_experts, hidden, recv_capacity, peer_slots, slot_capacity,
                                    static_cast<int*>(error), static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

int gpu_kernels_nvfp4_moe_quantise_route(const void* x_bf16, const void* ids, const void* weights, int tokens, int topk,
                                         int hidden, int experts, const void* offsets, void* cursor, void* const* peer_recv,
                                         void* const* peer_meta, int world, int local_experts, int recv_capacity, void* error,
                                         void* pool_packed, void* pool_scales, void* pool_weight, void* route_row, void* stream) {
    return guarded([&] {
        nvfp4_b200::moe_quantise_route(x_bf16, static_cast<const long long*>(ids), static_cast<const float*>(weights), tokens,
                                       topk, hidden, experts, static_cast<const int*>(offsets), static_cast<int*>(cursor),
                                       peer_recv, peer_meta, world, local_experts, recv_capacity, static_cast<int*>(error),
                                       static_cast<uint8_t*>(pool_packed), static_cast<uint8_t*>(pool_scales),
                                       static_cast<float*>(pool_weight), static_cast<int*>(route_row),
                                       static_cast<cudaStream_t>(stream));
    });
}

int gpu_kernels_nvfp4_peer_state_bytes(int world, int max_ints, size_t* bytes) {
    return guarded([&] {
        if (!bytes) throw std::invalid_argument("peer_state_bytes: null result pointer");
        *bytes = nvfp4_b200::peer_state_bytes(world, max_ints);
    });
}

int gpu_kernels_nvfp4_peer_exchange(void* own, const void* peers_device, int world, int rank, const void* payload, int ints,
                                    int max_ints, void* out, void* stream) {
    return guarded([&] {
        nvfp4_b200::peer_exchange(own, static_cast<void* const*>(peers_device), world, rank, static_cast<const int*>(payload),
                                  ints, max_ints, static_cast<int*>(out), nullptr, 0, static_cast<cudaStream_t>(stream));
    });
}

int gpu_kernels_nvfp4_moe_count_exchange(const void* ids, int routes, int experts, void* own, const void* peers_device, int world,
                                         int rank, int max_ints, void* counts_matrix, void* stream) {
    return guarded([&] {
        if (!ids) throw std::invalid_argument("moe count_exchange: null ids");
        nvfp4_b200::peer_exchange(own, static_cast<void* const*>(peers_device), world, rank, nullptr, experts, max_ints,
                                  static_cast<int*>(counts_matrix), static_cast<const long long*>(ids), routes,
                                  static_cast<cudaStream_t>(stream));
        nvfp4_b200::g_launches.fetch_add(1, std::memory_order_relaxed);
    });
}

/* ---- device buffers that other processes of the box can map (CUDA IPC) ---- */

int gpu_kernels_nvfp4_ipc_alloc(size_t bytes, void** ptr, void* handle64) {
    return guarded([&] {
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
        if (!ptr || !handle64 || bytes == 0) throw std::invalid_argument("ipc_alloc: bad argument");
        void* p = nullptr;
        nvfp4_b200::cuda_check(cudaMalloc(&p, bytes));
        cudaIpcMemHandle_t h{};
        const cudaError_t e = cudaIpcGetMemHandle(&h, p);
        if (e != cudaSuccess) { cudaFree(p); nvfp4_b200::cuda_check(e); }
        nvfp4_b200::cuda_check(cudaMemset(p, 0, bytes));
        std::memcpy(handle64, &h, sizeof(h));
        *ptr = p;
    });
}

int gpu_kernels_nvfp4_ipc_open(const void* handle64, void** ptr) {
    return guarded([&] {
        if (!ptr || !handle64) throw std::invalid_argument("ipc_open: bad argument");
        cudaIpcMemHandle_t h{};
        std::memcpy(&h, handle64, sizeof(h));
        void* p = nullptr;
        nvfp4_b200::cuda_check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        *ptr = p;
    });
}

int gpu_kernels_nvfp4_ipc_close(void* ptr) {
    return guarded([&] { if (ptr) nvfp4_b200::cuda_check(cudaIpcCloseMemHandle(ptr)); });
}

int gpu_kernels_nvfp4_ipc_free(void* ptr) {
    return guarded([&] { if (ptr) nvfp4_b200::cuda_check(cudaFree(ptr)); });
}

int gpu_kernels_nvfp4_plan_placement_misses(void* plan, unsigned* misses) {
    return guarded([&] {
        if (!misses) throw std::invalid_argument("plan_placement_misses: null output");
        *misses = gpu_kernels::nvfp4_placement_misses(as_plan(plan).params);
    });
}

int gpu_kernels_nvfp4_side_route(const unsigned char* unit_side, int units, int tiles, unsigned* route) {
    return guarded([&] {
        if (!unit_side || !route || units < 1 || tiles < 0) throw std::invalid_argument("side_route: bad argument");
        const std::vector<uint8_t> sides(unit_side, unit_side + units);
        const std::vector<uint32_t> r = nvfp4_b200::build_side_route(sides, tiles);
        std::memcpy(route, r.data(), r.size() * sizeof(uint32_t));
    });
}

int gpu_kernels_nvfp4_l2_census(unsigned* cycles_by_sm, int capacity, int* written) {
    return guarded([&] {
        if (!cycles_by_sm || !written) throw std::invalid_argument("l2_census: null output");
        int device = 0;
        nvfp4_b200::cuda_check(cudaGetDevice(&device));
        *written = nvfp4_b200::l2_side_census_cycles(device, cycles_by_sm, capacity);
    });
}

const char* gpu_kernels_nvfp4_version(void) { return "nvfp4-b200 0.2 (sm_100a)"; }

unsigned long long gpu_kernels_nvfp4_launch_count(void) {
    return nvfp4_b200::g_launches.load(std::memory_order_relaxed);
}

}  // extern "C"
