// An entry point for callers that must not allocate device memory.
//
// Some users of this library run where cudaMalloc is off limits: inside a
// region that a memory pool or a capture-safe allocator owns, in a real-time
// serving loop that forbids allocator calls once warm, or in a host process
// that hands out a fixed device-memory budget and treats any further
// allocation as a fault. `mcep_buffer_create` allocates (symmetric buffer,
// workspace), so those callers could not use the library at all for the one
// case that needs no peer memory: the single-rank combine.
//
// `mcep_combine_single_rank_static` is that case with its scratch - the
// (token, k) -> packed-row map that `ep_combine_invert_kernel` fills and
// `ep_combine_reduce_direct_kernel` reads - in a file-scope device array instead of a
// cudaMalloc'ed workspace. It calls no cudaMalloc, cudaFree or allocating
// library routine. The array is part of the library image: every GPU that loads
// libmcep.so holds it until the process exits.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/mcep.h"
#include "ep_kernels.cuh"

namespace {

constexpr int kMaxDevices = 64;
constexpr size_t kHeaderBytes = 256;  // [0] int32 "rank 0 is active" = 1, [64] int32 status
constexpr size_t kScratchBytes = kHeaderBytes + (size_t)MCEP_STATIC_MAX_ENTRIES * sizeof(int32_t);

// In host code this name is only a handle for cudaGetSymbolAddress: it is not a
// device address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

struct DeviceSetup {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_static_scratch on this device
    int num_sms = 0;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mu;

thread_local char g_static_error[512];

}  // namespace

extern "C" const char* mcep_static_last_error(void) { return g_static_error; }

#define STATIC_FAIL(code, ...)                                       \
    do {                                                             \
        snprintf(g_static_error, sizeof(g_static_error), __VA_ARGS__); \
        return (code);                                               \
    } while (0)

#define STATIC_CUDA(expr)                                                                   \
    do {                                                                                    \
        cudaError_t e_ = (expr);                                                            \
        if (e_ != cudaSuccess)                                                              \
            STATIC_FAIL(MCEP_ERR_CUDA, "Failed: CUDA error %s:%d '%s' (%s)", __FILE__, __LINE__, \
                        cudaGetErrorString(e_), #expr);                                     \
    } while (0)

extern "C" int mcep_combine_single_rank_static(const void* x, const int64_t* topk_idx,
                                               const float* topk_weights, const int32_t* src_info,
                                               const int64_t* layout_range, int num_experts,
                                               int num_combined_tokens, int hidden, int num_topk,
                                               int num_max_dispatch_tokens_per_rank,
                                               void* combined_x, uint64_t stream) {
    g_static_error[0] = 0;
    const int E = num_experts, T = num_combined_tokens, H = hidden, K = num_topk;
    const int M = num_max_dispatch_tokens_per_rank;
    if (E <= 0 || E > MCEP_MAX_EXPERTS || T < 0 || T > M || H <= 0 || H % 128 != 0 || K < 1 ||
        K > MCEP_MAX_TOPK)
        STATIC_FAIL(MCEP_ERR_INVALID, "Failed: Assertion error: bad shape (E=%d T=%d M=%d H=%d K=%d)", E,
                    T, M, H, K);
    if ((long long)T * K > MCEP_STATIC_MAX_ENTRIES)
        STATIC_FAIL(MCEP_ERR_INVALID,
                    "Failed: num_combined_tokens * num_topk = %lld exceeds the static scratch of %d "
                    "entries (MCEP_STATIC_MAX_ENTRIES); use mcep_combine with a buffer instead",
                    (long long)T * K, MCEP_STATIC_MAX_ENTRIES);
    if (T > 0 && (!x || !topk_idx || !topk_weights || !combined_x))
        STATIC_FAIL(MCEP_ERR_INVALID, "Failed: Assertion error: null tensor pointer");
    if (!src_info || !layout_range)
        STATIC_FAIL(MCEP_ERR_INVALID, "Failed: Assertion error: null handle pointer");
    if (reinterpret_cast<uintptr_t>(x) % 32 || reinterpret_cast<uintptr_t>(combined_x) % 32)
        STATIC_FAIL(MCEP_ERR_INVALID, "Failed: Assertion error: x and combined_x must be 32-byte aligned");

    int dev = 0;
    STATIC_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) STATIC_FAIL(MCEP_ERR_INVALID, "Failed: device index %d", dev);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    DeviceSetup setup;
    {
        std::lock_guard<std::mutex> lk(g_setup_mu);
        if (!g_setup[dev].ready) {
            // Once per device, with that device current: turn the symbol into
            // this device's address of the array and write the two constants.
            void* p = nullptr;
            STATIC_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
            int sms = 0;
            STATIC_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
            const int32_t one = 1, zero = 0;
            STATIC_CUDA(cudaMemcpy(p, &one, sizeof(one), cudaMemcpyHostToDevice));
            STATIC_CUDA(cudaMemcpy(static_cast<unsigned char*>(p) + 64, &zero, sizeof(zero),
                                   cudaMemcpyHostToDevice));
            g_setup[dev].scratch = static_cast<unsigned char*>(p);
            g_setup[dev].num_sms = sms;
            g_setup[dev].ready = true;
        }
        setup = g_setup[dev];
    }
    int32_t* active = reinterpret_cast<int32_t*>(setup.scratch);
    int32_t* status = reinterpret_cast<int32_t*>(setup.scratch + 64);
    int32_t* rowmap = reinterpret_cast<int32_t*>(setup.scratch + kHeaderBytes);
    if (T == 0) return MCEP_OK;

    // The array keeps the previous call's contents: entries this call's handle
    // does not cover must read as "no row" (-1), not as a stale row.
    STATIC_CUDA(cudaMemsetAsync(rowmap, 0xFF, (size_t)T * K * sizeof(int32_t), s));

    mcep::LaunchCtx ctx{s, setup.num_sms, false};
    mcep::CombineInvertParams ip = {};
    ip.src_info = src_info, ip.layout_range = layout_range, ip.topk_idx = topk_idx;
    ip.L = E, ip.R = 1, ip.M = M, ip.T = T, ip.K = K, ip.rank = 0;
    ip.rowmap = rowmap, ip.status = status;
    STATIC_CUDA(mcep::launch_combine_invert(ip, ctx));

    mcep::DirectCombineParams rp = {};
    rp.topk_idx = topk_idx, rp.topk_weights = topk_weights, rp.active_ranks = active;
    rp.T = T, rp.K = K, rp.E = E, rp.M = M, rp.H = H;
    rp.x = x, rp.rowmap = rowmap, rp.search = 0;
    rp.src_info = src_info, rp.layout_range = layout_range;
    rp.combined_x = combined_x;
    STATIC_CUDA(mcep::launch_direct_combine(rp, ctx));
    return MCEP_OK;
}

// The kernels record anomalies of the handle they were given (a row or a token
// index out of range) in a word of the static array instead of trapping. This
// reads that word for the current device and clears it; like the entry point
// above it allocates nothing. A call that has not run on this device yet reads
// as 0.
extern "C" int mcep_static_status(int32_t* out) {
    g_static_error[0] = 0;
    if (out == nullptr) STATIC_FAIL(MCEP_ERR_INVALID, "Failed: Assertion error: null output pointer");
    *out = 0;
    int dev = 0;
    STATIC_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) STATIC_FAIL(MCEP_ERR_INVALID, "Failed: device index %d", dev);
    DeviceSetup setup;
    {
        std::lock_guard<std::mutex> lk(g_setup_mu);
        setup = g_setup[dev];
    }
    if (!setup.ready) return MCEP_OK;
    // plain cudaMemcpy: ordered after the kernels of earlier calls on any
    // blocking stream; callers on non-blocking streams synchronise first
    STATIC_CUDA(cudaDeviceSynchronize());
    STATIC_CUDA(cudaMemcpy(out, setup.scratch + 64, sizeof(int32_t), cudaMemcpyDeviceToHost));
    if (*out != 0) {
        const int32_t zero = 0;
        STATIC_CUDA(cudaMemcpy(setup.scratch + 64, &zero, sizeof(zero), cudaMemcpyHostToDevice));
    }
    return MCEP_OK;
}
