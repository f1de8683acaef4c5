// Host runtime behind the C ABI of include/mcep.h.
//
// Counterpart of mooncake-ep/src/mooncake_ep_buffer.cpp (buffer bookkeeping,
// stream/event choreography, launches) and of the symmetric-buffer / IPC part
// of mooncake-transfer-engine/src/transport/device/p2p_device_transport.cpp.
// No RDMA route, no CPU fallback: every path launches the kernels of
// ep_kernels.cu or fails with an error.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <string>
#include <vector>

#include "../../include/mcep.h"
#include "ep_kernels.cuh"

namespace {

thread_local std::string g_error;

int fail(int code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_error = buf;
    return code;
}

#define MCEP_CUDA(expr)                                                              \
    do {                                                                             \
        cudaError_t e_ = (expr);                                                     \
        if (e_ != cudaSuccess)                                                       \
            return fail(MCEP_ERR_CUDA, "Failed: CUDA error %s:%d '%s' (%s)", __FILE__, \
                        __LINE__, cudaGetErrorString(e_), #expr);                    \
    } while (0)

#define MCEP_REQUIRE(cond)                                                              \
    do {                                                                                \
        if (!(cond))                                                                    \
            return fail(MCEP_ERR_INVALID, "Failed: Assertion error %s:%d '%s'", __FILE__, \
                        __LINE__, #cond);                                               \
    } while (0)

constexpr size_t kWorkspaceBytes = 32u << 20;  // as NUM_WORKSPACE_BYTES in the reference
// Front of the symmetric allocation, ahead of the caller-sized data area:
// flags[parity 2][direction 2][MCEP_MAX_EXPERTS] u64.
constexpr size_t kFlagBlock = (size_t)MCEP_MAX_EXPERTS * sizeof(uint64_t);
constexpr size_t kHeaderRegion = 4 * kFlagBlock;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

struct mcep_event {
    cudaEvent_t ev = nullptr;
};

struct mcep_hook {
    std::function<int()> fn;
};

struct mcep_buffer {
    int rank = 0, num_ranks = 1, device = 0, num_sms = 0;
    int64_t num_bytes = 0;
    bool p2p_enabled = true;
    bool all_peers = false;
    bool force_staged = false;
    bool pdl = true;
    bool fuse_layout = true;
    bool one_kernel = true;
    int64_t hard_timeout_ns = 10ll * 1000 * 1000 * 1000;
    char* base = nullptr;            // symmetric allocation: header region + data area
    char* workspace = nullptr;
    int32_t* status = nullptr;       // device words
    void** peer_dev = nullptr;       // device table [R]
    std::vector<void*> peer_host;    // same, host copy
    std::vector<int32_t> available;  // host copy of the availability table
    std::vector<void*> ipc_opened;   // mappings to close
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_a = nullptr, ev_b = nullptr;  // reusable ordering events
    uint32_t seq = 0;                // calls issued so far (dispatch + combine)

    // workspace carve-up (per parity so two calls in flight do not share scratch)
    struct Scratch {
        int32_t *slot, *count, *done, *cdone, *rowmap;
        uint64_t *dres, *cres;  // verdict words of the receive kernels
        unsigned* ticket;
    } scratch[2];
    size_t scratch_entries = 0;  // capacity of slot/rowmap in int32
};

namespace {

struct Geometry {
    int L, RM, ntiles;
    size_t msg_stride;      // staged dispatch message
    size_t dstage_bytes;    // one parity's dispatch staging
    size_t cstage_bytes;    // one parity's combine staging
    size_t parity_bytes;
};

Geometry geometry(int R, int E, int M, int H, bool fp8) {
    Geometry g;
    g.L = E / R;
    g.RM = R * M;
    g.ntiles = (H + mcep::kTileChannels - 1) / mcep::kTileChannels;
    // sized for the larger (bf16) message so the carve-up does not depend on the mode
    (void)fp8;
    g.msg_stride = align_up((size_t)mcep::kHeaderBytes + 2 * (size_t)H, 32);
    g.dstage_bytes = (size_t)E * M * g.msg_stride;
    g.cstage_bytes = (size_t)E * M * 2 * (size_t)H;
    g.parity_bytes = g.dstage_bytes + g.cstage_bytes;
    return g;
}

int64_t to_ns(int64_t timeout_us) { return timeout_us < 0 ? -1 : timeout_us * 1000; }

bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int order_after(cudaStream_t later, cudaStream_t earlier, cudaEvent_t ev) {
    MCEP_CUDA(cudaEventRecord(ev, earlier));
    MCEP_CUDA(cudaStreamWaitEvent(later, ev, 0));
    return MCEP_OK;
}

int check_connected(const mcep_buffer* b) {
    if (b->num_ranks == 1) return MCEP_OK;
    if (!b->all_peers)
        return fail(MCEP_ERR_STATE,
                    "Failed: peers are not mapped (call sync_nvlink_ipc_handles first); this "
                    "library has no fallback path");
    return MCEP_OK;
}

}  // namespace

extern "C" {

const char* mcep_last_error(void) { return g_error.c_str(); }

uint64_t mcep_kernel_launch_count(void) { return mcep::kernel_launch_count(); }

int mcep_set_kernel_timing(int on) {
    mcep::set_kernel_timing(on != 0);
    return MCEP_OK;
}

int mcep_drain_kernel_times(char* out, size_t capacity) {
    MCEP_REQUIRE(out != nullptr && capacity > 0);
    const std::string s = mcep::drain_kernel_times();
    const size_t n = s.size() < capacity - 1 ? s.size() : capacity - 1;
    std::memcpy(out, s.data(), n);
    out[n] = 0;
    return MCEP_OK;
}

uint64_t mcep_get_ep_buffer_size_hint(int M, int hidden, int num_ranks, int num_experts) {
    (void)num_ranks;
    const uint64_t signaling = (uint64_t)num_experts * sizeof(int);
    const uint64_t send_recv = (uint64_t)num_experts * (uint64_t)M * (2 * 16 + (uint64_t)hidden * 2);
    return 4 * signaling + 4 * send_recv;
}

int mcep_buffer_create(int rank, int num_ranks, int64_t num_ep_buffer_bytes, int disable_p2p,
                       mcep_buffer** out) {
    MCEP_REQUIRE(out != nullptr);
    MCEP_REQUIRE(num_ranks >= 1 && num_ranks <= mcep::kMaxRanks && rank >= 0 && rank < num_ranks);
    MCEP_REQUIRE(num_ep_buffer_bytes >= 0);
    auto* b = new mcep_buffer();
    b->rank = rank;
    b->num_ranks = num_ranks;
    b->num_bytes = num_ep_buffer_bytes;
    b->p2p_enabled = !disable_p2p;
    auto cleanup = [&](int code) {
        mcep_buffer_destroy(b);
        return code;
    };
#define CK(expr)                                                                          \
    do {                                                                                  \
        cudaError_t e_ = (expr);                                                          \
        if (e_ != cudaSuccess)                                                            \
            return cleanup(fail(MCEP_ERR_CUDA, "Failed: CUDA error %s:%d '%s' (%s)",      \
                                __FILE__, __LINE__, cudaGetErrorString(e_), #expr));      \
    } while (0)
    CK(cudaGetDevice(&b->device));
    CK(cudaDeviceGetAttribute(&b->num_sms, cudaDevAttrMultiProcessorCount, b->device));
    int lo = 0, hi = 0;
    if (cudaDeviceGetStreamPriorityRange(&lo, &hi) != cudaSuccess) {
        cudaGetLastError();
        lo = hi = 0;
    }
    CK(cudaStreamCreateWithPriority(&b->comm_stream, cudaStreamNonBlocking, hi));
    CK(cudaEventCreateWithFlags(&b->ev_a, cudaEventDisableTiming));
    CK(cudaEventCreateWithFlags(&b->ev_b, cudaEventDisableTiming));
    const size_t total = kHeaderRegion + align_up((size_t)num_ep_buffer_bytes, 256);
    CK(cudaMalloc(reinterpret_cast<void**>(&b->base), total));
    CK(cudaMemset(b->base, 0, total));
    CK(cudaMalloc(reinterpret_cast<void**>(&b->workspace), kWorkspaceBytes));
    CK(cudaMemset(b->workspace, 0, kWorkspaceBytes));
    CK(cudaMalloc(reinterpret_cast<void**>(&b->peer_dev), sizeof(void*) * num_ranks));
    b->peer_host.assign(num_ranks, nullptr);
    b->available.assign(num_ranks, 0);
    b->peer_host[rank] = b->base;
    b->available[rank] = 1;
    CK(cudaMemcpy(b->peer_dev, b->peer_host.data(), sizeof(void*) * num_ranks,
                  cudaMemcpyHostToDevice));
    b->all_peers = (num_ranks == 1);
#undef CK
    // workspace: [status 256 B][parity 0 scratch][parity 1 scratch]
    b->status = reinterpret_cast<int32_t*>(b->workspace);
    const size_t small = (size_t)(MCEP_MAX_EXPERTS + 64) * sizeof(int32_t);
    const size_t half = (kWorkspaceBytes - 256) / 2;
    const size_t big = (half - 7 * small - 256) / 2;  // bytes for each of slot / rowmap
    b->scratch_entries = big / sizeof(int32_t);
    for (int par = 0; par < 2; ++par) {
        char* w = b->workspace + 256 + par * half;
        auto& s = b->scratch[par];
        s.ticket = reinterpret_cast<unsigned*>(w);
        w += 256;
        s.count = reinterpret_cast<int32_t*>(w), w += small;
        s.done = reinterpret_cast<int32_t*>(w), w += small;
        s.dres = reinterpret_cast<uint64_t*>(w), w += 2 * small;
        s.cres = reinterpret_cast<uint64_t*>(w), w += 2 * small;
        s.cdone = reinterpret_cast<int32_t*>(w), w += small;
        s.slot = reinterpret_cast<int32_t*>(w), w += big / 256 * 256;
        s.rowmap = reinterpret_cast<int32_t*>(w);
    }
    if (const char* env = std::getenv("MCEP_DISABLE_PDL"))
        if (env[0] == '1') b->pdl = false;
    *out = b;
    return MCEP_OK;
}

int mcep_buffer_destroy(mcep_buffer* b) {
    if (b == nullptr) return MCEP_OK;
    // the caller may have moved to another device since the buffer was created
    int cur = b->device;
    cudaGetDevice(&cur);
    if (cur != b->device) cudaSetDevice(b->device);
    cudaDeviceSynchronize();
    for (void* p : b->ipc_opened) cudaIpcCloseMemHandle(p);
    if (b->base) cudaFree(b->base);
    if (b->workspace) cudaFree(b->workspace);
    if (b->peer_dev) cudaFree(b->peer_dev);
    if (b->ev_a) cudaEventDestroy(b->ev_a);
    if (b->ev_b) cudaEventDestroy(b->ev_b);
    if (b->comm_stream) cudaStreamDestroy(b->comm_stream);
    if (cur != b->device) cudaSetDevice(cur);
    cudaGetLastError();
    delete b;
    return MCEP_OK;
}

int mcep_buffer_ibgda_disabled(const mcep_buffer*) { return 1; }
int mcep_buffer_p2p_enabled(const mcep_buffer* b) { return b && b->p2p_enabled ? 1 : 0; }
int mcep_buffer_is_roce(const mcep_buffer*) { return 0; }
int mcep_buffer_use_fast_path(const mcep_buffer* b) { return b && b->all_peers ? 1 : 0; }

int mcep_buffer_get_ipc_handle(mcep_buffer* b, int32_t* out, int capacity, int* n_written) {
    MCEP_REQUIRE(b != nullptr && n_written != nullptr);
    *n_written = 0;
    if (!b->p2p_enabled) return MCEP_OK;
    MCEP_REQUIRE(out != nullptr && capacity >= MCEP_IPC_HANDLE_INT32S);
    static_assert(sizeof(cudaIpcMemHandle_t) == MCEP_IPC_HANDLE_INT32S * sizeof(int32_t),
                  "handle size");
    cudaIpcMemHandle_t h;
    MCEP_CUDA(cudaIpcGetMemHandle(&h, b->base));
    std::memcpy(out, &h, sizeof(h));
    *n_written = MCEP_IPC_HANDLE_INT32S;
    return MCEP_OK;
}

static int publish_peers(mcep_buffer* b, const int32_t* mask) {
    MCEP_CUDA(cudaMemcpy(b->peer_dev, b->peer_host.data(), sizeof(void*) * b->num_ranks,
                         cudaMemcpyHostToDevice));
    b->all_peers = true;
    for (int r = 0; r < b->num_ranks; ++r) {
        if (mask && mask[r] == 0) continue;
        if (!b->available[r] || b->peer_host[r] == nullptr) b->all_peers = false;
    }
    return MCEP_OK;
}

int mcep_buffer_sync_nvlink_ipc_handles(mcep_buffer* b, const int32_t* handles, int n_per_handle,
                                        const int32_t* mask) {
    MCEP_REQUIRE(b != nullptr);
    if (!b->p2p_enabled) return MCEP_OK;
    MCEP_REQUIRE(handles != nullptr && n_per_handle >= MCEP_IPC_HANDLE_INT32S);
    MCEP_CUDA(cudaDeviceSynchronize());
    for (void* p : b->ipc_opened) cudaIpcCloseMemHandle(p);
    b->ipc_opened.clear();
    for (int r = 0; r < b->num_ranks; ++r) {
        if (r == b->rank) continue;
        b->peer_host[r] = nullptr;
        b->available[r] = 0;
        if (mask && mask[r] == 0) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + (size_t)r * n_per_handle, sizeof(h));
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            fprintf(stderr, "[mcep] rank %d: cannot map rank %d's buffer: %s\n", b->rank, r,
                    cudaGetErrorString(e));
            continue;
        }
        b->ipc_opened.push_back(p);
        b->peer_host[r] = p;
        b->available[r] = 1;
    }
    return publish_peers(b, mask);
}

int mcep_buffer_local_base(mcep_buffer* b, void** base) {
    MCEP_REQUIRE(b != nullptr && base != nullptr);
    *base = b->base;
    return MCEP_OK;
}

int mcep_buffer_set_peer_bases(mcep_buffer* b, void* const* bases, const int32_t* available) {
    MCEP_REQUIRE(b != nullptr && bases != nullptr);
    for (int r = 0; r < b->num_ranks; ++r) {
        if (r == b->rank) continue;
        b->peer_host[r] = bases[r];
        b->available[r] = (available ? available[r] : 1) && bases[r] != nullptr;
    }
    return publish_peers(b, available);
}

int mcep_buffer_set_option(mcep_buffer* b, const char* name, int64_t value) {
    MCEP_REQUIRE(b != nullptr && name != nullptr);
    if (!std::strcmp(name, "force_staged")) {
        b->force_staged = value != 0;
    } else if (!std::strcmp(name, "hard_timeout_ms")) {
        MCEP_REQUIRE(value > 0);
        b->hard_timeout_ns = value * 1000 * 1000;
    } else if (!std::strcmp(name, "pdl")) {
        b->pdl = value != 0;
    } else if (!std::strcmp(name, "fuse_layout")) {
        b->fuse_layout = value != 0;
    } else if (!std::strcmp(name, "one_kernel")) {
        b->one_kernel = value != 0;
    } else {
        return fail(MCEP_ERR_INVALID, "Failed: unknown option '%s'", name);
    }
    return MCEP_OK;
}

int mcep_buffer_status(mcep_buffer* b, int32_t* out, int n) {
    MCEP_REQUIRE(b != nullptr && out != nullptr && n >= 1 && n <= 64);
    MCEP_CUDA(cudaMemcpy(out, b->status, sizeof(int32_t) * n, cudaMemcpyDeviceToHost));
    return MCEP_OK;
}

// -----------------------------------------------------------------------------
// dispatch
// -----------------------------------------------------------------------------
int mcep_dispatch(mcep_buffer* b, const mcep_dispatch_args* a, mcep_event** out_event,
                  mcep_hook** out_hook) {
    MCEP_REQUIRE(b != nullptr && a != nullptr && out_event != nullptr && out_hook != nullptr);
    *out_event = nullptr;
    *out_hook = nullptr;
    const int R = b->num_ranks, E = a->num_experts, M = a->num_max_dispatch_tokens_per_rank;
    const int T = a->num_tokens, H = a->hidden, K = a->num_topk;
    // checks of mooncake_ep_buffer.cpp:202-251
    MCEP_REQUIRE(E > 0 && E % R == 0 && E <= MCEP_MAX_EXPERTS);
    MCEP_REQUIRE(H > 0 && H % 16 == 0 && H % 128 == 0);
    MCEP_REQUIRE(T >= 0 && T <= M);
    MCEP_REQUIRE(K >= 1 && K <= MCEP_MAX_TOPK);
    MCEP_REQUIRE(!(a->async_finish && a->return_recv_hook));
    MCEP_REQUIRE(a->active_ranks != nullptr);
    MCEP_REQUIRE(T == 0 || (a->x != nullptr && a->topk_idx != nullptr));
    MCEP_REQUIRE(a->packed_recv_x != nullptr && a->packed_recv_count != nullptr);
    MCEP_REQUIRE(a->packed_recv_src_info != nullptr && a->packed_recv_layout_range != nullptr);
    if (a->use_fp8) {
        MCEP_REQUIRE((R * M) % 4 == 0);
        MCEP_REQUIRE(a->packed_recv_x_scales != nullptr);
    }
    MCEP_REQUIRE(aligned(a->x, 32) && aligned(a->packed_recv_x, 32));
    MCEP_REQUIRE((size_t)T * K <= b->scratch_entries);
    if (int rc = check_connected(b)) return rc;

    const bool fp8 = a->use_fp8 != 0;
    const bool direct = (R == 1) && !b->force_staged;
    const Geometry g = geometry(R, E, M, H, fp8);
    if (!direct && 2 * g.parity_bytes > (size_t)b->num_bytes)
        return fail(MCEP_ERR_INVALID,
                    "Failed: Assertion error %s:%d 'layout.total_bytes <= num_ep_buffer_bytes' "
                    "(need %zu, have %lld)",
                    __FILE__, __LINE__, 2 * g.parity_bytes, (long long)b->num_bytes);

    const uint32_t seq = ++b->seq;
    const int par = seq & 1;
    auto& sc = b->scratch[par];
    const size_t data0 = kHeaderRegion + (size_t)par * g.parity_bytes;
    const size_t dflag_off = (size_t)(par * 2 + 0) * kFlagBlock;

    cudaStream_t compute = reinterpret_cast<cudaStream_t>(a->compute_stream);
    // Without a hook or an event the caller's stream has to wait for the result
    // anyway, so the kernels go straight onto it; `async_finish` runs them on
    // the communication stream behind everything queued on the caller's stream.
    cudaStream_t stream = a->async_finish ? b->comm_stream : compute;
    if (a->async_finish)
        if (int rc = order_after(stream, compute, b->ev_a)) return rc;

    mcep::LaunchCtx first{stream, b->num_sms, false};
    mcep::LaunchCtx next{stream, b->num_sms, b->pdl};

    // (the in-kernel layout keeps three E-sized tables in shared memory)
    const bool fused = mcep::dispatch_send_can_fuse_layout(T, K, H, b->num_sms) && b->fuse_layout &&
                       E <= 2048;
    if (!fused) {
        mcep::LayoutParams lp = {};
        lp.topk_idx = a->topk_idx;
        lp.T = T, lp.K = K, lp.E = E, lp.R = R;
        lp.count = sc.count, lp.slot = sc.slot, lp.done = sc.done, lp.ticket = sc.ticket;
        if (direct) {
            lp.recv_count = a->packed_recv_count;
            lp.layout_range = a->packed_recv_layout_range;
        }
        MCEP_CUDA(mcep::launch_layout(lp, first));
    }

    mcep::DispatchSendParams sp = {};
    sp.x = a->x, sp.topk_idx = a->topk_idx, sp.slot = sc.slot, sp.count = sc.count;
    sp.done = sc.done, sp.active_ranks = a->active_ranks, sp.peer_base = b->peer_dev;
    sp.T = T, sp.K = K, sp.E = E, sp.R = R, sp.M = M, sp.H = H, sp.rank = b->rank;
    sp.use_fp8 = fp8, sp.fused = fused;
    sp.stage_off = data0, sp.flag_off = dflag_off, sp.msg_stride = g.msg_stride;
    sp.seq = seq, sp.status = b->status;
    sp.direct = direct, sp.recv_x = a->packed_recv_x, sp.recv_scales = a->packed_recv_x_scales;
    sp.recv_src_info = a->packed_recv_src_info;
    sp.recv_count = a->packed_recv_count, sp.layout_range = a->packed_recv_layout_range;

    // receive phase, now or from the hook
    mcep::DispatchRecvParams pp = {};
    pp.w.flags = reinterpret_cast<const uint64_t*>(b->base + dflag_off);
    pp.w.resolved = sc.dres, pp.w.active_ranks = a->active_ranks, pp.w.seq = seq;
    pp.w.timeout_ns = to_ns(a->timeout_us), pp.w.hard_timeout_ns = b->hard_timeout_ns;
    pp.w.status = b->status;
    pp.stage = b->base + data0;
    pp.L = g.L, pp.R = R, pp.M = M, pp.H = H, pp.use_fp8 = fp8;
    pp.expected_rows = T * K > 64 ? T * K : 64;
    pp.msg_stride = g.msg_stride, pp.recv_x = a->packed_recv_x;
    pp.recv_scales = a->packed_recv_x_scales, pp.recv_src_info = a->packed_recv_src_info;
    pp.recv_count = a->packed_recv_count, pp.layout_range = a->packed_recv_layout_range;

    const bool pdl = b->pdl;
    const int num_sms = b->num_sms;
    // Small batches in a group, no hook: both phases in one launch.
    const bool one_kernel = fused && !direct && !a->return_recv_hook && b->one_kernel &&
                            mcep::call_can_be_one_kernel(T, K, H, num_sms);
    if (one_kernel) {
        cudaError_t e1 = mcep::launch_dispatch_one_kernel(sp, pp, first);
        if (e1 == cudaErrorInvalidConfiguration) {
            cudaGetLastError();  // would not be resident at once on this device: two launches
            MCEP_CUDA(mcep::launch_dispatch_send(sp, first));
            MCEP_CUDA(mcep::launch_dispatch_recv(pp, next));
        } else {
            MCEP_CUDA(e1);
        }
    } else {
        MCEP_CUDA(mcep::launch_dispatch_send(sp, fused ? first : next));
    }
    auto recv = [=](cudaStream_t s, bool chained) -> int {
        if (direct || one_kernel) return MCEP_OK;
        mcep::LaunchCtx c0{s, num_sms, chained && pdl};
        MCEP_CUDA(mcep::launch_dispatch_recv(pp, c0));
        return MCEP_OK;
    };

    if (a->return_recv_hook) {
        auto* h = new mcep_hook();
        h->fn = [=]() { return recv(compute, false); };
        *out_hook = h;
        return MCEP_OK;
    }
    if (int rc = recv(stream, true)) return rc;
    if (a->async_finish) {
        auto* ev = new mcep_event();
        if (cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventRecord(ev->ev, stream) != cudaSuccess) {
            delete ev;
            return fail(MCEP_ERR_CUDA, "Failed: CUDA error creating the completion event");
        }
        *out_event = ev;
    }
    return MCEP_OK;
}

// -----------------------------------------------------------------------------
// combine
// -----------------------------------------------------------------------------
int mcep_combine(mcep_buffer* b, const mcep_combine_args* a, mcep_event** out_event,
                 mcep_hook** out_hook) {
    MCEP_REQUIRE(b != nullptr && a != nullptr && out_event != nullptr && out_hook != nullptr);
    *out_event = nullptr;
    *out_hook = nullptr;
    const int R = b->num_ranks, E = a->num_experts, M = a->num_max_dispatch_tokens_per_rank;
    const int T = a->num_combined_tokens, H = a->hidden, K = a->num_topk;
    // checks of mooncake_ep_buffer.cpp:351-367
    MCEP_REQUIRE(E > 0 && E % R == 0 && E <= MCEP_MAX_EXPERTS);
    MCEP_REQUIRE(a->num_local_experts == E / R);
    MCEP_REQUIRE(H > 0 && H % 16 == 0 && H % 128 == 0);
    MCEP_REQUIRE(T >= 0 && T <= M);
    MCEP_REQUIRE(K >= 1 && K <= MCEP_MAX_TOPK);
    MCEP_REQUIRE(!(a->async_finish && a->return_recv_hook));
    MCEP_REQUIRE(T == 0 || (a->x != nullptr && a->topk_idx != nullptr && a->topk_weights != nullptr));
    MCEP_REQUIRE(a->src_info != nullptr && a->layout_range != nullptr);
    MCEP_REQUIRE(a->active_ranks != nullptr);
    MCEP_REQUIRE(T == 0 || a->combined_x != nullptr);
    if (a->zero_copy)
        return fail(MCEP_ERR_INVALID,
                    "Failed: zero-copy combine is not supported; pass the expert output tensor "
                    "with zero_copy=False");
    MCEP_REQUIRE(aligned(a->x, 32) && aligned(a->combined_x, 32));
    MCEP_REQUIRE((size_t)T * K <= b->scratch_entries);
    if (int rc = check_connected(b)) return rc;

    const bool direct = (R == 1) && !b->force_staged;
    const Geometry g = geometry(R, E, M, H, false);
    if (!direct && 2 * g.parity_bytes > (size_t)b->num_bytes)
        return fail(MCEP_ERR_INVALID,
                    "Failed: Assertion error %s:%d 'layout.total_bytes <= num_ep_buffer_bytes' "
                    "(need %zu, have %lld)",
                    __FILE__, __LINE__, 2 * g.parity_bytes, (long long)b->num_bytes);

    const uint32_t seq = ++b->seq;
    const int par = seq & 1;
    auto& sc = b->scratch[par];
    const size_t cstage_off = kHeaderRegion + (size_t)par * g.parity_bytes + g.dstage_bytes;
    const size_t cflag_off = (size_t)(par * 2 + 1) * kFlagBlock;

    cudaStream_t compute = reinterpret_cast<cudaStream_t>(a->compute_stream);
    cudaStream_t stream = a->async_finish ? b->comm_stream : compute;
    if (a->async_finish)
        if (int rc = order_after(stream, compute, b->ev_a)) return rc;
    mcep::LaunchCtx first{stream, b->num_sms, false};

    // small single-rank batches: the reduce kernel finds the rows in the handle itself
    const bool search = direct && (long long)T * K <= 4096;
    if (direct && !search) {
        mcep::CombineInvertParams ip = {};
        ip.src_info = a->src_info, ip.layout_range = a->layout_range, ip.topk_idx = a->topk_idx;
        ip.L = g.L, ip.R = R, ip.M = M, ip.T = T, ip.K = K, ip.rank = b->rank;
        ip.rowmap = sc.rowmap, ip.status = b->status;
        MCEP_CUDA(mcep::launch_combine_invert(ip, first));
    }
    mcep::CombineSendParams sp = {};
    sp.x = a->x, sp.src_info = a->src_info, sp.layout_range = a->layout_range;
    sp.active_ranks = a->active_ranks, sp.peer_base = b->peer_dev, sp.done = sc.cdone;
    sp.L = g.L, sp.R = R, sp.M = M, sp.H = H, sp.rank = b->rank;
    sp.stage_off = cstage_off, sp.flag_off = cflag_off, sp.seq = seq, sp.status = b->status;
    const bool one_kernel = !direct && !a->return_recv_hook && b->one_kernel &&
                            mcep::call_can_be_one_kernel(T, K, H, b->num_sms);
    if (!direct && !one_kernel) MCEP_CUDA(mcep::launch_combine_send(sp, first));

    mcep::CombineReduceParams rp = {};
    rp.topk_idx = a->topk_idx, rp.topk_weights = a->topk_weights, rp.active_ranks = a->active_ranks;
    rp.T = T, rp.K = K, rp.E = E, rp.L = g.L, rp.M = M, rp.H = H;
    rp.w.flags = reinterpret_cast<const uint64_t*>(b->base + cflag_off);
    rp.w.resolved = sc.cres, rp.w.active_ranks = a->active_ranks, rp.w.seq = seq;
    rp.w.timeout_ns = to_ns(a->timeout_us), rp.w.hard_timeout_ns = b->hard_timeout_ns;
    rp.w.status = b->status;
    rp.stage = b->base + cstage_off, rp.direct = direct, rp.x = a->x, rp.rowmap = sc.rowmap;
    rp.RM = g.RM, rp.combined_x = a->combined_x;
    rp.search = search, rp.src_info = a->src_info, rp.layout_range = a->layout_range;

    const bool pdl = b->pdl;
    const int num_sms = b->num_sms;
    if (one_kernel) MCEP_CUDA(mcep::launch_combine_one_kernel(sp, rp, first));
    auto recv = [=](cudaStream_t s, bool chained) -> int {
        if (one_kernel) return MCEP_OK;
        mcep::LaunchCtx c0{s, num_sms, chained && pdl && !search};
        MCEP_CUDA(mcep::launch_combine_reduce(rp, c0));
        return MCEP_OK;
    };

    if (a->return_recv_hook) {
        auto* h = new mcep_hook();
        h->fn = [=]() { return recv(compute, false); };
        *out_hook = h;
        return MCEP_OK;
    }
    if (int rc = recv(stream, true)) return rc;
    if (a->async_finish) {
        auto* ev = new mcep_event();
        if (cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventRecord(ev->ev, stream) != cudaSuccess) {
            delete ev;
            return fail(MCEP_ERR_CUDA, "Failed: CUDA error creating the completion event");
        }
        *out_event = ev;
    }
    return MCEP_OK;
}

// -----------------------------------------------------------------------------
// events, hooks
// -----------------------------------------------------------------------------
int mcep_event_create(uint64_t stream, mcep_event** out) {
    MCEP_REQUIRE(out != nullptr);
    auto* ev = new mcep_event();
    cudaError_t e = cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventRecord(ev->ev, reinterpret_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) {
        if (ev->ev) cudaEventDestroy(ev->ev);
        delete ev;
        return fail(MCEP_ERR_CUDA, "Failed: CUDA error '%s' (event create/record)",
                    cudaGetErrorString(e));
    }
    *out = ev;
    return MCEP_OK;
}

int mcep_event_current_stream_wait(mcep_event* ev, uint64_t stream) {
    MCEP_REQUIRE(ev != nullptr && ev->ev != nullptr);
    MCEP_CUDA(cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(stream), ev->ev, 0));
    return MCEP_OK;
}

int mcep_event_synchronize(mcep_event* ev) {
    MCEP_REQUIRE(ev != nullptr && ev->ev != nullptr);
    MCEP_CUDA(cudaEventSynchronize(ev->ev));
    return MCEP_OK;
}

int mcep_event_free(mcep_event* ev) {
    if (ev == nullptr) return MCEP_OK;
    if (ev->ev) cudaEventDestroy(ev->ev);
    delete ev;
    return MCEP_OK;
}

int mcep_hook_run(mcep_hook* h) {
    MCEP_REQUIRE(h != nullptr && h->fn);
    return h->fn();
}

int mcep_hook_free(mcep_hook* h) {
    delete h;
    return MCEP_OK;
}

// -----------------------------------------------------------------------------
// routing layout, standalone
// -----------------------------------------------------------------------------
size_t mcep_routing_layout_scratch_bytes(void) { return 256; }

int mcep_routing_layout(const int64_t* topk_idx, int T, int K, int E, int R, int32_t* count,
                        int32_t* rank_count, int32_t* expert_prefix, int32_t* slot, void* scratch,
                        uint64_t stream) {
    MCEP_REQUIRE(T >= 0 && K >= 1 && K <= MCEP_MAX_TOPK && E > 0 && R >= 1 && E % R == 0);
    MCEP_REQUIRE(T == 0 || topk_idx != nullptr);
    MCEP_REQUIRE(count != nullptr && slot != nullptr && scratch != nullptr);
    int dev = 0, sms = 0;
    MCEP_CUDA(cudaGetDevice(&dev));
    MCEP_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    mcep::LayoutParams lp = {};
    lp.topk_idx = topk_idx, lp.T = T, lp.K = K, lp.E = E, lp.R = R;
    lp.count = count, lp.slot = slot, lp.rank_count = rank_count, lp.expert_prefix = expert_prefix;
    lp.ticket = reinterpret_cast<unsigned*>(scratch);
    mcep::LaunchCtx ctx{reinterpret_cast<cudaStream_t>(stream), sms, false};
    MCEP_CUDA(mcep::launch_layout(lp, ctx));
    return MCEP_OK;
}

}  // extern "C"
