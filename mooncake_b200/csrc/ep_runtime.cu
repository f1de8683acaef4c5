// Host runtime behind the C ABI of include/mcep.h.
//
// Counterpart of mooncake-ep/src/mooncake_ep_buffer.cpp (buffer bookkeeping,
// stream/event choreography, launches) and of the symmetric-buffer / IPC part
// of mooncake-transfer-engine/src/transport/device/p2p_device_transport.cpp.
// No RDMA route, no CPU fallback: every path launches the kernels of
// ep_kernels.cu or fails with an error.
#include <cuda.h>  // types of the virtual-memory API only; entry points are looked up at run time
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
#include "ep_runtime_internal.h"

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
constexpr size_t kChunkHistBytes = 2u << 20;   // per-chunk histograms of the routing layout (per parity)
// Front of the symmetric allocation, ahead of the caller-sized data area: the
// words ranks write into each other's memory, twice (one set per parity):
//   cnt   [MCEP_MAX_EXPERTS] u64   counts announced to this rank (owner side)
//   beg   [MCEP_MAX_EXPERTS] u64   first rows answered to this rank (sender side)
//   dflag [64] u64, cflag [64] u64 payload / combine-input words
// and, at the very end, the two call counters this rank last published (read
// by its peers when the group's membership is refreshed).
constexpr size_t kWordBlock = (size_t)MCEP_MAX_EXPERTS * sizeof(uint64_t);
constexpr size_t kHeaderParity = 128u << 10;
constexpr size_t kHeaderRegion = 2 * kHeaderParity;
constexpr size_t kPubSeqOff = kHeaderRegion - 256;
constexpr size_t kBarrierOff = kHeaderParity - 1024;  // [64] u64 barrier words (free tail of parity 0's block)
static_assert(2 * kWordBlock + 2 * 64 * sizeof(uint64_t) <= kHeaderParity - 1024, "header layout");

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace

// ---- fabric-handle allocation (the reference's MC_USE_NVLINK_IPC=0 mode) -----------
// mooncake-transfer-engine/src/transport/device/p2p_device_transport.cpp:40-60
// (when it applies), :271-386 (allocation), :414-431 (export), :520-580 (import).
// The symmetric buffer is then a cuMemCreate allocation that is exported as a
// CUmemFabricHandle instead of a cudaIpcMemHandle_t. The driver entry points are
// resolved through the runtime, so the library has no link-time dependency on
// the driver and still loads on a machine without one.
namespace {

struct DriverApi {
    CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
    CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                           CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                          unsigned long long) = nullptr;
    CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                           unsigned long long) = nullptr;
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                             CUmemAllocationHandleType) = nullptr;
    bool ok = false;
};

template <typename F>
bool driver_symbol(const char* name, F* fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult st;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &st) != cudaSuccess ||
        st != cudaDriverEntryPointSuccess || p == nullptr) {
        cudaGetLastError();
        return false;
    }
    *fn = reinterpret_cast<F>(p);
    return true;
}

const DriverApi& driver_api() {
    static DriverApi api = [] {
        DriverApi a;
        a.ok = driver_symbol("cuDeviceGet", &a.DeviceGet) &&
               driver_symbol("cuDeviceGetAttribute", &a.DeviceGetAttribute) &&
               driver_symbol("cuMemGetAllocationGranularity", &a.MemGetAllocationGranularity) &&
               driver_symbol("cuMemCreate", &a.MemCreate) && driver_symbol("cuMemRelease", &a.MemRelease) &&
               driver_symbol("cuMemAddressReserve", &a.MemAddressReserve) &&
               driver_symbol("cuMemAddressFree", &a.MemAddressFree) &&
               driver_symbol("cuMemMap", &a.MemMap) && driver_symbol("cuMemUnmap", &a.MemUnmap) &&
               driver_symbol("cuMemSetAccess", &a.MemSetAccess) &&
               driver_symbol("cuMemExportToShareableHandle", &a.MemExportToShareableHandle) &&
               driver_symbol("cuMemImportFromShareableHandle", &a.MemImportFromShareableHandle);
        return a;
    }();
    return api;
}

// MC_USE_NVLINK_IPC=0 asks for fabric handles; they are used only where every
// visible device supports them (the reference's supportFabricMem).
bool fabric_requested_and_supported() {
    const char* env = std::getenv("MC_USE_NVLINK_IPC");
    if (env == nullptr || std::strcmp(env, "0") != 0) return false;
    const DriverApi& d = driver_api();
    if (!d.ok) return false;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        return false;
    }
    for (int i = 0; i < n; ++i) {
        CUdevice dev;
        int supported = 0;
        if (d.DeviceGet(&dev, i) != CUDA_SUCCESS ||
            d.DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED, dev) !=
                CUDA_SUCCESS ||
            !supported)
            return false;
    }
    return true;
}

struct FabricMapping {  // one mapped allocation: this rank's own, or an imported peer's
    CUdeviceptr va = 0;
    size_t size = 0;
    CUmemGenericAllocationHandle handle = 0;
};

bool fabric_map(const DriverApi& d, CUmemGenericAllocationHandle handle, size_t size, size_t align,
                int device, FabricMapping* out) {
    CUdeviceptr va = 0;
    if (d.MemAddressReserve(&va, size, align, 0, 0) != CUDA_SUCCESS) return false;
    if (d.MemMap(va, size, 0, handle, 0) != CUDA_SUCCESS) {
        d.MemAddressFree(va, size);
        return false;
    }
    CUmemAccessDesc acc = {};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    if (d.MemSetAccess(va, size, &acc, 1) != CUDA_SUCCESS) {
        d.MemUnmap(va, size);
        d.MemAddressFree(va, size);
        return false;
    }
    out->va = va, out->size = size, out->handle = handle;
    return true;
}

void fabric_unmap(const DriverApi& d, FabricMapping* m) {
    if (m->va) {
        d.MemUnmap(m->va, m->size);
        d.MemAddressFree(m->va, m->size);
    }
    if (m->handle) d.MemRelease(m->handle);
    *m = FabricMapping();
}

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
    bool fabric = false;             // the buffer is a cuMemCreate allocation shared through fabric handles
    FabricMapping own;               // fabric mode: this rank's allocation
    std::vector<FabricMapping> fabric_peers;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ev_a = nullptr, ev_b = nullptr;  // reusable ordering events
    uint32_t dseq = 0, cseq = 0;     // dispatch / combine calls issued so far
    uint32_t barrier_epoch = 0;      // barriers issued so far

    // workspace carve-up (per parity so two calls in flight do not share scratch)
    struct Scratch {
        int32_t *slot, *count, *rowmap, *rowmap_inv, *chunk_hist;
        uint64_t *res_cnt, *res_dflag, *res_cflag;  // verdict words
        unsigned *layout_ticket, *send_ticket, *publish_ticket;
    } scratch[2];
    size_t scratch_entries = 0;  // capacity of slot/rowmap in int32

    // In-process groups: calls are prepared but not launched until
    // mcep_launch_deferred starts all ranks' work in one launch.
    // Graph mode: the sequence number of the next call of each kind and parity
    // lives in device memory ([0..1] dispatch, [2..3] combine; parity = index & 1),
    // so that a captured call can be replayed (see mcep_buffer_set_option).
    bool graph_mode = false;
    uint32_t* dev_next_seq = nullptr;
    bool defer = false;
    struct Pending {
        int kind = 0;                // 0 none, 1 dispatch, 2 combine
        int phases = 0;              // dispatch: 1 send / 3 send + receive; combine: 1 publish / 3 both
        bool then_second = false;    // launch the second phase right after (no hook was asked for)
        cudaStream_t stream = nullptr;
        mcep::GroupDispatchParams d;
        mcep::GroupCombineParams c;
    } pending;
    std::function<int()> after_deferred;  // run once the prepared dispatch has been launched
    bool chain_first_once = false;        // see allow_chained_first_launch

    // what combine needs to know about the dispatch call a handle came from
    struct DispatchRecord {
        const void* key = nullptr;  // the handle's src_info tensor
        uint32_t seq = 0;
        uint64_t stamp = 0;         // host-side order of the dispatch calls (the newer record wins)
        int T = 0, K = 0, E = 0, M = 0, H = 0;
    } record[2];
    uint64_t record_clock = 0;
};

namespace {

// Data area of one parity: [dispatch area | combine input].
//   dispatch area  E*M*(32 + 2H) bytes: receive rows [L][R*M][H or 2H], then the
//                  side messages [L][R*M][meta_stride]
//   combine input  [L][R*M][2H]
// Twice that never exceeds the reference's size hint 16E + 4*E*M*(32 + 2H).
struct Geometry {
    int L, RM, ntiles;
    int row_bytes, meta_stride;
    size_t darea_bytes, cin_bytes, parity_bytes;
    size_t meta_off;  // inside the dispatch area
};

Geometry geometry(int R, int E, int M, int H, bool fp8) {
    Geometry g;
    g.L = E / R;
    g.RM = R * M;
    g.ntiles = (H + mcep::kTileChannels - 1) / mcep::kTileChannels;
    g.row_bytes = H * (fp8 ? 1 : 2);
    g.meta_stride = mcep::kMetaHeaderBytes + (fp8 ? 16 * g.ntiles : 0);
    g.darea_bytes = (size_t)E * M * (32 + 2 * (size_t)H);
    g.cin_bytes = (size_t)E * M * 2 * (size_t)H;
    g.parity_bytes = g.darea_bytes + g.cin_bytes;
    g.meta_off = (size_t)E * M * g.row_bytes;
    return g;
}

int64_t to_ns(int64_t timeout_us) { return timeout_us < 0 ? -1 : timeout_us * 1000; }

// Kernels of one call are chained with programmatic dependent launch - except
// while the stream is being captured into a graph, where plain dependencies are
// recorded.
bool chain_with_pdl(const mcep_buffer* b, cudaStream_t stream);

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

namespace {
bool chain_with_pdl(const mcep_buffer* b, cudaStream_t stream) {
    if (!b->pdl) return false;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return st == cudaStreamCaptureStatusNone;
}
}  // namespace

namespace mcep {

BufferView view_of(mcep_buffer* b) {
    BufferView v;
    v.base = b->base, v.data_off = kHeaderRegion, v.num_bytes = b->num_bytes;
    v.peer_host = b->peer_host.data();
    v.rank = b->rank, v.num_ranks = b->num_ranks, v.num_sms = b->num_sms;
    v.status = b->status, v.comm_stream = b->comm_stream;
    v.group = b->num_ranks > 1 || b->force_staged;
    v.defer = b->defer;
    return v;
}

size_t exchange_bytes(int num_ranks, int num_experts, int M, int hidden) {
    return 2 * geometry(num_ranks, num_experts, M, hidden, false).parity_bytes;
}

void set_after_deferred(mcep_buffer* b, std::function<int()> fn) { b->after_deferred = std::move(fn); }

void allow_chained_first_launch(mcep_buffer* b) { b->chain_first_once = true; }

int report_failure(int code, const char* message) { return fail(code, "%s", message); }

}  // namespace mcep

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
    if (num_ranks > 1 && b->p2p_enabled && fabric_requested_and_supported()) {
        // the reference's fabric mode: a cuMemCreate allocation with a fabric handle
        const DriverApi& d = driver_api();
        CUmemAllocationProp prop = {};
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = b->device;
        prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_FABRIC;
        size_t gran = 0;
        CUmemGenericAllocationHandle h = 0;
        if (d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS &&
            gran > 0) {
            const size_t size = align_up(total, gran);
            if (d.MemCreate(&h, size, &prop, 0) == CUDA_SUCCESS) {
                if (fabric_map(d, h, size, gran, b->device, &b->own)) {
                    b->fabric = true;
                    b->base = reinterpret_cast<char*>(b->own.va);
                } else {
                    d.MemRelease(h);
                }
            }
        }
        if (!b->fabric)
            fprintf(stderr, "[mcep] rank %d: fabric-handle allocation failed, using cudaMalloc + CUDA IPC\n", rank);
    }
    if (!b->fabric) CK(cudaMalloc(reinterpret_cast<void**>(&b->base), total));
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
    b->dev_next_seq = reinterpret_cast<uint32_t*>(b->workspace + 256 + 192);  // beside parity 0's tickets
    const size_t words = (size_t)MCEP_MAX_EXPERTS * sizeof(uint64_t);
    const size_t small = (size_t)(MCEP_MAX_EXPERTS + 64) * sizeof(int32_t);
    const size_t half = (kWorkspaceBytes - 256) / 2;
    const size_t fixed = 256 + small + words + 2 * 64 * sizeof(uint64_t) + kChunkHistBytes;
    const size_t big = ((half - fixed - 1024) / 3) / 256 * 256;  // bytes for each of slot / rowmap / rowmap_inv
    b->scratch_entries = big / sizeof(int32_t);
    for (int par = 0; par < 2; ++par) {
        char* w = b->workspace + 256 + par * half;
        auto& s = b->scratch[par];
        s.layout_ticket = reinterpret_cast<unsigned*>(w);
        s.send_ticket = reinterpret_cast<unsigned*>(w + 64);
        s.publish_ticket = reinterpret_cast<unsigned*>(w + 128);
        w += 256;
        s.count = reinterpret_cast<int32_t*>(w), w += small;
        s.res_cnt = reinterpret_cast<uint64_t*>(w), w += words;
        s.res_dflag = reinterpret_cast<uint64_t*>(w), w += 64 * sizeof(uint64_t);
        s.res_cflag = reinterpret_cast<uint64_t*>(w), w += 64 * sizeof(uint64_t);
        s.chunk_hist = reinterpret_cast<int32_t*>(w), w += kChunkHistBytes;
        s.slot = reinterpret_cast<int32_t*>(w), w += big;
        s.rowmap = reinterpret_cast<int32_t*>(w), w += big;
        s.rowmap_inv = reinterpret_cast<int32_t*>(w);
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
    mcep::elastic_release(b);
    for (void* p : b->ipc_opened) cudaIpcCloseMemHandle(p);
    if (b->fabric) {
        for (auto& m : b->fabric_peers) fabric_unmap(driver_api(), &m);
        fabric_unmap(driver_api(), &b->own);
    } else if (b->base) {
        cudaFree(b->base);
    }
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
int mcep_buffer_uses_fabric_handles(const mcep_buffer* b) { return b && b->fabric ? 1 : 0; }

// The words ranks exchange carry the number of the call they belong to, so all
// ranks of a group must count their calls alike. A rank that sat out some calls
// (masked out, or re-created from scratch) is brought back in step when the
// membership is refreshed: every rank leaves its two counters in its own
// symmetric memory before the handles are exchanged, reads every mapped peer's
// afterwards and continues from the largest.
// Graph mode: the device words are the truth (replayed graphs advance them, the
// host never hears of it). next[par] = sequence number the next call of that
// parity will carry, so the last call made carried max(next[0], next[1]) - 2.
static int read_device_seq(mcep_buffer* b) {
    if (!b->graph_mode) return MCEP_OK;
    uint32_t w[4];
    MCEP_CUDA(cudaMemcpy(w, b->dev_next_seq, sizeof(w), cudaMemcpyDeviceToHost));
    b->dseq = (w[0] > w[1] ? w[0] : w[1]) - 2;
    b->cseq = (w[2] > w[3] ? w[2] : w[3]) - 2;
    return MCEP_OK;
}

static int write_device_seq(mcep_buffer* b) {
    uint32_t w[4];
    const uint32_t d = b->dseq + 1, c = b->cseq + 1;  // the next calls' numbers
    w[d & 1] = d, w[(d + 1) & 1] = d + 1;
    w[2 + (c & 1)] = c, w[2 + ((c + 1) & 1)] = c + 1;
    MCEP_CUDA(cudaMemcpy(b->dev_next_seq, w, sizeof(w), cudaMemcpyHostToDevice));
    return MCEP_OK;
}

static int publish_seq(mcep_buffer* b) {
    if (int rc = read_device_seq(b)) return rc;
    const uint32_t pub[3] = {b->dseq, b->cseq, b->barrier_epoch};
    MCEP_CUDA(cudaMemcpy(b->base + kPubSeqOff, pub, sizeof(pub), cudaMemcpyHostToDevice));
    return MCEP_OK;
}

static int adopt_largest_seq(mcep_buffer* b) {
    uint32_t d = b->dseq, c = b->cseq;
    for (int r = 0; r < b->num_ranks; ++r) {
        if (r == b->rank || !b->available[r] || b->peer_host[r] == nullptr) continue;
        uint32_t pub[3] = {0, 0, 0};
        MCEP_CUDA(cudaMemcpy(pub, static_cast<char*>(b->peer_host[r]) + kPubSeqOff, sizeof(pub),
                             cudaMemcpyDeviceToHost));
        if (pub[0] > d) d = pub[0];
        if (pub[1] > c) c = pub[1];
        if (pub[2] > b->barrier_epoch) b->barrier_epoch = pub[2];  // barriers are counted alike, too
    }
    if (d != b->dseq || c != b->cseq) {
        // handles of calls made before the jump no longer name a known call
        b->record[0] = mcep_buffer::DispatchRecord();
        b->record[1] = mcep_buffer::DispatchRecord();
    }
    b->dseq = d;
    b->cseq = c;
    if (b->graph_mode) return write_device_seq(b);
    return MCEP_OK;
}

int mcep_buffer_get_ipc_handle(mcep_buffer* b, int32_t* out, int capacity, int* n_written) {
    MCEP_REQUIRE(b != nullptr && n_written != nullptr);
    *n_written = 0;
    if (!b->p2p_enabled) return MCEP_OK;
    MCEP_REQUIRE(out != nullptr && capacity >= MCEP_IPC_HANDLE_INT32S);
    static_assert(sizeof(cudaIpcMemHandle_t) == MCEP_IPC_HANDLE_INT32S * sizeof(int32_t),
                  "handle size");
    MCEP_CUDA(cudaDeviceSynchronize());
    if (int rc = publish_seq(b)) return rc;
    if (b->fabric) {
        // [CUmemFabricHandle 64 B | size 8 B] as 18 int32, the reference's serialisation
        // (p2p_device_transport.cpp:61-75); the length tells the importer which kind it is
        MCEP_REQUIRE(capacity >= MCEP_FABRIC_HANDLE_INT32S);
        CUmemFabricHandle fh;
        if (driver_api().MemExportToShareableHandle(&fh, b->own.handle, CU_MEM_HANDLE_TYPE_FABRIC, 0) !=
            CUDA_SUCCESS)
            return fail(MCEP_ERR_CUDA, "Failed: CUDA error %s:%d 'cuMemExportToShareableHandle(FABRIC)'",
                        __FILE__, __LINE__);
        static_assert(sizeof(CUmemFabricHandle) + sizeof(uint64_t) == MCEP_FABRIC_HANDLE_INT32S * sizeof(int32_t),
                      "fabric handle size");
        const uint64_t size = b->own.size;
        std::memcpy(out, &fh, sizeof(fh));
        std::memcpy(reinterpret_cast<char*>(out) + sizeof(fh), &size, sizeof(size));
        *n_written = MCEP_FABRIC_HANDLE_INT32S;
        return MCEP_OK;
    }
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
    return adopt_largest_seq(b);
}

int mcep_buffer_sync_nvlink_ipc_handles(mcep_buffer* b, const int32_t* handles, int n_per_handle,
                                        const int32_t* mask) {
    MCEP_REQUIRE(b != nullptr);
    if (!b->p2p_enabled) return MCEP_OK;
    MCEP_REQUIRE(handles != nullptr && n_per_handle >= MCEP_IPC_HANDLE_INT32S);
    MCEP_CUDA(cudaDeviceSynchronize());
    for (void* p : b->ipc_opened) cudaIpcCloseMemHandle(p);
    b->ipc_opened.clear();
    for (auto& m : b->fabric_peers) fabric_unmap(driver_api(), &m);
    b->fabric_peers.clear();
    if (b->fabric) {
        MCEP_REQUIRE(n_per_handle >= MCEP_FABRIC_HANDLE_INT32S);
        const DriverApi& d = driver_api();
        for (int r = 0; r < b->num_ranks; ++r) {
            if (r == b->rank) continue;
            b->peer_host[r] = nullptr;
            b->available[r] = 0;
            if (mask && mask[r] == 0) continue;
            CUmemFabricHandle fh;
            uint64_t size = 0;
            const char* src = reinterpret_cast<const char*>(handles + (size_t)r * n_per_handle);
            std::memcpy(&fh, src, sizeof(fh));
            std::memcpy(&size, src + sizeof(fh), sizeof(size));
            CUmemGenericAllocationHandle h = 0;
            FabricMapping m;
            if (size == 0 || d.MemImportFromShareableHandle(&h, &fh, CU_MEM_HANDLE_TYPE_FABRIC) != CUDA_SUCCESS) {
                fprintf(stderr, "[mcep] rank %d: cuMemImportFromShareableHandle(FABRIC) failed for rank %d\n",
                        b->rank, r);
                continue;
            }
            if (!fabric_map(d, h, (size_t)size, 0, b->device, &m)) {
                d.MemRelease(h);
                fprintf(stderr, "[mcep] rank %d: cannot map rank %d's fabric allocation\n", b->rank, r);
                continue;
            }
            b->fabric_peers.push_back(m);
            b->peer_host[r] = reinterpret_cast<void*>(m.va);
            b->available[r] = 1;
        }
        return publish_peers(b, mask);
    }
    int device_count = 1;
    if (cudaGetDeviceCount(&device_count) != cudaSuccess || device_count < 1) {
        cudaGetLastError();
        device_count = 1;
    }
    for (int r = 0; r < b->num_ranks; ++r) {
        if (r == b->rank) continue;
        b->peer_host[r] = nullptr;
        b->available[r] = 0;
        if (mask && mask[r] == 0) continue;
        // Rank r runs on device r % device_count of this node (the placement the
        // reference assumes, p2p_device_transport.cpp:591-604): ask the driver
        // whether that device can be reached before mapping its memory. With one
        // visible device per process the question cannot be asked; the mapping
        // call below then decides.
        const int dst_device = r % device_count;
        if (dst_device != b->device) {
            int can_access = 0;
            if (cudaDeviceCanAccessPeer(&can_access, b->device, dst_device) != cudaSuccess) {
                cudaGetLastError();
                can_access = 0;
            }
            if (!can_access) {
                fprintf(stderr, "[mcep] [EP P2P] rank %d (device %d) -> rank %d (device %d): "
                                "canAccessPeer=0\n", b->rank, b->device, r, dst_device);
                continue;
            }
        }
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
    // in-process groups exchange base pointers instead of handles: this is the
    // moment a rank leaves its call counters for its peers
    MCEP_CUDA(cudaDeviceSynchronize());
    return publish_seq(b);
}

int mcep_buffer_set_peer_bases(mcep_buffer* b, void* const* bases, const int32_t* available) {
    MCEP_REQUIRE(b != nullptr && bases != nullptr);
    MCEP_CUDA(cudaDeviceSynchronize());
    for (int r = 0; r < b->num_ranks; ++r) {
        if (r == b->rank) continue;
        b->available[r] = (available ? available[r] : 1) && bases[r] != nullptr;
        b->peer_host[r] = b->available[r] ? bases[r] : nullptr;  // an unavailable rank is never mapped
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
    } else if (!std::strcmp(name, "defer_launch")) {
        b->defer = value != 0;
    } else if (!std::strcmp(name, "graph_mode")) {
        MCEP_CUDA(cudaDeviceSynchronize());
        if (value != 0 && !b->graph_mode) {
            if (int rc = write_device_seq(b)) return rc;
            b->graph_mode = true;
        } else if (value == 0 && b->graph_mode) {
            if (int rc = read_device_seq(b)) return rc;
            b->graph_mode = false;
        }
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

int mcep_buffer_call_counts(mcep_buffer* b, uint32_t* dispatch_calls, uint32_t* combine_calls) {
    MCEP_REQUIRE(b != nullptr && dispatch_calls != nullptr && combine_calls != nullptr);
    if (b->graph_mode) {
        MCEP_CUDA(cudaDeviceSynchronize());
        if (int rc = read_device_seq(b)) return rc;
    }
    *dispatch_calls = b->dseq;
    *combine_calls = b->cseq;
    return MCEP_OK;
}

static bool is_group(const mcep_buffer* b) { return b->num_ranks > 1 || b->force_staged; }

int mcep_buffer_next_recv_x(mcep_buffer* b, int M, int hidden, int num_experts, int use_fp8,
                            void** out, size_t* bytes) {
    MCEP_REQUIRE(b != nullptr && out != nullptr);
    *out = nullptr;
    if (bytes) *bytes = 0;
    if (!is_group(b)) return MCEP_OK;  // a single rank writes the caller's tensor directly
    MCEP_REQUIRE(num_experts > 0 && num_experts % b->num_ranks == 0 && M > 0 && hidden > 0);
    const Geometry g = geometry(b->num_ranks, num_experts, M, hidden, use_fp8 != 0);
    if (2 * g.parity_bytes > (size_t)b->num_bytes) return MCEP_OK;  // dispatch will report it
    const int par = (b->dseq + 1) & 1;
    *out = b->base + kHeaderRegion + (size_t)par * g.parity_bytes;
    if (bytes) *bytes = (size_t)num_experts * M * g.row_bytes;
    return MCEP_OK;
}

int mcep_buffer_next_combine_buffer(mcep_buffer* b, int M, int hidden, int num_experts, void** out,
                                    size_t* bytes) {
    MCEP_REQUIRE(b != nullptr && out != nullptr);
    *out = nullptr;
    if (bytes) *bytes = 0;
    if (!is_group(b)) return MCEP_OK;  // a single rank reads the caller's tensor directly
    MCEP_REQUIRE(num_experts > 0 && num_experts % b->num_ranks == 0 && M > 0 && hidden > 0);
    const Geometry g = geometry(b->num_ranks, num_experts, M, hidden, false);
    if (2 * g.parity_bytes > (size_t)b->num_bytes)
        return fail(MCEP_ERR_INVALID,
                    "Failed: Assertion error %s:%d 'layout.total_bytes <= num_ep_buffer_bytes' "
                    "(need %zu, have %lld)",
                    __FILE__, __LINE__, 2 * g.parity_bytes, (long long)b->num_bytes);
    const int par = (b->cseq + 1) & 1;
    *out = b->base + kHeaderRegion + (size_t)par * g.parity_bytes + g.darea_bytes;
    if (bytes) *bytes = g.cin_bytes;
    return MCEP_OK;
}

static mcep::Words words_of(int dpar, int cpar) {
    mcep::Words w;
    w.cnt_off = (size_t)dpar * kHeaderParity;
    w.beg_off = w.cnt_off + kWordBlock;
    w.dflag_off = w.beg_off + kWordBlock;
    w.cflag_off = (size_t)cpar * kHeaderParity + 2 * kWordBlock + 64 * sizeof(uint64_t);
    return w;
}

static int completion_event(cudaStream_t stream, mcep_event** out_event) {
    auto* ev = new mcep_event();
    if (cudaEventCreateWithFlags(&ev->ev, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventRecord(ev->ev, stream) != cudaSuccess) {
        delete ev;
        return fail(MCEP_ERR_CUDA, "Failed: CUDA error creating the completion event");
    }
    *out_event = ev;
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
    const bool group = is_group(b);
    const Geometry g = geometry(R, E, M, H, fp8);
    if (group && 2 * g.parity_bytes > (size_t)b->num_bytes)
        return fail(MCEP_ERR_INVALID,
                    "Failed: Assertion error %s:%d 'layout.total_bytes <= num_ep_buffer_bytes' "
                    "(need %zu, have %lld)",
                    __FILE__, __LINE__, 2 * g.parity_bytes, (long long)b->num_bytes);

    const uint32_t seq = ++b->dseq;
    const int par = seq & 1;
    auto& sc = b->scratch[par];

    cudaStream_t compute = reinterpret_cast<cudaStream_t>(a->compute_stream);
    // Without a hook or an event the caller's stream has to wait for the result
    // anyway, so the kernels go straight onto it; `async_finish` runs them on
    // the communication stream behind everything queued on the caller's stream.
    cudaStream_t stream = a->async_finish ? b->comm_stream : compute;
    if (a->async_finish)
        if (int rc = order_after(stream, compute, b->ev_a)) return rc;

    const bool pdl = chain_with_pdl(b, stream) && chain_with_pdl(b, compute);
    const bool chain_first = b->chain_first_once && pdl && !b->defer;
    b->chain_first_once = false;
    mcep::LaunchCtx first{stream, b->num_sms, chain_first};
    mcep::LaunchCtx next{stream, b->num_sms, pdl};

    const bool fused = mcep::can_fuse_layout(T, K, E, b->num_sms) && b->fuse_layout;
    if (!fused) {
        mcep::LayoutParams lp = {};
        lp.topk_idx = a->topk_idx;
        lp.T = T, lp.K = K, lp.E = E, lp.R = R;
        lp.count = sc.count, lp.slot = sc.slot, lp.ticket = sc.layout_ticket;
        lp.chunk_hist = sc.chunk_hist, lp.chunk_hist_entries = kChunkHistBytes / sizeof(int32_t);
        if (!group) {
            lp.recv_count = a->packed_recv_count;
            lp.layout_range = a->packed_recv_layout_range;
        }
        MCEP_CUDA(mcep::launch_layout(lp, first));
    }

    if (!group) {
        // a single rank: the packed outputs are written directly, no words, no waits
        mcep::DirectDispatchParams dp = {};
        dp.x = a->x, dp.topk_idx = a->topk_idx, dp.slot = sc.slot, dp.count = sc.count;
        dp.T = T, dp.K = K, dp.E = E, dp.M = M, dp.H = H, dp.use_fp8 = fp8, dp.fused = fused;
        dp.status = b->status, dp.recv_x = a->packed_recv_x;
        dp.recv_scales = a->packed_recv_x_scales, dp.recv_src_info = a->packed_recv_src_info;
        dp.recv_count = a->packed_recv_count, dp.layout_range = a->packed_recv_layout_range;
        dp.rowmap = sc.rowmap;
        auto& rec = b->record[par];
        rec.key = a->packed_recv_src_info, rec.seq = seq, rec.stamp = ++b->record_clock;
        rec.T = T, rec.K = K, rec.E = E, rec.M = M, rec.H = H;
        MCEP_CUDA(mcep::launch_direct_dispatch(dp, fused ? first : next));
        if (a->return_recv_hook) {
            auto* h = new mcep_hook();
            h->fn = []() { return MCEP_OK; };
            *out_hook = h;
            return MCEP_OK;
        }
        if (a->async_finish) return completion_event(stream, out_event);
        return MCEP_OK;
    }

    char* area = b->base + kHeaderRegion + (size_t)par * g.parity_bytes;
    mcep::GroupDispatchParams p = {};
    p.x = a->x, p.topk_idx = a->topk_idx, p.slot = sc.slot, p.count = sc.count;
    p.peer_base = b->peer_dev, p.local_base = b->base;
    p.T = T, p.K = K, p.E = E, p.R = R, p.M = M, p.H = H, p.rank = b->rank;
    p.use_fp8 = fp8, p.fused = fused;
    p.w = words_of(par, 0);
    p.rx_off = (size_t)(area - b->base), p.meta_off = p.rx_off + g.meta_off;
    p.row_bytes = g.row_bytes, p.meta_stride = g.meta_stride;
    p.seq = seq;
    uint32_t* seq_word = b->graph_mode ? b->dev_next_seq + par : nullptr;
    p.seq_ptr = seq_word;
    p.wait.active_ranks = a->active_ranks, p.wait.timeout_ns = to_ns(a->timeout_us);
    p.wait.hard_timeout_ns = b->hard_timeout_ns, p.wait.status = b->status;
    p.res_cnt = sc.res_cnt, p.res_dflag = sc.res_dflag, p.ticket = sc.send_ticket;
    p.rowmap = sc.rowmap;
    p.recv_x = a->packed_recv_x, p.recv_scales = a->packed_recv_x_scales;
    p.recv_src_info = a->packed_recv_src_info, p.recv_count = a->packed_recv_count;
    p.layout_range = a->packed_recv_layout_range;
    // the caller either took the tensor mcep_buffer_next_recv_x names (rows land in
    // it, nothing to copy) or passes memory of its own (rows are copied out)
    p.copy_rows = (a->packed_recv_x != static_cast<void*>(area));

    auto& rec = b->record[par];
    rec.key = a->packed_recv_src_info, rec.seq = seq, rec.stamp = ++b->record_clock;
    rec.T = T, rec.K = K, rec.E = E, rec.M = M, rec.H = H;

    const int num_sms = b->num_sms;
    // Small batches, rows in place, no hook: one launch does it all.
    bool one_kernel = fused && !p.copy_rows && !a->return_recv_hook && b->one_kernel &&
                      mcep::group_call_can_be_one_kernel(T, K, E, num_sms);
    if (b->defer) {
        MCEP_REQUIRE(!a->async_finish && !b->graph_mode);
        b->pending.kind = 1, b->pending.phases = one_kernel ? 3 : 1, b->pending.d = p;
        b->pending.then_second = !one_kernel && !a->return_recv_hook;
        b->pending.stream = compute;
        if (a->return_recv_hook) {
            auto* h = new mcep_hook();
            h->fn = [=]() {
                mcep::LaunchCtx c0{compute, num_sms, false};
                MCEP_CUDA(mcep::launch_group_dispatch_recv(p, c0));
                return MCEP_OK;
            };
            *out_hook = h;
        }
        return MCEP_OK;
    }
    if (one_kernel) {
        cudaError_t e1 = mcep::launch_group_dispatch(p, first);
        if (e1 == cudaErrorInvalidConfiguration) {
            cudaGetLastError();  // would not be resident at once on this device: two launches
            one_kernel = false;
        } else {
            MCEP_CUDA(e1);
        }
    }
    if (!one_kernel) MCEP_CUDA(mcep::launch_group_dispatch_send(p, fused ? first : next));
    auto recv = [=](cudaStream_t s, bool chained) -> int {
        mcep::LaunchCtx c0{s, num_sms, chained && pdl};
        if (!one_kernel) MCEP_CUDA(mcep::launch_group_dispatch_recv(p, c0));
        // graph mode: the call is over, its parity's word moves on
        if (seq_word) MCEP_CUDA(mcep::launch_advance_seq(seq_word, c0));
        return MCEP_OK;
    };

    if (a->return_recv_hook) {
        auto* h = new mcep_hook();
        h->fn = [=]() { return recv(compute, false); };
        *out_hook = h;
        return MCEP_OK;
    }
    if (int rc = recv(stream, true)) return rc;
    if (a->async_finish) return completion_event(stream, out_event);
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
    MCEP_REQUIRE(T == 0 || (a->topk_idx != nullptr && a->topk_weights != nullptr));
    MCEP_REQUIRE(a->zero_copy || T == 0 || a->x != nullptr);
    MCEP_REQUIRE(a->src_info != nullptr && a->layout_range != nullptr);
    MCEP_REQUIRE(a->active_ranks != nullptr);
    MCEP_REQUIRE(T == 0 || a->combined_x != nullptr);
    MCEP_REQUIRE(aligned(a->x, 32) && aligned(a->combined_x, 32));
    MCEP_REQUIRE((size_t)T * K <= b->scratch_entries);
    if (int rc = check_connected(b)) return rc;

    const bool group = is_group(b);
    const Geometry g = geometry(R, E, M, H, false);
    if (group && 2 * g.parity_bytes > (size_t)b->num_bytes)
        return fail(MCEP_ERR_INVALID,
                    "Failed: Assertion error %s:%d 'layout.total_bytes <= num_ep_buffer_bytes' "
                    "(need %zu, have %lld)",
                    __FILE__, __LINE__, 2 * g.parity_bytes, (long long)b->num_bytes);

    cudaStream_t compute = reinterpret_cast<cudaStream_t>(a->compute_stream);
    cudaStream_t stream = a->async_finish ? b->comm_stream : compute;
    const bool pdl = chain_with_pdl(b, stream) && chain_with_pdl(b, compute);
    const int num_sms = b->num_sms;

    if (!group) {
        // a single rank gathers straight from the expert-output tensor; with
        // zero_copy the caller's tensor IS the combine buffer (nothing differs)
        const uint32_t seq = ++b->cseq;
        auto& sc = b->scratch[seq & 1];
        if (a->async_finish)
            if (int rc = order_after(stream, compute, b->ev_a)) return rc;
        mcep::LaunchCtx first{stream, num_sms, false};
        // The rows of (token, k) inside their experts: kept from the dispatch call
        // when the handle is that of one of the last two; otherwise found again
        // in the handle itself - by the reduce kernel (small batches) or by an
        // inversion pass of its own.
        const int32_t* rowmap = nullptr;
        {
            const mcep_buffer::DispatchRecord* rec = nullptr;
            for (int i = 0; i < 2; ++i) {
                const auto& c = b->record[i];
                if (c.key != nullptr && c.key == a->src_info && (rec == nullptr || c.stamp > rec->stamp))
                    rec = &c;
            }
            if (rec && rec->T == T && rec->K == K && rec->E == E && rec->M == M && rec->H == H)
                rowmap = b->scratch[rec->seq & 1].rowmap;
        }
        const bool search = rowmap == nullptr && (long long)T * K <= 4096;
        if (rowmap == nullptr && !search) {
            mcep::CombineInvertParams ip = {};
            ip.src_info = a->src_info, ip.layout_range = a->layout_range, ip.topk_idx = a->topk_idx;
            ip.L = E, ip.R = 1, ip.M = M, ip.T = T, ip.K = K, ip.rank = 0;
            ip.rowmap = sc.rowmap_inv, ip.status = b->status;
            MCEP_CUDA(mcep::launch_combine_invert(ip, first));
            rowmap = sc.rowmap_inv;
        }
        const bool chain = rowmap == sc.rowmap_inv && !search;
        mcep::DirectCombineParams dp = {};
        dp.topk_idx = a->topk_idx, dp.topk_weights = a->topk_weights;
        dp.active_ranks = a->active_ranks;
        dp.T = T, dp.K = K, dp.E = E, dp.M = M, dp.H = H;
        dp.x = a->x, dp.rowmap = rowmap, dp.search = search;
        dp.src_info = a->src_info, dp.layout_range = a->layout_range;
        dp.combined_x = a->combined_x;
        auto reduce = [=](cudaStream_t s, bool chained) -> int {
            mcep::LaunchCtx c0{s, num_sms, chained && pdl && chain};
            MCEP_CUDA(mcep::launch_direct_combine(dp, c0));
            return MCEP_OK;
        };
        if (a->return_recv_hook) {
            auto* h = new mcep_hook();
            h->fn = [=]() { return reduce(compute, false); };
            *out_hook = h;
            return MCEP_OK;
        }
        if (int rc = reduce(stream, true)) return rc;
        if (a->async_finish) return completion_event(stream, out_event);
        return MCEP_OK;
    }

    // Which dispatch call does this handle come from? Its rows' positions at the
    // experts' owners were recorded then; the two most recent calls are kept.
    const mcep_buffer::DispatchRecord* rec = nullptr;
    for (int i = 0; i < 2; ++i) {
        const auto& c = b->record[i];
        if (c.key != nullptr && c.key == a->src_info && (rec == nullptr || c.stamp > rec->stamp)) rec = &c;
    }
    if (rec == nullptr)
        return fail(MCEP_ERR_STATE,
                    "Failed: Assertion error %s:%d 'combine needs the handle of one of the last two "
                    "dispatch calls of this buffer'",
                    __FILE__, __LINE__);
    if (rec->T != T || rec->K != K || rec->E != E || rec->M != M || rec->H != H)
        return fail(MCEP_ERR_INVALID,
                    "Failed: Assertion error %s:%d 'combine arguments match the dispatch call of the "
                    "handle' (dispatch: T=%d K=%d E=%d M=%d H=%d)",
                    __FILE__, __LINE__, rec->T, rec->K, rec->E, rec->M, rec->H);
    const int dpar = rec->seq & 1;

    const uint32_t seq = ++b->cseq;
    const int par = seq & 1;
    if (a->async_finish)
        if (int rc = order_after(stream, compute, b->ev_a)) return rc;
    mcep::LaunchCtx first{stream, num_sms, false};

    mcep::GroupCombineParams p = {};
    p.x = a->x, p.layout_range = a->layout_range, p.topk_idx = a->topk_idx;
    p.topk_weights = a->topk_weights, p.rowmap = b->scratch[dpar].rowmap;
    p.peer_base = b->peer_dev, p.local_base = b->base;
    p.T = T, p.K = K, p.E = E, p.R = R, p.M = M, p.H = H, p.rank = b->rank;
    p.zero_copy = a->zero_copy != 0;
    p.w = words_of(0, par);
    p.cin_off = kHeaderRegion + (size_t)par * g.parity_bytes + g.darea_bytes;
    p.seq = seq;
    uint32_t* seq_word = b->graph_mode ? b->dev_next_seq + 2 + par : nullptr;
    p.seq_ptr = seq_word;
    p.wait.active_ranks = a->active_ranks, p.wait.timeout_ns = to_ns(a->timeout_us);
    p.wait.hard_timeout_ns = b->hard_timeout_ns, p.wait.status = b->status;
    p.res_cflag = b->scratch[par].res_cflag, p.ticket = b->scratch[par].publish_ticket;
    p.combined_x = a->combined_x;

    const bool one_kernel = !a->return_recv_hook && b->one_kernel &&
                            mcep::group_call_can_be_one_kernel(T, K, E, num_sms);
    MCEP_REQUIRE(!(b->defer && b->graph_mode));
    if (b->defer && !a->return_recv_hook) {
        // The publish phase waits for nobody and can be launched rank by rank,
        // the reduce phase only once every rank has published; both phases in one
        // launch need all ranks in that launch.
        MCEP_REQUIRE(!a->async_finish);
        if (!one_kernel) MCEP_CUDA(mcep::launch_group_combine_publish(p, first));
        b->pending.kind = 2, b->pending.phases = one_kernel ? 3 : 2, b->pending.c = p;
        b->pending.then_second = false, b->pending.stream = compute;
        return MCEP_OK;
    }
    if (one_kernel)
        MCEP_CUDA(mcep::launch_group_combine(p, first));
    else
        MCEP_CUDA(mcep::launch_group_combine_publish(p, first));
    auto reduce = [=](cudaStream_t s, bool chained) -> int {
        mcep::LaunchCtx c0{s, num_sms, chained && pdl};
        if (!one_kernel) MCEP_CUDA(mcep::launch_group_combine_reduce(p, c0));
        if (seq_word) MCEP_CUDA(mcep::launch_advance_seq(seq_word, c0));
        return MCEP_OK;
    };

    if (a->return_recv_hook) {
        auto* h = new mcep_hook();
        h->fn = [=]() { return reduce(compute, false); };
        *out_hook = h;
        return MCEP_OK;
    }
    if (int rc = reduce(stream, true)) return rc;
    if (a->async_finish) return completion_event(stream, out_event);
    return MCEP_OK;
}

// -----------------------------------------------------------------------------
// barrier
// -----------------------------------------------------------------------------
int mcep_buffer_barrier(mcep_buffer* b, const int32_t* active_ranks, uint64_t stream) {
    MCEP_REQUIRE(b != nullptr);
    if (b->num_ranks == 1) return MCEP_OK;
    if (int rc = check_connected(b)) return rc;
    mcep::BarrierParams p = {};
    p.peer_base = b->peer_dev, p.local_base = b->base, p.active_ranks = active_ranks;
    p.bar_off = kBarrierOff, p.rank = b->rank, p.R = b->num_ranks;
    p.epoch = ++b->barrier_epoch;
    p.hard_timeout_ns = b->hard_timeout_ns, p.status = b->status;
    mcep::LaunchCtx ctx{reinterpret_cast<cudaStream_t>(stream), b->num_sms, false};
    MCEP_CUDA(mcep::launch_barrier(p, ctx));
    return MCEP_OK;
}

// -----------------------------------------------------------------------------
// in-process groups: start what the ranks have prepared, in one launch
// -----------------------------------------------------------------------------
int mcep_launch_deferred(mcep_buffer* const* bufs, int n) {
    MCEP_REQUIRE(bufs != nullptr && n >= 1 && n <= mcep::kMaxRanks);
    std::vector<mcep::GroupDispatchParams> dps;
    std::vector<mcep::GroupCombineParams> cps;
    std::vector<mcep_buffer*> who;
    int kind = 0, phases = 0;
    cudaStream_t stream = nullptr;
    for (int i = 0; i < n; ++i) {
        mcep_buffer* b = bufs[i];
        MCEP_REQUIRE(b != nullptr);
        if (b->pending.kind == 0) continue;
        if (kind == 0) kind = b->pending.kind, phases = b->pending.phases, stream = b->pending.stream;
        MCEP_REQUIRE(b->pending.kind == kind && b->pending.phases == phases);
        MCEP_REQUIRE(b->pending.stream == stream && b->device == bufs[0]->device);
        if (kind == 1) dps.push_back(b->pending.d); else cps.push_back(b->pending.c);
        who.push_back(b);
    }
    if (kind == 0) return MCEP_OK;
    mcep_buffer* b0 = who[0];
    const size_t need = kind == 1 ? sizeof(mcep::GroupDispatchParams) * dps.size()
                                  : sizeof(mcep::GroupCombineParams) * cps.size();
    static void* dev_params = nullptr;
    static size_t dev_params_bytes = 0;
    if (need > dev_params_bytes) {
        if (dev_params) cudaFree(dev_params);
        dev_params = nullptr, dev_params_bytes = 0;
        MCEP_CUDA(cudaMalloc(&dev_params, need));
        dev_params_bytes = need;
    }
    mcep::LaunchCtx ctx{stream, b0->num_sms, false};
    if (kind == 2 && phases == 2) {  // every rank has published: the reduce phases, rank by rank
        for (mcep_buffer* b : who) {
            b->pending.kind = 0;
            MCEP_CUDA(mcep::launch_group_combine_reduce(b->pending.c, ctx));
        }
        return MCEP_OK;
    }
    cudaError_t e;
    if (kind == 1)
        e = mcep::launch_group_dispatch_multi(dps.data(), (int)dps.size(),
                                              static_cast<mcep::GroupDispatchParams*>(dev_params),
                                              phases, ctx);
    else
        e = mcep::launch_group_combine_multi(cps.data(), (int)cps.size(),
                                             static_cast<mcep::GroupCombineParams*>(dev_params), ctx);
    for (mcep_buffer* b : who) b->pending.kind = 0;
    MCEP_CUDA(e);
    if (kind == 1) {
        for (mcep_buffer* b : who)
            if (b->pending.then_second) MCEP_CUDA(mcep::launch_group_dispatch_recv(b->pending.d, ctx));
        for (mcep_buffer* b : who) {
            if (!b->after_deferred) continue;
            std::function<int()> fn;
            fn.swap(b->after_deferred);
            if (int rc = fn()) return rc;
        }
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
size_t mcep_routing_layout_scratch_bytes(void) { return 256 + kChunkHistBytes; }

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
    lp.chunk_hist = reinterpret_cast<int32_t*>(static_cast<char*>(scratch) + 256);
    lp.chunk_hist_entries = kChunkHistBytes / sizeof(int32_t);
    mcep::LaunchCtx ctx{reinterpret_cast<cudaStream_t>(stream), sms, false};
    MCEP_CUDA(mcep::launch_layout(lp, ctx));
    return MCEP_OK;
}

}  // extern "C"
