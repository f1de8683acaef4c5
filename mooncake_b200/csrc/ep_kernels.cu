// Hand-written sm_100a kernels of the EP hot path: routing layout, dispatch and
// combine, for a single rank and for a group of ranks on one NVLink domain.
//
// What they replace in the reference (paths inside the Mooncake tree):
//   mooncake-ep/src/mooncake_ep_kernel.cu:138-470  `dispatch`
//   mooncake-ep/src/mooncake_ep_kernel.cu:550-754  `combine`
// Design differences, all deliberate:
//   * receive order is deterministic (source rank, then token index): a token's
//     row inside its expert is (first row of the source's segment) + (earlier
//     tokens of the same source for that expert), never an atomic in arrival
//     order;
//   * dispatch has ONE data pass: the owner of an expert collects the counts
//     every source announces, answers each source with the first row of its
//     segment, and the source then stores the row - read once, quantised in
//     registers - straight into its final place in the owner's packed receive
//     area over NVLink (the reference stages the row locally, copies it to the
//     owner's staging and copies it again into the packed output);
//   * combine has ONE data pass over NVLink: expert outputs are made readable in
//     symmetric memory, and the token owner reads its K rows from the experts'
//     owners and reduces them in registers (the reference pushes every row into
//     staging at the token owner first);
//   * no cooperative launch, no grid-wide barrier; sender blocks depend on the
//     control block (block 0, resident first) and on other GPUs only;
//   * work is split by token and by row, not by expert, so the grid fills 148
//     SMs for 8 experts as well as for 256;
//   * the words ranks exchange are 64-bit (call sequence number << 32 | value)
//     and are never cleaned.
#include "ep_kernels.cuh"

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "ep_device.cuh"

namespace mcep {

static std::atomic<uint64_t> g_launches{0};
uint64_t kernel_launch_count() { return g_launches.load(); }

// Optional per-kernel timing: every launch is bracketed by two events on its own
// stream (which also serialises kernels that would otherwise overlap through
// programmatic dependent launch), so a caller can read each kernel's device time.
namespace {
struct TimingRec {
    const char* name;
    cudaEvent_t a, b;
};
std::atomic<bool> g_timing{false};
std::mutex g_timing_mu;
std::vector<TimingRec> g_recs;
}  // namespace

void set_kernel_timing(bool on) { g_timing.store(on); }

std::string drain_kernel_times() {
    std::lock_guard<std::mutex> lk(g_timing_mu);
    std::map<std::string, std::pair<int, double>> agg;
    for (auto& r : g_recs) {
        float ms = 0.f;
        if (cudaEventSynchronize(r.b) == cudaSuccess &&
            cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            auto& e = agg[r.name];
            e.first += 1;
            e.second += ms;
        }
        cudaEventDestroy(r.a);
        cudaEventDestroy(r.b);
    }
    g_recs.clear();
    std::string out;
    for (auto& kv : agg) {
        char line[256];
        snprintf(line, sizeof(line), "%s %d %.6f\n", kv.first.c_str(), kv.second.first,
                 kv.second.second);
        out += line;
    }
    return out;
}

LaunchScope::LaunchScope(const char* name, cudaStream_t stream) : name_(name), stream_(stream) {
    if (g_timing.load()) {
        cudaEventCreate(&a_);
        cudaEventCreate(&b_);
        cudaEventRecord(a_, stream_);
    }
}

cudaError_t LaunchScope::done(cudaError_t err) {
    if (a_ != nullptr) {
        cudaEventRecord(b_, stream_);
        std::lock_guard<std::mutex> lk(g_timing_mu);
        g_recs.push_back(TimingRec{name_, a_, b_});
    }
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

namespace kernels {

constexpr unsigned kFull = 0xffffffffu;

template <typename... KArgs, typename... Args>
cudaError_t launch(const char* name, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                   const LaunchCtx& ctx, Args&&... args) {
    if (g_timing.load()) {
        TimingRec r{name, nullptr, nullptr};
        cudaEventCreate(&r.a);
        cudaEventCreate(&r.b);
        cudaEventRecord(r.a, ctx.stream);
        kernel<<<grid, block, smem, ctx.stream>>>(args...);
        cudaError_t err = cudaGetLastError();
        cudaEventRecord(r.b, ctx.stream);
        std::lock_guard<std::mutex> lk(g_timing_mu);
        g_recs.push_back(r);
        if (err == cudaSuccess) g_launches.fetch_add(1);
        return err;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx.stream;
    cudaLaunchAttribute attr[1];
    if (ctx.pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

__device__ __forceinline__ int warp_inclusive_scan(int v, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        int u = __shfl_up_sync(kFull, v, d);
        if (lane >= d) v += u;
    }
    return v;
}

// In-place exclusive scan of a[0..n) in shared memory; a[n] receives the total.
// Every thread of the block must call it.
__device__ void block_exclusive_scan(int* a, int n, int* warp_totals /*[32]*/) {
    const int nthr = blockDim.x, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    const int per = (n + nthr - 1) / nthr;
    const int b = min(tid * per, n), e = min(b + per, n);
    int sum = 0;
    for (int i = b; i < e; ++i) sum += a[i];
    int incl = warp_inclusive_scan(sum, lane);
    if (lane == 31) warp_totals[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = lane < nwarps ? warp_totals[lane] : 0;
        int wi = warp_inclusive_scan(w, lane);
        warp_totals[lane] = wi - w;
        if (lane == 31) a[n] = wi;
    }
    __syncthreads();
    int run = warp_totals[warp] + incl - sum;
    for (int i = b; i < e; ++i) {
        int v = a[i];
        a[i] = run;
        run += v;
    }
    __syncthreads();
}

// Last index i in [0, n) with pre[i] <= g (pre is a non-decreasing exclusive
// prefix, pre[0] == 0): the non-empty segment that holds row g.
__device__ __forceinline__ int find_segment(const int* pre, int n, int g) {
    int lo = 0, hi = n;
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (pre[mid] <= g)
            lo = mid;
        else
            hi = mid;
    }
    return lo;
}

// =============================================================================
// waiting for words of other ranks
// =============================================================================
// The timeout rule of mooncake-ep/src/mooncake_ep_kernel.cu:417-429 and :685-699:
// after `timeout` the waiter clears active_ranks[src]; whoever sees the entry
// cleared stops waiting. Every wait is also bounded by the hard limit.

//
// Waits of one dispatch call form a chain: an owner waits for the sources'
// counts; a sender waits for the owner's answer, which a live owner may hold
// back until it has given up on a dead source; a receiver waits for the senders'
// payload words, which may be late for the same reason. So the answer is given
// twice, and the payload word three times, the bound of the count - otherwise
// one dead rank would make every live rank give up on every other. The dead
// rank itself is still given up on after ONE timeout: whoever times out clears
// its entry of the mask, and every waiter looks at the mask.
__device__ __forceinline__ WaitCfg scaled(const WaitCfg& w, int times) {
    WaitCfg r = w;
    if (r.timeout_ns >= 0) r.timeout_ns *= times;
    r.hard_timeout_ns *= times;
    return r;
}

// One waiter per word (or waiters that may disagree harmlessly). Returns the
// word's value (>= 1) or 0 when given up.
__device__ __forceinline__ uint32_t wait_word(const uint64_t* word, uint32_t seq, const WaitCfg& w,
                                              int src) {
    uint64_t start = 0;
    while (true) {
        const uint64_t v = ld_acquire_sys(word);
        if ((uint32_t)(v >> 32) == seq) return (uint32_t)v;
        const uint64_t now = globaltimer_ns();
        if (start == 0) start = now;
        const int64_t waited = (int64_t)(now - start);
        if (w.timeout_ns >= 0 && waited > w.timeout_ns) st_volatile_s32(w.active_ranks + src, 0);
        if (waited > w.hard_timeout_ns) {
            st_volatile_s32(w.active_ranks + src, 0);
            atomicOr(w.status, kStatusHardTimeout);
        }
        if (!ld_volatile_s32(w.active_ranks + src)) return 0;
    }
}

// Many waiters per word that must agree (or one token of a result would count a
// rank in and the next would not): the first block to reach a verdict publishes
// it with a compare-and-swap into a local word, and every block - that one
// included - takes the verdict from that word:
//   resolved = seq << 32 | value     arrived
//   resolved = seq << 32 | 0         given up
// No block waits for another block: each keeps polling the peer's word itself
// until some verdict exists. Returns the value, or 0.
__device__ __forceinline__ uint32_t resolve_flag(const uint64_t* flags, uint64_t* resolved, int i,
                                                 uint32_t seq, const WaitCfg& w, int src,
                                                 bool primary = true) {
    unsigned long long* res = reinterpret_cast<unsigned long long*>(resolved + i);
    uint64_t start = 0;
    if (!primary) {
        // Many blocks want the same verdict. One of them (the "primary" for this
        // flag) goes for the flag at once; the others look at the verdict word
        // alone for a short while, which keeps hundreds of blocks from hammering
        // one address with compare-and-swaps, and then fall back to doing the
        // work themselves - they never depend on the primary making progress.
        start = globaltimer_ns();
        while (globaltimer_ns() - start < 4000) {
            const uint64_t r = ld_acquire_gpu(resolved + i);
            if ((uint32_t)(r >> 32) == seq) {
                const uint32_t v = (uint32_t)r;
                if (v) (void)ld_acquire_sys(flags + i);
                return v;
            }
        }
    }
    while (true) {
        // both words are requested together: one round trip in the common case
        const uint64_t r = ld_acquire_gpu(resolved + i);
        const uint64_t f = ld_acquire_sys(flags + i);
        if ((uint32_t)(r >> 32) == seq) {
            // decided already (possibly by another block). If it is an arrival,
            // the flag load above was our own acquire of the sender's release -
            // unless it raced ahead of the flag, then take it again.
            const uint32_t v = (uint32_t)r;
            if (v && (uint32_t)(f >> 32) != seq) (void)ld_acquire_sys(flags + i);
            return v;
        }
        unsigned long long mine;
        if ((uint32_t)(f >> 32) == seq) {
            mine = (unsigned long long)f;  // arrived
        } else {
            const uint64_t now = globaltimer_ns();
            if (start == 0) start = now;
            const int64_t waited = (int64_t)(now - start);
            if (w.timeout_ns >= 0 && waited > w.timeout_ns) st_volatile_s32(w.active_ranks + src, 0);
            if (waited > w.hard_timeout_ns) {
                st_volatile_s32(w.active_ranks + src, 0);
                atomicOr(w.status, kStatusHardTimeout);
            }
            if (ld_volatile_s32(w.active_ranks + src)) continue;  // keep waiting
            mine = (unsigned long long)seq << 32;                 // given up
        }
        // first verdict wins; the value the swap returns is the winner's
        const unsigned long long old = atomicCAS(res, (unsigned long long)r, mine);
        const unsigned long long verdict = (old == (unsigned long long)r) ? mine : old;
        if ((uint32_t)(verdict >> 32) != seq) continue;  // lost to a stale word: look again
        const uint32_t v = (uint32_t)verdict;
        if (v && (uint32_t)(f >> 32) != seq) (void)ld_acquire_sys(flags + i);
        return v;
    }
}

// A word another block of this GPU writes (the control block's verdicts). The
// writer is resident before any reader and never waits for a reader.
__device__ __forceinline__ uint32_t wait_local_word(const uint64_t* word, uint32_t seq,
                                                    const WaitCfg& w) {
    uint64_t start = 0;
    while (true) {
        const uint64_t v = ld_acquire_gpu(word);
        if ((uint32_t)(v >> 32) == seq) return (uint32_t)v;
        const uint64_t now = globaltimer_ns();
        if (start == 0) start = now;
        if ((int64_t)(now - start) > w.hard_timeout_ns) {
            atomicOr(w.status, kStatusHardTimeout);
            return 0;
        }
    }
}

// =============================================================================
// phase trace (diagnostic builds only: -DMCEP_PHASE_TRACE)
// =============================================================================
// Thread 0 of every block stamps the global nanosecond timer at phase
// boundaries, so blocks - and kernels - can be lined up against each other.
// Compiled out of the normal library.
#ifdef MCEP_PHASE_TRACE
constexpr int kTraceBodies = 4, kTraceBlocks = 1024, kTraceSlots = 8;
__device__ unsigned long long g_phase_trace[kTraceBodies][kTraceBlocks][kTraceSlots];
#define MCEP_TRACE(body, slot)                                              \
    do {                                                                    \
        if (threadIdx.x == 0 && blockIdx.x < kTraceBlocks)                  \
            g_phase_trace[body][blockIdx.x][slot] = globaltimer_ns();       \
    } while (0)
#else
#define MCEP_TRACE(body, slot) \
    do {                       \
    } while (0)
#endif

// =============================================================================
// routing layout
// =============================================================================
// One block owns `epc` consecutive experts. It builds, in shared memory, one
// bit per (expert, token) and a popcount prefix per 32-token word; a slot is
// then prefix + popcount of the lower bits. Token order is the only order.
__global__ void __launch_bounds__(1024)
    ep_routing_layout_kernel(LayoutParams p, int epc, int words) {
    extern __shared__ uint32_t smem_u32[];
    uint32_t* mask = smem_u32;
    uint32_t* wpre = smem_u32 + (size_t)epc * words;
    __shared__ bool s_last;

    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    const int e0 = blockIdx.x * epc;
    const int e1 = min(p.E, e0 + epc);
    const int ne = e1 - e0;
    const int n = p.T * p.K;

    for (int i = tid; i < ne * words; i += nthr) mask[i] = 0;
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
    // Every block reads the whole index matrix; the loads are issued eight at a
    // time so a pass costs a few memory round trips, not one per entry.
    constexpr int kU = 8;
    for (int i0 = tid; i0 < n; i0 += nthr * kU) {
        int ev[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int i = i0 + u * nthr;
            ev[u] = i < n ? (int)__ldg(p.topk_idx + i) : -1;
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int e = ev[u];
            if (e >= e0 && e < e1) {
                const int t = (i0 + u * nthr) / p.K;
                atomicOr(&mask[(e - e0) * words + (t >> 5)], 1u << (t & 31));
            }
        }
    }
    __syncthreads();
    for (int le = warp; le < ne; le += nwarps) {
        int carry = 0;
        for (int w0 = 0; w0 < words; w0 += 32) {
            const int w = w0 + lane;
            const int c = w < words ? __popc(mask[le * words + w]) : 0;
            const int incl = warp_inclusive_scan(c, lane);
            if (w < words) wpre[le * words + w] = carry + incl - c;
            carry += __shfl_sync(kFull, incl, 31);
        }
        if (lane == 0) {
            const int e = e0 + le;
            p.count[e] = carry;
            if (p.recv_count) p.recv_count[e] = carry;
            if (p.layout_range) p.layout_range[e] = carry;  // begin 0 | count
        }
    }
    __syncthreads();
    for (int i0 = tid; i0 < n; i0 += nthr * kU) {
        int ev[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int i = i0 + u * nthr;
            ev[u] = i < n ? (int)__ldg(p.topk_idx + i) : -2;
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int i = i0 + u * nthr;
            const int e = ev[u];
            if (e >= e0 && e < e1) {
                const int t = i / p.K, k = i - t * p.K;
                bool dup = false;
                for (int kk = 0; kk < k; ++kk) dup |= ((int)__ldg(p.topk_idx + t * p.K + kk) == e);
                const int o = (e - e0) * words + (t >> 5);
                p.slot[i] = dup ? -1 : (int)(wpre[o] + __popc(mask[o] & ((1u << (t & 31)) - 1u)));
            } else if (e < 0 && i < n && blockIdx.x == 0) {
                p.slot[i] = -1;
            }
        }
    }
    if (p.rank_count == nullptr && p.expert_prefix == nullptr) return;

    // The block that finishes last turns the per-expert counts into per-rank
    // counts and prefix offsets inside each rank's block of experts.
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = (atomicInc(p.ticket, gridDim.x - 1) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int L = p.E / p.R;
    for (int r = warp; r < p.R; r += nwarps) {
        int carry = 0;
        for (int b = 0; b < L; b += 32) {
            const int le = b + lane;
            const int c = le < L ? __ldcg(p.count + r * L + le) : 0;
            const int incl = warp_inclusive_scan(c, lane);
            if (le < L && p.expert_prefix) p.expert_prefix[r * L + le] = carry + incl - c;
            carry += __shfl_sync(kFull, incl, 31);
        }
        if (lane == 0 && p.rank_count) p.rank_count[r] = carry;
    }
}

// ---- the same layout in two passes over token chunks ------------------------------
// The kernel above lets every block read the whole index matrix (each block owns
// some experts). For large batches that costs more than the work itself, so the
// usual route is two small kernels in which a block owns a CHUNK of tokens and
// reads only that chunk:
//   pass 1  per-chunk histogram of the (de-duplicated) expert choices;
//   pass 2  per expert, the count of all earlier chunks (a short column sum) plus
//           the position inside the chunk (bitmap + popcount, as above) = slot;
//           the block of the last chunk also writes the totals.
// A repeated expert inside a token counts once; token order is the only order.
// One lane per token: the token's K choices are requested together (one memory
// round trip) and de-duplicated in registers; e[k] = -1 for masked, out-of-range
// and repeated entries.
__device__ __forceinline__ void request_token_choices(const int64_t* topk_idx, int t, int T, int K,
                                                      int E, int (&e)[kMaxTopk]) {
#pragma unroll
    for (int k = 0; k < kMaxTopk; ++k) {
        e[k] = -1;
        if (t < T && k < K) {
            const int v = (int)__ldg(topk_idx + (size_t)t * K + k);
            e[k] = (v >= 0 && v < E) ? v : -1;
        }
    }
}
__device__ __forceinline__ void drop_repeated_choices(int (&e)[kMaxTopk]) {
#pragma unroll
    for (int k = 1; k < kMaxTopk; ++k) {
        bool dup = false;
#pragma unroll
        for (int kk = 0; kk < k; ++kk) dup |= (e[kk] == e[k]);
        if (dup) e[k] = -1;
    }
}
__device__ __forceinline__ void load_token_choices(const int64_t* topk_idx, int t, int T, int K, int E,
                                                   int (&e)[kMaxTopk]) {
    request_token_choices(topk_idx, t, T, K, E, e);
    drop_repeated_choices(e);
}

// a chunk is `warps` x 32 tokens: warp w of the block takes tokens [32w, 32w + 32)
__global__ void __launch_bounds__(256) ep_layout_hist_kernel(LayoutParams p) {
    extern __shared__ int smem_i32[];
    int* hist = smem_i32;  // [E]
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int t = blockIdx.x * nthr + tid;
    int e[kMaxTopk];
    load_token_choices(p.topk_idx, t, p.T, p.K, p.E, e);
    for (int i = tid; i < p.E; i += nthr) hist[i] = 0;
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
#pragma unroll
    for (int k = 0; k < kMaxTopk; ++k)
        if (e[k] >= 0) atomicAdd(&hist[e[k]], 1);
    __syncthreads();
    for (int i = tid; i < p.E; i += nthr) p.chunk_hist[(size_t)blockIdx.x * p.E + i] = hist[i];
}

__global__ void __launch_bounds__(256) ep_layout_slot_kernel(LayoutParams p) {
    extern __shared__ int smem_i32[];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, words = nthr >> 5;
    int* base = smem_i32;                                          // [E] tokens of earlier chunks
    uint32_t* mask = reinterpret_cast<uint32_t*>(smem_i32 + p.E);  // [E][words], word w written by warp w only
    const int t = blockIdx.x * nthr + tid;
    int e[kMaxTopk];
    load_token_choices(p.topk_idx, t, p.T, p.K, p.E, e);
    for (int i = tid; i < p.E * words; i += nthr) mask[i] = 0;
    __syncthreads();
    // bit (expert, token): lanes of a warp that chose the same expert in the same
    // position k form a group; its lowest lane ORs the group into the warp's word
    for (int k = 0; k < p.K; ++k) {
        const unsigned key = e[k] >= 0 ? (unsigned)e[k] : (0x80000000u | lane);
        const unsigned grp = __match_any_sync(kFull, key);
        if (e[k] >= 0 && (int)(__ffs(grp) - 1) == lane) mask[e[k] * words + warp] |= grp;
        __syncwarp();
    }
    pdl_wait();
    pdl_launch_dependents();
    for (int i = tid; i < p.E; i += nthr) {
        // column sum over the earlier chunks, eight loads in flight at a time
        int sum = 0;
        for (int c0 = 0; c0 < (int)blockIdx.x; c0 += 8) {
            int v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = c0 + u < (int)blockIdx.x ? __ldcg(p.chunk_hist + (size_t)(c0 + u) * p.E + i) : 0;
#pragma unroll
            for (int u = 0; u < 8; ++u) sum += v[u];
        }
        base[i] = sum;
    }
    __syncthreads();
    if (t < p.T) {
        const unsigned lower = (1u << lane) - 1u;
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
            if (k >= p.K) break;
            int slot = -1;
            if (e[k] >= 0) {
                const uint32_t* m = mask + e[k] * words;
                slot = base[e[k]] + __popc(m[warp] & lower);
                for (int w = 0; w < warp; ++w) slot += __popc(m[w]);
            }
            p.slot[(size_t)t * p.K + k] = slot;
        }
    }
    if (blockIdx.x != gridDim.x - 1) return;
    // the block of the last chunk knows every total
    __syncthreads();
    for (int i = tid; i < p.E; i += nthr) {
        int c = base[i];
        for (int w = 0; w < words; ++w) c += __popc(mask[i * words + w]);
        base[i] = c;
        p.count[i] = c;
        if (p.recv_count) p.recv_count[i] = c;
        if (p.layout_range) p.layout_range[i] = c;  // begin 0 | count
    }
    if (p.rank_count == nullptr && p.expert_prefix == nullptr) return;
    __syncthreads();
    const int L = p.E / p.R;
    for (int r = warp; r < p.R; r += words) {
        int carry = 0;
        for (int b = 0; b < L; b += 32) {
            const int le = b + lane;
            const int c = le < L ? base[r * L + le] : 0;
            const int incl = warp_inclusive_scan(c, lane);
            if (le < L && p.expert_prefix) p.expert_prefix[r * L + le] = carry + incl - c;
            carry += __shfl_sync(kFull, incl, 31);
        }
        if (lane == 0 && p.rank_count) p.rank_count[r] = carry;
    }
}

// =============================================================================
// sending token rows (single rank and groups)
// =============================================================================
// One block per token (blocks stride over the tokens), one warp per 512-channel
// tile of the row. The block reads the bf16 row once (32 bytes per lane),
// quantises it in registers when FP8 is on, and stores it to the row of every
// selected expert's packed receive area: this GPU's (single rank, or an expert
// this rank owns) or a peer's, over NVLink.
//
// kFused: the position of the token among this rank's tokens for each of its
// experts is counted here instead of read from the layout kernel - every warp
// takes whole tokens of the (small) index matrix. The host uses it when one
// block per token fits the machine in one wave.
//
// What goes where for entry (t, k) with expert e, owner rank o, local expert le,
// row r = first row of this rank's segment in e + earlier tokens of this rank:
//   payload    -> o's receive rows   [le][r][H e4m3 | H bf16]
//   o == this rank: token index and scales go straight into the caller's
//                   src_info / transposed scales tensors;
//   o is a peer:    a side message [16 B: token index | 16 B of scales per 512
//                   channels] goes to o's side area [le][r]; o's receive duty
//                   moves it into its src_info / scales tensors.
struct SendView {
    const char* x;
    const int64_t* topk_idx;
    const int32_t* slot;
    int T, K, E, R, M, H, rank;
    int L, RM;
    int32_t* status;
    // rows this rank owns
    char* recv_x;
    float* recv_scales;
    int32_t* recv_src_info;
    int row_bytes;
    // groups only
    const uint64_t* beg;      // local words: first row of this rank's segment per expert
    uint32_t seq;
    WaitCfg wait;
    size_t rx_off, meta_off;
    int meta_stride;
    int32_t* rowmap;
    char* const* s_peer;      // shared-memory copies of the peer table and the mask
    const int* s_active;
};

// One pass of all warps over the whole index matrix. With kHist it leaves the
// whole-batch count per expert in hist[]; with t_own >= 0 it counts, for every
// expert of token t_own (kmap: expert -> k), the earlier tokens that chose it
// (s_before[k]). A repeated expert inside a token is counted once (lanes holding
// the same (token, expert) elect the lowest lane).
constexpr int kScanAhead = 4;

template <bool kHist, bool kAhead>
__device__ __forceinline__ void scan_index_matrix(const int64_t* topk_idx, int T, int K, int E,
                                                  int* hist, const int* kmap, int* s_before,
                                                  int t_own, const int (&e_ahead)[kScanAhead]) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const int tpw = 32 / K;  // tokens per warp pass (K <= 16)
    const int sk = lane % K, st = lane / K;
    const bool lane_used = st < tpw;
    auto count_pass = [&](int base, int e) {
        const int t2 = base + st;
        const bool valid = lane_used && t2 < T;
        if (!valid || e >= E) e = -1;
        const unsigned key = e >= 0 ? (((unsigned)st << 16) | (unsigned)e) : (0x80000000u | lane);
        const unsigned grp = __match_any_sync(kFull, key);
        if (e >= 0 && (int)(__ffs(grp) - 1) == lane) {
            if (kHist) atomicAdd(&hist[e], 1);
            if (t2 < t_own) {
                const int kk = kmap[e];
                if (kk >= 0) atomicAdd(&s_before[kk], 1);
            }
        }
    };
    if (kAhead) {
#pragma unroll
        for (int u = 0; u < kScanAhead; ++u) {
            const int base = (warp + u * nwarps) * tpw;
            if (base < T) count_pass(base, e_ahead[u]);
        }
    }
    for (int base = (warp + (kAhead ? kScanAhead : 0) * nwarps) * tpw; base < T;
         base += nwarps * tpw) {
        const int t2 = base + st;
        count_pass(base, (lane_used && t2 < T) ? (int)__ldg(topk_idx + (size_t)t2 * K + sk) : -1);
    }
}


// Requests the first kScanAhead passes of the scan (so the scan does not pay a
// memory round trip per pass).
__device__ __forceinline__ void scan_prefetch(const int64_t* topk_idx, int T, int K, bool on,
                                              int (&e_ahead)[kScanAhead]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int tpw = 32 / K;
    const int sk = lane % K, st = lane / K;
#pragma unroll
    for (int u = 0; u < kScanAhead; ++u) {
        const int t2 = (warp + u * nwarps) * tpw + st;
        e_ahead[u] = -1;
        if (on && st < tpw && t2 < T) e_ahead[u] = (int)__ldg(topk_idx + (size_t)t2 * K + sk);
    }
}

template <bool kFP8, bool kGroup, bool kFused>
__device__ __forceinline__ void send_tokens(const SendView& v, int first_token, int token_stride,
                                            int* hist /* fused && !group: [E] */,
                                            int* kmap /* fused: [E] */) {
    __shared__ char* s_dst[kMaxTopk];
    __shared__ char* s_meta[kMaxTopk];
    __shared__ int s_exp[kMaxTopk];
    __shared__ int s_le[kMaxTopk];
    __shared__ int s_row[kMaxTopk];
    __shared__ int s_before[kMaxTopk];
    __shared__ int s_raw[kMaxTopk];

    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    const int nchunks = v.H / 16;
    const int ntiles = (v.H + kTileChannels - 1) / kTileChannels;
    const int S = v.H / 128;

    for (int t = first_token; t < v.T; t += token_stride) {
        const char* xrow = v.x + (size_t)t * v.H * 2;
        V32 first = {};
        if (warp < ntiles && warp * 32 + lane < nchunks)
            first = ld32_readonly(xrow + (size_t)(warp * 32 + lane) * 32);
        // (in production a fused launch has one block per token; blocks that take
        // several tokens - in-process groups - scan once per token)
        const bool scan_now = kFused;
        int e_ahead[kScanAhead];
        scan_prefetch(v.topk_idx, v.T, v.K, scan_now, e_ahead);
        int my_slot = -1;
        if (tid < kMaxTopk) {
            int e = tid < v.K ? (int)__ldg(v.topk_idx + (size_t)t * v.K + tid) : -1;
            if (!kFused && tid < v.K) my_slot = __ldg(v.slot + (size_t)t * v.K + tid);
            s_raw[tid] = (e >= 0 && e < v.E) ? e : -1;
            s_before[tid] = 0;
        }
        __syncthreads();
        if (tid < kMaxTopk) {
            int e = s_raw[tid];
            for (int kk = 0; kk < tid; ++kk)
                if (s_raw[kk] == e) e = -1;  // a repeat of an earlier entry of this token
            s_exp[tid] = e;
            if (scan_now && e >= 0) kmap[e] = tid;
        }
        __syncthreads();
        if (scan_now) {
            if (kGroup)
                scan_index_matrix<false, true>(v.topk_idx, v.T, v.K, v.E, nullptr, kmap, s_before,
                                               t, e_ahead);
            else
                scan_index_matrix<true, true>(v.topk_idx, v.T, v.K, v.E, hist, kmap, s_before, t,
                                              e_ahead);
            __syncthreads();
        }
        if (tid < kMaxTopk) {
            char* dst = nullptr;
            char* meta = nullptr;
            int row = -1, le = 0;
            const int e = s_exp[tid];
            if (e >= 0) {
                const int s = kFused ? s_before[tid] : my_slot;
                if (s >= v.M) {
                    atomicOr(v.status, kStatusSlotRange);
                } else if (s >= 0) {
                    if (!kGroup) {
                        le = e;
                        row = s;
                        dst = v.recv_x + ((size_t)e * v.RM + s) * (size_t)v.row_bytes;
                    } else {
                        const int dr = e / v.L;
                        le = e - dr * v.L;
                        if (v.s_active[dr]) {
                            // the owner's answer: first row of this rank's segment
                            const uint32_t b = wait_word(v.beg + e, v.seq, v.wait, dr);
                            if (b) {
                                row = (int)(b - 1) + s;
                                if (row >= v.RM) {
                                    atomicOr(v.status, kStatusSlotRange);
                                    row = -1;
                                } else if (dr == v.rank) {
                                    dst = v.recv_x + ((size_t)le * v.RM + row) * (size_t)v.row_bytes;
                                } else {
                                    const size_t r = (size_t)le * v.RM + row;
                                    dst = v.s_peer[dr] + v.rx_off + r * (size_t)v.row_bytes;
                                    meta = v.s_peer[dr] + v.meta_off + r * (size_t)v.meta_stride;
                                }
                            }
                        }
                    }
                }
            }
            if (tid < v.K && v.rowmap != nullptr) v.rowmap[(size_t)t * v.K + tid] = row;
            if (scan_now && e >= 0) kmap[e] = -1;  // leave the table clean for the next token
            s_dst[tid] = dst;
            s_meta[tid] = meta;
            s_le[tid] = le;
            s_row[tid] = row;
        }
        __syncthreads();
        if (kGroup) MCEP_TRACE(0, 7);  // the owners' answers are in, rows can go
        // A repeated expert in a token's list was sent once; combine still adds
        // that row once per listing (mooncake_ep_kernel.cu:734-742 reads the
        // (expert, token) slot for every k), so the repeat records the same row.
        if (tid < v.K && v.rowmap != nullptr && s_exp[tid] < 0 && s_raw[tid] >= 0) {
            for (int kk = 0; kk < tid; ++kk)
                if (s_exp[kk] == s_raw[tid]) v.rowmap[(size_t)t * v.K + tid] = s_row[kk];
        }

        for (int tile = warp; tile < ntiles; tile += nwarps) {
            const int c = tile * 32 + lane;
            const bool act = c < nchunks;
            V32 cur = first;
            if (tile != warp) {
                cur = V32{};
                if (act) cur = ld32_readonly(xrow + (size_t)c * 32);
            }
            if (kFP8) {
                float sinv;
                const uint4 q = quantize16(cur, sinv);
                float4 sc;
                if (kGroup) {
                    sc.x = __shfl_sync(kFull, sinv, 0);
                    sc.y = __shfl_sync(kFull, sinv, 8);
                    sc.z = __shfl_sync(kFull, sinv, 16);
                    sc.w = __shfl_sync(kFull, sinv, 24);
                }
#pragma unroll 4
                for (int k = 0; k < v.K; ++k) {
                    char* d = s_dst[k];
                    if (d == nullptr) continue;
                    if (act) st16(d + (size_t)c * 16, q);
                    char* m = kGroup ? s_meta[k] : nullptr;
                    if (m != nullptr) {
                        if (lane == 0)
                            st16(m + kMetaHeaderBytes + (size_t)tile * 16,
                                 *reinterpret_cast<uint4*>(&sc));
                    } else if (act && (lane & 7) == 0) {
                        v.recv_scales[((size_t)s_le[k] * S + (c >> 3)) * v.RM + s_row[k]] = sinv;
                    }
                }
            } else {
#pragma unroll 4
                for (int k = 0; k < v.K; ++k) {
                    char* d = s_dst[k];
                    if (d == nullptr || !act) continue;
                    st32(d + (size_t)c * 32, cur);
                }
            }
        }
        if (tid < v.K && s_dst[tid] != nullptr) {
            if (kGroup && s_meta[tid] != nullptr)
                st16(s_meta[tid], make_uint4((uint32_t)t, 0u, 0u, 0u));
            else
                v.recv_src_info[(size_t)s_le[tid] * v.RM + s_row[tid]] = t;
        }
        __syncthreads();
    }
}

// =============================================================================
// single rank: dispatch writes the packed outputs directly
// =============================================================================
template <bool kFP8, bool kFused>
__global__ void __launch_bounds__(512) ep_dispatch_send_direct_kernel(DirectDispatchParams p) {
    extern __shared__ int smem_i32[];
    int* hist = smem_i32;        // [E] whole-batch counts (fused)
    int* kmap = smem_i32 + p.E;  // [E] expert -> k of this block's token (fused)
    const int tid = threadIdx.x, nthr = blockDim.x;
    pdl_wait();
    pdl_launch_dependents();
    if (kFused)
        for (int e = tid; e < p.E; e += nthr) hist[e] = 0, kmap[e] = -1;
    // (the token loop has a barrier before the first use of these tables; a
    // block without tokens only reads hist after the barrier below)
    SendView v = {};
    v.x = reinterpret_cast<const char*>(p.x), v.topk_idx = p.topk_idx, v.slot = p.slot;
    v.T = p.T, v.K = p.K, v.E = p.E, v.R = 1, v.M = p.M, v.H = p.H, v.rank = 0;
    v.L = p.E, v.RM = p.M, v.status = p.status;
    v.recv_x = reinterpret_cast<char*>(p.recv_x), v.recv_scales = p.recv_scales;
    v.recv_src_info = p.recv_src_info, v.row_bytes = p.H * (kFP8 ? 1 : 2);
    v.rowmap = p.rowmap;
    send_tokens<kFP8, false, kFused>(v, blockIdx.x, gridDim.x, hist, kmap);
    if (kFused) {
        // the receive layout of a single rank, spread over the grid. A block
        // without a token has not scanned: it has nothing to add (its share of
        // the experts is written by... itself, so it scans now).
        if ((int)blockIdx.x >= p.T) {
            __syncthreads();
            const int none[kScanAhead] = {-1, -1, -1, -1};
            scan_index_matrix<true, false>(p.topk_idx, p.T, p.K, p.E, hist, kmap, nullptr, -1, none);
            __syncthreads();
        }
        for (int e = blockIdx.x * nthr + tid; e < p.E; e += gridDim.x * nthr) {
            const int c = hist[e];
            p.recv_count[e] = c;
            p.layout_range[e] = c;  // begin 0 | count
        }
    }
}

// Single rank: rowmap[t][k] = packed row of (token t, expert topk[t][k]) as the
// handle records it.
__global__ void __launch_bounds__(256) ep_combine_invert_kernel(CombineInvertParams p) {
    const int RM = p.R * p.M;
    const long long total = (long long)p.L * p.M;
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int le = (int)(i / p.M), j = (int)(i - (long long)le * p.M);
        const long long lr = __ldg(p.layout_range + le * p.R + p.rank);
        const int cnt = (int)(lr & 0xffffffffll);
        if (j >= cnt) continue;
        const int row = (int)(lr >> 32) + j;
        if (row >= RM) {
            atomicOr(p.status, kStatusSlotRange);
            continue;
        }
        const int t = __ldg(p.src_info + (size_t)le * RM + row);
        if (t < 0 || t >= p.T) {
            atomicOr(p.status, kStatusBadSource);
            continue;
        }
        const int e = p.rank * p.L + le;
        for (int k = 0; k < p.K; ++k)
            if ((int)__ldg(p.topk_idx + (size_t)t * p.K + k) == e) p.rowmap[(size_t)t * p.K + k] = row;
    }
}

// =============================================================================
// weighted top-k reduction
// =============================================================================
// One block per token, one warp per 512-channel tile; each lane owns 16
// channels: up to K 32-byte loads in flight, fp32 FMA accumulation in k order,
// one bf16 rounding, one 32-byte store (mooncake_ep_kernel.cu:715-752).
// kDepth rows are requested before the first of them is used. s_ptr has kMaxTopk
// entries, null where nothing is to be added.
template <int kDepth, bool kReadOnly>
__device__ __forceinline__ void reduce_rows(const char* const* s_ptr, const float* s_w, int K,
                                            int H, void* out_row) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int nchunks = H / 16;
    const int ntiles = (H + kTileChannels - 1) / kTileChannels;
    for (int tile = warp; tile < ntiles; tile += nwarps) {
        const int c = tile * 32 + lane;
        if (c >= nchunks) continue;
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] = 0.f;
        for (int k0 = 0; k0 < K; k0 += kDepth) {
            V32 v[kDepth];
#pragma unroll
            for (int b = 0; b < kDepth; ++b) {
                const char* rp = s_ptr[k0 + b];
                if (rp != nullptr)
                    v[b] = kReadOnly ? ld32_readonly(rp + (size_t)c * 32)
                                     : ld32_coherent(rp + (size_t)c * 32);
            }
#pragma unroll
            for (int b = 0; b < kDepth; ++b) {
                if (s_ptr[k0 + b] == nullptr) continue;
                const float wk = s_w[k0 + b];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    acc[2 * i] = fmaf(bf16lo(v[b].w[i]), wk, acc[2 * i]);
                    acc[2 * i + 1] = fmaf(bf16hi(v[b].w[i]), wk, acc[2 * i + 1]);
                }
            }
        }
        st32(reinterpret_cast<char*>(out_row) + (size_t)c * 32, pack_bf16x16(acc));
    }
}

template <int kDepth>
__global__ void __launch_bounds__(512) ep_combine_reduce_direct_kernel(DirectCombineParams p) {
    static_assert(kMaxTopk % kDepth == 0, "the row batches must tile the top-k table");
    __shared__ const char* s_ptr[kMaxTopk];
    __shared__ float s_w[kMaxTopk];
    __shared__ int s_row[kMaxTopk];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    pdl_wait();
    pdl_launch_dependents();
    for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
        int e = -1, r = 0;
        float w = 0.f;
        if (tid < p.K) {
            e = (int)__ldg(p.topk_idx + (size_t)t * p.K + tid);
            w = __ldg(p.topk_weights + (size_t)t * p.K + tid);
            if (!p.search) r = __ldcg(p.rowmap + (size_t)t * p.K + tid);
        }
        if (p.search) {
            // Small batches: no separate inversion pass. Warp k looks the token
            // up in the handle itself - the segment of expert topk[t][k] - 32
            // entries of src_info at a time.
            for (int k = warp; k < p.K; k += nwarps) {
                const int ek = (int)__ldg(p.topk_idx + (size_t)t * p.K + k);
                int row = -1;
                if (ek >= 0 && ek < p.E) {
                    const long long lr = __ldg(p.layout_range + ek);
                    const int cnt = (int)(lr & 0xffffffffll), begin = (int)(lr >> 32);
                    for (int j0 = 0; j0 < cnt; j0 += 32) {
                        const int j = begin + j0 + lane;
                        const bool hit = j0 + lane < cnt && j < p.M &&
                                         __ldg(p.src_info + (size_t)ek * p.M + j) == t;
                        const unsigned m = __ballot_sync(kFull, hit);
                        if (m) {
                            row = begin + j0 + __ffs(m) - 1;
                            break;
                        }
                    }
                }
                if (lane == 0) s_row[k] = row;
            }
        }
        __syncthreads();  // s_row is in place; the previous token's rows are done with s_ptr
        if (tid < kMaxTopk) {
            const char* ptr = nullptr;
            if (p.search && tid < p.K) r = s_row[tid];
            if (tid < p.K && e >= 0 && e < p.E) {
                if (ld_volatile_s32(p.active_ranks) && r >= 0 && r < p.M)
                    ptr = reinterpret_cast<const char*>(p.x) + ((size_t)e * p.M + r) * p.H * 2;
            }
            s_ptr[tid] = ptr;
            s_w[tid] = w;
        }
        __syncthreads();
        reduce_rows<kDepth, true>(s_ptr, s_w, p.K, p.H,
                                  reinterpret_cast<char*>(p.combined_x) + (size_t)t * p.H * 2);
    }
}

// =============================================================================
// groups: dispatch
// =============================================================================
__device__ __forceinline__ void load_peer_tables(void* const* peer_base, const int32_t* active_ranks,
                                                 int R, int32_t* status, char** s_peer,
                                                 int* s_active) {
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        char* pb = reinterpret_cast<char*>(peer_base[r]);
        int a = ld_volatile_s32(active_ranks + r);
        if (a && pb == nullptr) {  // marked active but never mapped: leave it alone
            atomicOr(status, kStatusNoPeer);
            a = 0;
        }
        s_peer[r] = pb;
        s_active[r] = a;
    }
}

// The control block (block 0 of the send kernel).
//  1. announce: count of this rank's tokens per expert -> the expert's owner;
//  2. collect: for this rank's own experts, the counts of every active source
//     (bounded wait; a source that does not answer is marked inactive and
//     counts as zero);
//  3. fix the receive layout (source-rank order), write `layout_range` and
//     `recv_count`, leave the verdicts for the receive duty, and answer every
//     source with the first row of its segment in each of this rank's experts.
template <bool kFused>
__device__ __forceinline__ void dispatch_control(const GroupDispatchParams& p, int* smem_i32,
                                                 char* const* s_peer, const int* s_active,
                                                 int (&e)[kMaxTopk]) {
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int L = p.E / p.R, n = L * p.R;
    int* hist = smem_i32;                       // [E] (fused)
    int* s_cnt = smem_i32 + (kFused ? p.E : 0);  // [L*R]
    MCEP_TRACE(0, 1);
    if (kFused) {
        // one lane per token: its choices arrive in one memory round trip
        // (small batches: T <= 2 x the number of SMs, so one pass)
        // (the caller requested this thread's token before the peer tables)
        for (int i = tid; i < p.E; i += nthr) hist[i] = 0;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k)
            if (e[k] >= 0) atomicAdd(&hist[e[k]], 1);
        for (int t = tid + nthr; t < p.T; t += nthr) {
            load_token_choices(p.topk_idx, t, p.T, p.K, p.E, e);
#pragma unroll
            for (int k = 0; k < kMaxTopk; ++k)
                if (e[k] >= 0) atomicAdd(&hist[e[k]], 1);
        }
        __syncthreads();
    }
    for (int x = tid; x < p.E; x += nthr) {
        const int dr = x / L;
        if (!s_active[dr]) continue;
        const int c = kFused ? hist[x] : __ldg(p.count + x);
        uint64_t* wd = reinterpret_cast<uint64_t*>(s_peer[dr] + p.w.cnt_off) + (p.rank * L + (x - dr * L));
        st_relaxed_sys(wd, ((uint64_t)p.seq << 32) | (uint32_t)(c + 1));
    }
    MCEP_TRACE(0, 2);  // counts announced
    const uint64_t* my_cnt = reinterpret_cast<const uint64_t*>(p.local_base + p.w.cnt_off);
    for (int i = tid; i < n; i += nthr) {
        const int le = i / p.R, src = i - le * p.R;
        int c = -1;  // -1: nothing will come from this source (inactive, or given up on)
        if (s_active[src]) {
            const uint32_t v = wait_word(my_cnt + src * L + le, p.seq, p.wait, src);
            c = v ? (int)v - 1 : -1;
            if (c > p.M) {
                atomicOr(p.wait.status, kStatusSlotRange);
                c = 0;
            }
        }
        s_cnt[i] = c;
    }
    __syncthreads();
    MCEP_TRACE(0, 3);  // every source's counts are in
    // Every thread fixes its own (expert, source) entry: the rows of the lower
    // sources come first. The answer goes out at once; the outputs follow.
    for (int i = tid; i < n; i += nthr) {
        const int le = i / p.R, src = i - le * p.R;
        int begin = 0;
        for (int s2 = 0; s2 < src; ++s2) begin += max(s_cnt[le * p.R + s2], 0);
        // a source that is inactive, or went silent while its counts were
        // awaited, counts as zero and gets no answer
        const bool answered = s_cnt[i] >= 0;
        const int c = max(s_cnt[i], 0);
        if (answered) {
            uint64_t* wd = reinterpret_cast<uint64_t*>(s_peer[src] + p.w.beg_off) + (p.rank * L + le);
            st_relaxed_sys(wd, ((uint64_t)p.seq << 32) | (uint32_t)(begin + 1));
        }
        *reinterpret_cast<volatile uint64_t*>(p.res_cnt + i) = ((uint64_t)p.seq << 32) | (uint32_t)(c + 1);
        p.layout_range[i] = c ? (((int64_t)begin << 32) | (int64_t)c) : 0;
        if (src == p.R - 1) p.recv_count[le] = begin + c;
    }
    MCEP_TRACE(0, 4);  // answers are out
}

// Receive duty of dispatch, shared by `np` participants (blocks): rows that
// peers stored into this rank's receive area are complete once the source's
// payload word has arrived; their side messages are then moved into the
// caller's `src_info` and transposed `scales`, and - when the caller's recv_x
// is not the in-place tensor - the rows themselves are copied out.
// (Rows of experts this rank sent to itself need nothing: the sender wrote the
// final tensors.)
constexpr int kRowWarps = 8;

template <bool kFP8>
__device__ __forceinline__ void dispatch_recv_duty(const GroupDispatchParams& p, int j, int np,
                                                   int* smem_i32) {
    const int L = p.E / p.R, n = L * p.R;
    int* pre = smem_i32;          // [n + 1] rows to process per (expert, source), then prefix
    int* beg = smem_i32 + n + 1;  // [n] first row of each (expert, source)
    __shared__ int s_wt[32];
    __shared__ int s_ok[kMaxRanks];
    __shared__ int s_tot[kMaxRanks];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    const int RM = p.R * p.M;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    const int S = p.H / 128;
    for (int r = tid; r < p.R; r += nthr) s_tot[r] = 0;
    __syncthreads();
    // the control block's verdicts: what every source sends to every local expert
    for (int i = tid; i < n; i += nthr) {
        const uint32_t v = wait_local_word(p.res_cnt + i, p.seq, scaled(p.wait, 2));
        const int c = v ? (int)v - 1 : 0;
        pre[i] = c;
        if (c) atomicAdd(&s_tot[i % p.R], c);
    }
    __syncthreads();
    for (int le = tid; le < L; le += nthr) {
        int run = 0;
        for (int src = 0; src < p.R; ++src) {
            beg[le * p.R + src] = run;
            run += pre[le * p.R + src];
        }
    }
    __syncthreads();
    // rows this rank sent to itself need nothing; all of the above, and the
    // prefix below, is ready before the payload words are even looked at
    for (int i = tid; i < n; i += nthr)
        if (i % p.R == p.rank) pre[i] = 0;
    __syncthreads();
    block_exclusive_scan(pre, n, s_wt);
    // a peer's rows count once its payload word is here (one verdict per source
    // for all participants)
    for (int r = tid; r < p.R; r += nthr) {
        int ok = 0;
        if (r != p.rank && s_tot[r] > 0) {
            const uint64_t* flags = reinterpret_cast<const uint64_t*>(p.local_base + p.w.dflag_off);
            ok = resolve_flag(flags, p.res_dflag, r, p.seq, scaled(p.wait, 3), r,
                              np <= 80 || (j & 7) == (r & 7)) != 0;
        }
        s_ok[r] = ok;
    }
    __syncthreads();
    MCEP_TRACE(1, 1);  // every payload word has a verdict
    const int total = pre[n];
    const char* rx = p.local_base + p.rx_off;
    const char* mt = p.local_base + p.meta_off;
    // rows are dealt to the participants one at a time (warp w of participant j
    // takes row w * np + j, ...): a batch with fewer rows than there are warps
    // still spreads over all of them
    for (int g = warp * np + j; g < total; g += np * nwarps) {
        const int i = find_segment(pre, n, g);
        const int le = i / p.R;
        if (!s_ok[i - le * p.R]) continue;  // a source that was given up on
        const int row = beg[i] + (g - pre[i]);
        if (row >= RM) {
            if (lane == 0) atomicOr(p.wait.status, kStatusSlotRange);
            continue;
        }
        const size_t r = (size_t)le * RM + row;
        const char* meta = mt + r * (size_t)p.meta_stride;
        // one round trip: the token index and 16 bytes (four scales) per lane are
        // requested together, then scattered into the transposed scales
        const int tok = lane == 31 ? ld_s32_coherent(meta) : 0;
        if (kFP8) {
            for (int q0 = 0; q0 < ntiles; q0 += 32) {
                const int q = q0 + lane;
                if (q >= ntiles) continue;
                const uint4 sc = ld16_coherent(meta + kMetaHeaderBytes + (size_t)q * 16);
                const uint32_t w4[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (4 * q + u < S)
                        p.recv_scales[((size_t)le * S + 4 * q + u) * RM + row] = __uint_as_float(w4[u]);
            }
        }
        if (lane == 31) p.recv_src_info[r] = tok;
        if (!p.copy_rows) continue;
        const char* src = rx + r * (size_t)p.row_bytes;
        char* out = reinterpret_cast<char*>(p.recv_x) + r * (size_t)p.row_bytes;
        if (kFP8) {
            constexpr int kB = 8;  // 8 x 16 B per lane in flight
            for (int t0 = 0; t0 < ntiles; t0 += kB) {
                uint4 v[kB];
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks) v[b] = ld16_coherent(src + (size_t)c * 16);
                }
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks) st16(out + (size_t)c * 16, v[b]);
                }
            }
        } else {
            constexpr int kB = 4;  // 4 x 32 B per lane in flight
            for (int t0 = 0; t0 < ntiles; t0 += kB) {
                V32 v[kB];
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks) v[b] = ld32_coherent(src + (size_t)c * 32);
                }
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks) st32(out + (size_t)c * 32, v[b]);
                }
            }
        }
    }
    MCEP_TRACE(1, 2);
}

// Participants of the receive duty inside the one-launch kernel: the control
// block and the last sender blocks to finish (at most this many).
constexpr int kRecvHelpers = 64;

// kPhases: 1 = control + send; 3 = control + send + receive duty (one launch).
// `bid` of `nblocks`: the block's place in its rank's share of the grid (the
// whole grid, except for in-process groups where one launch carries all ranks).
template <bool kFP8, bool kFused, int kPhases>
__device__ __forceinline__ void dispatch_body(const GroupDispatchParams& p, int bid, int nblocks,
                                              int* smem_i32) {
    __shared__ char* s_peer[kMaxRanks];
    __shared__ int s_active[kMaxRanks];
    __shared__ int s_ticket;
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int nsend = nblocks - 1;
    const int nh = nsend < kRecvHelpers ? nsend : kRecvHelpers;
    MCEP_TRACE(0, 0);
    // the control block counts with one lane per token: its token's choices are
    // requested first, so they travel while the peer tables are read
    int ctl_choices[kMaxTopk];
    if (kFused && bid == 0) request_token_choices(p.topk_idx, tid, p.T, p.K, p.E, ctl_choices);
    load_peer_tables(p.peer_base, p.wait.active_ranks, p.R, p.wait.status, s_peer, s_active);
    if (kFused && bid == 0) drop_repeated_choices(ctl_choices);

    if (bid == 0) {
        __syncthreads();
        dispatch_control<kFused>(p, smem_i32, s_peer, s_active, ctl_choices);
        if (kPhases == 3) {
            __syncthreads();
            dispatch_recv_duty<kFP8>(p, nh, nh + 1, smem_i32);
        }
        return;
    }

    int* kmap = smem_i32;  // [E] (fused)
    if (kFused)
        for (int e = tid; e < p.E; e += nthr) kmap[e] = -1;
    const int sid = bid - 1;
    // (the token loop has barriers of its own before it reads the tables above;
    // a block without tokens reads them only after the barrier below)
    SendView v = {};
    v.x = reinterpret_cast<const char*>(p.x), v.topk_idx = p.topk_idx, v.slot = p.slot;
    v.T = p.T, v.K = p.K, v.E = p.E, v.R = p.R, v.M = p.M, v.H = p.H, v.rank = p.rank;
    v.L = p.E / p.R, v.RM = p.R * p.M, v.status = p.wait.status;
    v.recv_x = reinterpret_cast<char*>(p.recv_x), v.recv_scales = p.recv_scales;
    v.recv_src_info = p.recv_src_info, v.row_bytes = p.row_bytes;
    v.beg = reinterpret_cast<const uint64_t*>(p.local_base + p.w.beg_off);
    v.seq = p.seq, v.wait = scaled(p.wait, 2), v.rx_off = p.rx_off, v.meta_off = p.meta_off;
    v.meta_stride = p.meta_stride, v.rowmap = p.rowmap, v.s_peer = s_peer, v.s_active = s_active;
    send_tokens<kFP8, true, kFused>(v, sid, nsend, nullptr, kmap);
    MCEP_TRACE(0, 5);  // all rows of this block are issued

    // Completion. Rows are not fenced one by one: the block issues ONE
    // system-scope fence for everything it stored (it costs microseconds even
    // when idle), then takes a ticket. Whoever takes the last ticket has,
    // through the counter, observed every block's fence - all of this rank's
    // rows are performed system-wide - and tells every peer with one word.
    __syncthreads();
    if (tid == 0) {
        if (sid < p.T) __threadfence_system();
        s_ticket = (int)atomicAdd(p.ticket, 1u);
    }
    __syncthreads();
    MCEP_TRACE(0, 6);  // the fence has returned
    const int ticket = s_ticket;
    if (ticket == nsend - 1) {
        if (tid == 0) *p.ticket = 0;
        __threadfence();
        for (int r = tid; r < p.R; r += nthr) {
            if (r == p.rank || !s_active[r] || !ld_volatile_s32(p.wait.active_ranks + r)) continue;
            uint64_t* f = reinterpret_cast<uint64_t*>(s_peer[r] + p.w.dflag_off) + p.rank;
            st_relaxed_sys(f, ((uint64_t)p.seq << 32) | 1u);
        }
    }
    if (kPhases == 3 && ticket >= nsend - nh) {
        __syncthreads();
        dispatch_recv_duty<kFP8>(p, ticket - (nsend - nh), nh + 1, smem_i32);
    }
}

// Graph mode: a captured launch is replayed with the arguments it was captured
// with, so the call's sequence number cannot be one of them; it is read from the
// device word the host named (stable until the call's last kernel has finished:
// the word of the other parity belongs to the other call that may be in flight).
template <typename Params>
__device__ __forceinline__ void resolve_seq(Params& p) {
    if (p.seq_ptr != nullptr) p.seq = *reinterpret_cast<const volatile uint32_t*>(p.seq_ptr);
}

__global__ void ep_advance_seq_kernel(uint32_t* word) { *word += 2; }

// One thread per rank: tell that rank "I am here", then wait until it has said
// the same. Bounded: a rank that never comes raises the hard-timeout status bit
// and the others go on.
__global__ void __launch_bounds__(kMaxRanks) ep_barrier_kernel(BarrierParams p) {
    const int r = threadIdx.x;
    if (r >= p.R || r == p.rank) return;
    if (p.active_ranks != nullptr && !ld_volatile_s32(p.active_ranks + r)) return;
    char* peer = reinterpret_cast<char*>(p.peer_base[r]);
    if (peer == nullptr) return;
    st_release_sys(reinterpret_cast<uint64_t*>(peer + p.bar_off) + p.rank, (uint64_t)p.epoch);
    const uint64_t* mine = reinterpret_cast<const uint64_t*>(p.local_base + p.bar_off) + r;
    const uint64_t start = globaltimer_ns();
    // (a peer that has left this barrier may already have announced the next one)
    while ((int32_t)((uint32_t)ld_acquire_sys(mine) - p.epoch) < 0) {
        if ((int64_t)(globaltimer_ns() - start) > p.hard_timeout_ns) {
            atomicOr(p.status, kStatusHardTimeout);
            return;
        }
    }
}

template <bool kFP8, bool kFused, int kPhases>
__global__ void __launch_bounds__(512) ep_dispatch_kernel(GroupDispatchParams p) {
    extern __shared__ int smem_i32[];
    pdl_wait();
    pdl_launch_dependents();
    resolve_seq(p);
    dispatch_body<kFP8, kFused, kPhases>(p, blockIdx.x, gridDim.x, smem_i32);
}

// In-process groups (several logical ranks on one GPU): the ranks' kernels wait
// for one another, so they cannot be separate launches - nothing would
// guarantee that they run at the same time. ONE cooperative launch carries all
// ranks: consecutive runs of `per_rank` blocks do the work of one rank each.
template <bool kFP8, bool kFused, int kPhases>
__global__ void __launch_bounds__(512)
    ep_dispatch_multi_kernel(const GroupDispatchParams* ps, int per_rank) {
    extern __shared__ int smem_i32[];
    __shared__ GroupDispatchParams s_p;
    const int which = blockIdx.x / per_rank;
    if (threadIdx.x == 0) s_p = ps[which];
    __syncthreads();
    dispatch_body<kFP8, kFused, kPhases>(s_p, blockIdx.x - which * per_rank, per_rank, smem_i32);
}

template <bool kFP8>
__global__ void __launch_bounds__(kRowWarps * 32, 4) ep_dispatch_recv_kernel(GroupDispatchParams p) {
    extern __shared__ int smem_i32[];
    pdl_wait();
    pdl_launch_dependents();
    resolve_seq(p);
    MCEP_TRACE(1, 0);
    dispatch_recv_duty<kFP8>(p, blockIdx.x, gridDim.x, smem_i32);
}

// =============================================================================
// groups: combine
// =============================================================================
// Publish duty, shared by `np` participants: rows of expert outputs that peers
// will ask for (every segment of the handle whose source is another rank) are
// copied into this rank's combine input in symmetric memory, same [expert][row]
// position; one system fence per block, a ticket, and whoever finishes last
// tells every peer. With zero copy the caller's kernels wrote the rows there
// already and only the word is sent.
__device__ __forceinline__ void combine_publish_duty(const GroupCombineParams& p, int j, int np,
                                                     int* smem_i32, char* const* s_peer,
                                                     const int* s_active) {
    const int L = p.E / p.R, n = L * p.R;
    int* pre = smem_i32;  // [n + 1]
    __shared__ int s_wt[32];
    __shared__ int s_last;
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    const int RM = p.R * p.M;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    bool stored = false;
    if (!p.zero_copy) {
        int* beg = smem_i32 + n + 1;  // [n] first row of each (expert, source) segment
        for (int i = tid; i < n; i += nthr) {
            const int src = i % p.R;
            const long long lr = __ldg(p.layout_range + i);
            int c = (int)(lr & 0xffffffffll);
            if (src == p.rank || !s_active[src]) c = 0;
            pre[i] = c;
            beg[i] = (int)(lr >> 32);
        }
        __syncthreads();
        block_exclusive_scan(pre, n, s_wt);
        const int total = pre[n];
        const char* xb = reinterpret_cast<const char*>(p.x);
        char* cin = p.local_base + p.cin_off;
        // A work item is a run of tiles of one row, sized so that the rows spread
        // over every warp of the participants and an item's loads are all in
        // flight at once (8 x 32 B per lane): the copy costs one memory round trip.
        constexpr int kB = 8;
        const int warps_total = np * nwarps;
        int parts = total > 0 ? warps_total / total : 1;
        if (parts < 1) parts = 1;
        if (parts > ntiles) parts = ntiles;
        int tpp = (ntiles + parts - 1) / parts;  // tiles per item
        if (tpp > kB && parts < ntiles) tpp = kB;
        parts = (ntiles + tpp - 1) / tpp;
        const long long items = (long long)total * parts;
        for (long long g = (long long)warp * np + j; g < items; g += (long long)np * nwarps) {
            const int rg = (int)(g / parts), part = (int)(g - (long long)rg * parts);
            const int i = find_segment(pre, n, rg);
            const int le = i / p.R;
            const int row = beg[i] + (rg - pre[i]);
            if (row >= RM) {
                if (lane == 0) atomicOr(p.wait.status, kStatusSlotRange);
                continue;
            }
            const size_t off = ((size_t)le * RM + row) * (size_t)p.H * 2;
            const int t_end = min(ntiles, (part + 1) * tpp);
            for (int t0 = part * tpp; t0 < t_end; t0 += kB) {
                V32 v[kB];
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < t_end && c < nchunks) v[b] = ld32_readonly(xb + off + (size_t)c * 32);
                }
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < t_end && c < nchunks) st32(cin + off + (size_t)c * 32, v[b]);
                }
            }
            stored = true;
        }
    }
    // One fence for the block's rows, then the ticket (see the dispatch kernel).
    // The rows were stored to THIS GPU's memory and peers read them through this
    // GPU's L2, so a device-scope fence (about 1 us) is enough to order them
    // before the word that goes out to the peers; the system-scope one (4 us and
    // more) is for stores that cross NVLink.
    const int any = __syncthreads_or(stored ? 1 : 0);
    MCEP_TRACE(2, 3);  // this block's rows are copied
    if (tid == 0) {
        if (any || (p.zero_copy && j == 0)) __threadfence();
        s_last = (atomicAdd(p.ticket, 1u) == (unsigned)(np - 1));
        if (s_last) *p.ticket = 0;
    }
    __syncthreads();
    if (s_last) {
        __threadfence();
        for (int r = tid; r < p.R; r += nthr) {
            if (r == p.rank || !s_active[r]) continue;
            uint64_t* f = reinterpret_cast<uint64_t*>(s_peer[r] + p.w.cflag_off) + p.rank;
            st_relaxed_sys(f, ((uint64_t)p.seq << 32) | 1u);
        }
    }
}

// Reduce duty: one block per token. Row k of token t lives at the owner of
// expert topk[t][k], at the row the dispatch call recorded; it is read from
// there (a peer's combine input over NVLink once that peer's word has arrived,
// or this rank's own expert output) and the K rows are reduced in registers.
// An owner that is inactive, or whose word does not arrive in time (it is then
// marked inactive), contributes nothing (mooncake_ep_kernel.cu:685-699, 728-732).
__device__ __forceinline__ void combine_reduce_duty(const GroupCombineParams& p, int first_token,
                                                    int token_stride, char* const* s_peer) {
    __shared__ const char* s_ptr[kMaxTopk];
    __shared__ float s_w[kMaxTopk];
    const int tid = threadIdx.x;
    const int L = p.E / p.R, RM = p.R * p.M;
    const uint64_t* flags = reinterpret_cast<const uint64_t*>(p.local_base + p.w.cflag_off);
    const char* own = p.zero_copy ? p.local_base + p.cin_off : reinterpret_cast<const char*>(p.x);
    for (int t = first_token; t < p.T; t += token_stride) {
        if (tid < kMaxTopk) {
            const char* ptr = nullptr;
            float w = 0.f;
            if (tid < p.K) {
                const int e = (int)__ldg(p.topk_idx + (size_t)t * p.K + tid);
                w = __ldg(p.topk_weights + (size_t)t * p.K + tid);
                const int row = __ldcg(p.rowmap + (size_t)t * p.K + tid);
                if (e >= 0 && e < p.E && row >= 0 && row < RM) {
                    const int o = e / L, le = e - o * L;
                    const size_t off = ((size_t)le * RM + row) * (size_t)p.H * 2;
                    if (o == p.rank) {
                        if (ld_volatile_s32(p.wait.active_ranks + o)) ptr = own + off;
                    } else if (ld_volatile_s32(p.wait.active_ranks + o) && s_peer[o] != nullptr) {
                        const uint32_t v = resolve_flag(flags, p.res_cflag, o, p.seq, p.wait, o,
                                                        ((first_token + o) & 7) == 0);
                        if (v && ld_volatile_s32(p.wait.active_ranks + o))
                            ptr = s_peer[o] + p.cin_off + off;
                    }
                }
            }
            s_ptr[tid] = ptr;
            s_w[tid] = w;
        }
        __syncthreads();
        if (t == first_token) MCEP_TRACE(2, 4);  // the owners' words are in, rows can be read
        reduce_rows<8, false>(s_ptr, s_w, p.K, p.H,
                              reinterpret_cast<char*>(p.combined_x) + (size_t)t * p.H * 2);
        __syncthreads();  // the rows are done with s_ptr
    }
}

// kPhases: 1 = publish, 2 = reduce, 3 = both in one launch.
template <int kPhases>
__device__ __forceinline__ void combine_body(const GroupCombineParams& p, int bid, int nblocks,
                                             int* smem_i32) {
    __shared__ char* s_peer[kMaxRanks];
    __shared__ int s_active[kMaxRanks];
    MCEP_TRACE(2, 0);
    load_peer_tables(p.peer_base, p.wait.active_ranks, p.R, p.wait.status, s_peer, s_active);
    __syncthreads();
    if (kPhases & 1) combine_publish_duty(p, bid, nblocks, smem_i32, s_peer, s_active);
    MCEP_TRACE(2, 1);
    if (kPhases & 2) {
        __syncthreads();
        combine_reduce_duty(p, bid, nblocks, s_peer);
    }
    MCEP_TRACE(2, 2);
}

template <int kPhases>
__global__ void __launch_bounds__(512) ep_combine_kernel(GroupCombineParams p) {
    extern __shared__ int smem_i32[];
    pdl_wait();
    pdl_launch_dependents();
    resolve_seq(p);
    combine_body<kPhases>(p, blockIdx.x, gridDim.x, smem_i32);
}

// All logical ranks of an in-process group in one cooperative launch (see
// ep_dispatch_multi_kernel).
__global__ void __launch_bounds__(512)
    ep_combine_multi_kernel(const GroupCombineParams* ps, int per_rank) {
    extern __shared__ int smem_i32[];
    __shared__ GroupCombineParams s_p;
    const int which = blockIdx.x / per_rank;
    if (threadIdx.x == 0) s_p = ps[which];
    __syncthreads();
    combine_body<3>(s_p, blockIdx.x - which * per_rank, per_rank, smem_i32);
}

// threads per block: one warp per tile, at most 16 warps
inline int block_threads(int H, int at_least = 32) {
    int ntiles = (H + kTileChannels - 1) / kTileChannels;
    if (ntiles > 16) ntiles = 16;
    if (ntiles < 1) ntiles = 1;
    int t = ntiles * 32;
    return t < at_least ? at_least : t;
}
// how many blocks of this kernel are resident at a time on the whole device
template <typename K>
inline long long resident_blocks(K kernel, int threads, size_t smem, const LaunchCtx& ctx) {
    // the occupancy query is not free: remember the answer per (kernel, block, smem)
    static std::mutex mu;
    static std::map<std::tuple<const void*, int, size_t>, int> cache;
    int per_sm = 0;
    {
        std::lock_guard<std::mutex> lk(mu);
        auto key = std::make_tuple(reinterpret_cast<const void*>(kernel), threads, smem);
        auto it = cache.find(key);
        if (it != cache.end()) {
            per_sm = it->second;
        } else {
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) !=
                    cudaSuccess ||
                per_sm < 1) {
                cudaGetLastError();
                per_sm = 1;
            }
            cache[key] = per_sm;
        }
    }
    return (long long)ctx.num_sms * per_sm;
}
// a grid that fills the machine once (blocks stride over the work items)
template <typename K>
inline int persistent_grid(long long items, K kernel, int threads, size_t smem, const LaunchCtx& ctx) {
    const long long cap = resident_blocks(kernel, threads, smem, ctx);
    long long g = items < cap ? items : cap;
    return (int)(g < 1 ? 1 : g);
}

}  // namespace kernels
using namespace kernels;

// =============================================================================
// launchers
// =============================================================================
// The chunked route: chunks of up to 256 tokens (fewer when the per-chunk bitmap
// of all experts would not fit 48 KB of shared memory), at most 128 chunks, and
// per-chunk histograms that fit the scratch the caller gave.
static bool layout_chunking(const LayoutParams& p, int* chunk_tokens, int* words, int* chunks) {
    if (p.chunk_hist == nullptr || p.T < 512) return false;
    int w = (int)(12288 / p.E) - 1;  // (1 + w) * E ints of shared memory, 48 KB at most
    if (w > 8) w = 8;
    if (w < 1) return false;
    const int ct = w * 32;
    const int c = (p.T + ct - 1) / ct;
    if (c > 128 || (size_t)c * p.E > p.chunk_hist_entries) return false;
    *chunk_tokens = ct, *words = w, *chunks = c;
    return true;
}

cudaError_t launch_layout(const LayoutParams& p, const LaunchCtx& ctx) {
    int chunk_tokens = 0, cwords = 0, chunks = 0;
    if (layout_chunking(p, &chunk_tokens, &cwords, &chunks)) {
        cudaError_t e = launch("ep_layout_hist", ep_layout_hist_kernel, dim3(chunks),
                               dim3(chunk_tokens), (size_t)p.E * sizeof(int), ctx, p);
        if (e != cudaSuccess) return e;
        LaunchCtx chained = ctx;
        chained.pdl = true;
        return launch("ep_layout_slot", ep_layout_slot_kernel, dim3(chunks), dim3(chunk_tokens),
                      (size_t)p.E * (1 + cwords) * sizeof(int), chained, p);
    }
    const int words = (p.T + 31) / 32 > 0 ? (p.T + 31) / 32 : 1;
    const long long n = (long long)p.T * p.K;
    // Every block reads the whole index matrix, so the number of blocks trades
    // parallelism against L2 traffic: keep blocks * n * 8 bytes around 8 MB.
    long long max_blocks = n > 0 ? (1ll << 20) / n : ctx.num_sms;
    if (max_blocks < 8) max_blocks = 8;
    if (max_blocks > ctx.num_sms) max_blocks = ctx.num_sms;
    int epc = (int)((p.E + max_blocks - 1) / max_blocks);
    if (epc < 1) epc = 1;
    const size_t budget = 200 * 1024;
    while (epc > 1 && (size_t)epc * words * 8 > budget) --epc;
    const size_t smem = (size_t)epc * words * 8;
    if (smem > budget) return cudaErrorInvalidValue;  // > 819k tokens per rank
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(ep_routing_layout_kernel,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
    }
    int threads = 128;
    while (threads < 1024 && threads * 4 < n) threads <<= 1;
    const int grid = (p.E + epc - 1) / epc;
    return launch("ep_routing_layout", ep_routing_layout_kernel, dim3(grid), dim3(threads), smem,
                  ctx, p, epc, words);
}

bool can_fuse_layout(int T, int K, int E, int num_sms) {
    // one block per token, all resident at once even at two blocks per SM, an
    // index matrix small enough to be scanned by every block, and expert tables
    // that fit the static shared-memory budget
    return (long long)T * K <= 4096 && T <= num_sms * 2 && E <= 2048;
}

cudaError_t launch_direct_dispatch(const DirectDispatchParams& p, const LaunchCtx& ctx) {
    const int threads = block_threads(p.H);
    const size_t smem = (size_t)(p.fused ? 2 * p.E : 0) * sizeof(int);
    void (*k)(DirectDispatchParams) = nullptr;
    switch ((p.use_fp8 ? 2 : 0) | (p.fused ? 1 : 0)) {
        case 0: k = ep_dispatch_send_direct_kernel<false, false>; break;
        case 1: k = ep_dispatch_send_direct_kernel<false, true>; break;
        case 2: k = ep_dispatch_send_direct_kernel<true, false>; break;
        default: k = ep_dispatch_send_direct_kernel<true, true>; break;
    }
    const int grid = p.fused ? (p.T > 0 ? p.T : 1) : persistent_grid(p.T, k, threads, smem, ctx);
    return launch("ep_dispatch_send_direct", k, dim3(grid), dim3(threads), smem, ctx, p);
}

cudaError_t launch_combine_invert(const CombineInvertParams& p, const LaunchCtx& ctx) {
    const long long total = (long long)p.L * p.M;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)ctx.num_sms * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return launch("ep_combine_invert", ep_combine_invert_kernel, dim3((int)blocks), dim3(256), 0,
                  ctx, p);
}

cudaError_t launch_direct_combine(const DirectCombineParams& p, const LaunchCtx& ctx) {
    const int threads = block_threads(p.H);
    const bool deep = p.T <= ctx.num_sms;  // one block per SM at most: spend registers on loads in flight
    auto k = deep ? ep_combine_reduce_direct_kernel<8> : ep_combine_reduce_direct_kernel<4>;
    const int grid = persistent_grid(p.T, k, threads, 0, ctx);
    return launch("ep_combine_reduce_direct", k, dim3(grid), dim3(threads), 0, ctx, p);
}

// ---- groups -----------------------------------------------------------------------
namespace {

using DispatchKernel = void (*)(GroupDispatchParams);

template <int kPhases>
DispatchKernel pick_dispatch(bool fp8, bool fused) {
    switch ((fp8 ? 2 : 0) | (fused ? 1 : 0)) {
        case 0: return ep_dispatch_kernel<false, false, kPhases>;
        case 1: return ep_dispatch_kernel<false, true, kPhases>;
        case 2: return ep_dispatch_kernel<true, false, kPhases>;
        default: return ep_dispatch_kernel<true, true, kPhases>;
    }
}

size_t dispatch_smem(const GroupDispatchParams& p, bool with_recv) {
    const size_t n = (size_t)p.E;  // L * R
    const size_t control = (size_t)(p.fused ? p.E : 0) + 2 * n;
    const size_t sender = p.fused ? (size_t)p.E : 0;
    const size_t recv = with_recv ? 2 * n + 1 : 0;
    size_t m = control > sender ? control : sender;
    if (recv > m) m = recv;
    return m * sizeof(int);
}

}  // namespace

bool group_call_can_be_one_kernel(int T, int K, int E, int num_sms) {
    // a small batch: one block per token plus the control block (the launcher
    // falls back to two launches when that many blocks are not resident at once)
    return can_fuse_layout(T, K, E, num_sms) && T + 1 <= 2 * num_sms;
}

cudaError_t launch_group_dispatch(const GroupDispatchParams& p, const LaunchCtx& ctx) {
    const int threads = block_threads(p.H, 256);
    const size_t smem = dispatch_smem(p, true);
    auto k = pick_dispatch<3>(p.use_fp8 != 0, true);
    const int grid = 1 + (p.T > 0 ? p.T : 1);
    if (grid > resident_blocks(k, threads, smem, ctx)) return cudaErrorInvalidConfiguration;
    return launch("ep_dispatch", k, dim3(grid), dim3(threads), smem, ctx, p);
}

cudaError_t launch_group_dispatch_send(const GroupDispatchParams& p, const LaunchCtx& ctx) {
    const int threads = block_threads(p.H, 256);
    const size_t smem = dispatch_smem(p, false);
    auto k = pick_dispatch<1>(p.use_fp8 != 0, p.fused != 0);
    // the control block, then one block per token (fused) or a resident wave
    int senders;
    if (p.fused) {
        senders = p.T > 0 ? p.T : 1;
    } else {
        long long cap = resident_blocks(k, threads, smem, ctx) - 1;
        if (cap < 1) cap = 1;
        senders = (int)(p.T < cap ? (p.T > 0 ? p.T : 1) : cap);
    }
    return launch("ep_dispatch_send", k, dim3(1 + senders), dim3(threads), smem, ctx, p);
}

cudaError_t launch_group_dispatch_recv(const GroupDispatchParams& p, const LaunchCtx& ctx) {
    const int threads = kRowWarps * 32;
    const size_t smem = (size_t)(2 * p.E + 1) * sizeof(int);
    auto k = p.use_fp8 ? ep_dispatch_recv_kernel<true> : ep_dispatch_recv_kernel<false>;
    // The row count is only known on the device. Under even routing a rank
    // receives about what it sends; the grid is sized for twice that - blocks
    // stride, so a skewed or larger load is still covered - and never beyond
    // one resident wave. Without a row copy the duty is light: fewer blocks.
    long long rows = 2ll * (p.T * p.K > 64 ? p.T * p.K : 64);
    const long long worst = (long long)p.E * p.M;
    if (rows > worst) rows = worst;
    long long blocks = (rows + kRowWarps - 1) / kRowWarps;
    if (!p.copy_rows && blocks > 2ll * ctx.num_sms) blocks = 2ll * ctx.num_sms;
    const int grid = persistent_grid(blocks, k, threads, smem, ctx);
    return launch("ep_dispatch_recv", k, dim3(grid), dim3(threads), smem, ctx, p);
}

cudaError_t launch_group_combine(const GroupCombineParams& p, const LaunchCtx& ctx) {
    const int threads = block_threads(p.H, 256);
    const size_t smem = (size_t)(2 * p.E + 1) * sizeof(int);
    auto k = ep_combine_kernel<3>;
    // one block per token for the reduce duty, and enough blocks for this rank's
    // share of the publish duty when it has few tokens of its own
    long long want = p.T > 64 ? p.T : 64;
    const int grid = persistent_grid(want, k, threads, smem, ctx);
    return launch("ep_combine", k, dim3(grid), dim3(threads), smem, ctx, p);
}

cudaError_t launch_group_combine_publish(const GroupCombineParams& p, const LaunchCtx& ctx) {
    const int threads = kRowWarps * 32;
    const size_t smem = (size_t)(2 * p.E + 1) * sizeof(int);
    auto k = ep_combine_kernel<1>;
    long long blocks = 1;
    if (!p.zero_copy) {
        const long long rows = (long long)p.E * p.M;  // L * R * M
        blocks = (rows + kRowWarps - 1) / kRowWarps;
    }
    const int grid = persistent_grid(blocks, k, threads, smem, ctx);
    return launch("ep_combine_publish", k, dim3(grid), dim3(threads), smem, ctx, p);
}

cudaError_t launch_group_combine_reduce(const GroupCombineParams& p, const LaunchCtx& ctx) {
    const int threads = block_threads(p.H);
    auto k = ep_combine_kernel<2>;
    const int grid = persistent_grid(p.T, k, threads, 0, ctx);
    return launch("ep_combine_reduce", k, dim3(grid), dim3(threads), 0, ctx, p);
}

cudaError_t launch_barrier(const BarrierParams& p, const LaunchCtx& ctx) {
    LaunchCtx plain = ctx;
    plain.pdl = false;
    return launch("ep_barrier", ep_barrier_kernel, dim3(1), dim3(kMaxRanks), 0, plain, p);
}

cudaError_t launch_advance_seq(uint32_t* word, const LaunchCtx& ctx) {
    LaunchCtx plain = ctx;
    plain.pdl = false;  // ordinary stream order: after everything the call launched
    return launch("ep_advance_seq", ep_advance_seq_kernel, dim3(1), dim3(1), 0, plain, word);
}

// ---- in-process groups: all ranks in one cooperative launch ------------------------
namespace {

template <typename... KArgs, typename... Args>
cudaError_t launch_cooperative(const char* name, void (*kernel)(KArgs...), int grid, int threads,
                               size_t smem, const LaunchCtx& ctx, Args... args) {
    (void)name;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, args...);
    if (err == cudaSuccess) g_launches.fetch_add(1);
    return err;
}

using DispatchMultiKernel = void (*)(const GroupDispatchParams*, int);

template <int kPhases>
DispatchMultiKernel pick_dispatch_multi(bool fp8, bool fused) {
    switch ((fp8 ? 2 : 0) | (fused ? 1 : 0)) {
        case 0: return ep_dispatch_multi_kernel<false, false, kPhases>;
        case 1: return ep_dispatch_multi_kernel<false, true, kPhases>;
        case 2: return ep_dispatch_multi_kernel<true, false, kPhases>;
        default: return ep_dispatch_multi_kernel<true, true, kPhases>;
    }
}

}  // namespace

cudaError_t launch_group_dispatch_multi(const GroupDispatchParams* params, int n,
                                        GroupDispatchParams* dev_params, int phases,
                                        const LaunchCtx& ctx) {
    if (n < 1) return cudaSuccess;
    int want = 2;
    size_t smem = 0;
    for (int i = 0; i < n; ++i) {
        if (params[i].use_fp8 != params[0].use_fp8 || params[i].fused != params[0].fused ||
            params[i].H != params[0].H)
            return cudaErrorInvalidValue;
        const int blocks = 1 + (params[i].T > 0 ? params[i].T : 1);
        if (blocks > want) want = blocks;
        const size_t sm = dispatch_smem(params[i], phases == 3);
        if (sm > smem) smem = sm;
    }
    const int threads = block_threads(params[0].H, 256);
    auto k = phases == 3 ? pick_dispatch_multi<3>(params[0].use_fp8 != 0, params[0].fused != 0)
                         : pick_dispatch_multi<1>(params[0].use_fp8 != 0, params[0].fused != 0);
    const long long cap = resident_blocks(k, threads, smem, ctx) / n;
    if (cap < 2) return cudaErrorInvalidConfiguration;
    const int per_rank = (int)(want < cap ? want : cap);
    cudaError_t e = cudaMemcpyAsync(dev_params, params, sizeof(GroupDispatchParams) * n,
                                    cudaMemcpyHostToDevice, ctx.stream);
    if (e != cudaSuccess) return e;
    // (the copy reads pageable host memory: it has been staged when the call returns)
    return launch_cooperative("ep_dispatch_multi", k, per_rank * n, threads, smem, ctx,
                              (const GroupDispatchParams*)dev_params, per_rank);
}

cudaError_t launch_group_combine_multi(const GroupCombineParams* params, int n,
                                       GroupCombineParams* dev_params, const LaunchCtx& ctx) {
    if (n < 1) return cudaSuccess;
    int want = 64;
    size_t smem = 0;
    for (int i = 0; i < n; ++i) {
        if (params[i].H != params[0].H) return cudaErrorInvalidValue;
        if (params[i].T > want) want = params[i].T;
        const size_t sm = (size_t)(2 * params[i].E + 1) * sizeof(int);
        if (sm > smem) smem = sm;
    }
    const int threads = block_threads(params[0].H, 256);
    const long long cap = resident_blocks(ep_combine_multi_kernel, threads, smem, ctx) / n;
    if (cap < 1) return cudaErrorInvalidConfiguration;
    const int per_rank = (int)(want < cap ? want : cap);
    cudaError_t e = cudaMemcpyAsync(dev_params, params, sizeof(GroupCombineParams) * n,
                                    cudaMemcpyHostToDevice, ctx.stream);
    if (e != cudaSuccess) return e;
    return launch_cooperative("ep_combine_multi", ep_combine_multi_kernel, per_rank * n, threads,
                              smem, ctx, (const GroupCombineParams*)dev_params, per_rank);
}

}  // namespace mcep

#ifdef MCEP_PHASE_TRACE
// Diagnostic builds only: copies the trace of the calling thread's device out
// ([body 4][block 1024][slot 8] u64) after waiting for the device to go idle.
extern "C" int mcep_debug_read_phase_trace(unsigned long long* out, size_t bytes) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (bytes > sizeof(mcep::kernels::g_phase_trace)) bytes = sizeof(mcep::kernels::g_phase_trace);
    return cudaMemcpyFromSymbol(out, mcep::kernels::g_phase_trace, bytes) == cudaSuccess ? 0 : -1;
}
#endif
