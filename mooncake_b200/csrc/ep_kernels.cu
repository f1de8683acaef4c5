// Hand-written sm_100a kernels of the EP hot path: routing layout, dispatch
// (send / wait / pack) and combine (send / wait / invert / reduce).
//
// What they replace in the reference (paths inside the Mooncake tree):
//   mooncake-ep/src/mooncake_ep_kernel.cu:138-470  `dispatch`
//   mooncake-ep/src/mooncake_ep_kernel.cu:550-754  `combine`
// Design differences, all deliberate:
//   * no cooperative launch and no grid-wide barrier: a phase ends with its
//     kernel, so no block of a kernel ever waits for another block of the same
//     kernel; the only waits are on flags written by peers (bounded in time);
//   * receive order is deterministic (source rank, then token index): slots
//     come from a layout kernel instead of atomics in arrival order;
//   * the token row is read once, quantised in registers and stored straight
//     into every destination's receive staging (no local send staging pass);
//   * work is split by (token, part-of-row) and by rows, not by expert, so the
//     grid fills 148 SMs for 8 experts as well as for 256;
//   * flags are 64-bit (call sequence number << 32 | value) and never cleaned.
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

// Decide one flag, once, for every block of the kernel.
//
// A flag is either seen to arrive (its word carries this call's sequence number)
// or given up on (the rule of mooncake-ep/src/mooncake_ep_kernel.cu:417-429: after
// `timeout` the waiter clears active_ranks[src]; whoever sees the entry cleared
// stops waiting). Several blocks may need the same flag and they must agree, or
// the receive layout would be torn; so the first block to reach a verdict
// publishes it with a compare-and-swap into a local word, and every block -
// including that one - takes the verdict from that word:
//   resolved = seq << 32 | flag value     arrived
//   resolved = seq << 32 | 0              given up
// No block waits for another block: each keeps polling the peer's flag itself
// until some verdict exists. Returns the flag's low word, or 0.
__device__ __forceinline__ uint32_t resolve_flag(const WaitSpec& w, int i, int src,
                                              bool primary = true) {
    unsigned long long* res = reinterpret_cast<unsigned long long*>(w.resolved + i);
    uint64_t start = 0;
    if (!primary) {
        // Many blocks want the same verdict. One of them (the "primary" for this
        // flag) goes for the flag at once; the others look at the verdict word
        // alone for a short while, which keeps hundreds of blocks from hammering
        // one address with compare-and-swaps, and then fall back to doing the
        // work themselves - they never depend on the primary making progress.
        start = globaltimer_ns();
        while (globaltimer_ns() - start < 4000) {
            const uint64_t r = ld_acquire_gpu(w.resolved + i);
            if ((uint32_t)(r >> 32) == w.seq) {
                const uint32_t v = (uint32_t)r;
                if (v) (void)ld_acquire_sys(w.flags + i);
                return v;
            }
        }
    }
    while (true) {
        // both words are requested together: one round trip in the common case
        const uint64_t r = ld_acquire_gpu(w.resolved + i);
        const uint64_t f = ld_acquire_sys(w.flags + i);
        if ((uint32_t)(r >> 32) == w.seq) {
            // decided already (possibly by another block). If it is an arrival,
            // the flag load above was our own acquire of the sender's release -
            // unless it raced ahead of the flag, then take it again.
            const uint32_t v = (uint32_t)r;
            if (v && (uint32_t)(f >> 32) != w.seq) (void)ld_acquire_sys(w.flags + i);
            return v;
        }
        unsigned long long mine;
        if ((uint32_t)(f >> 32) == w.seq) {
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
            mine = (unsigned long long)w.seq << 32;               // given up
        }
        // first verdict wins; the value the swap returns is the winner's
        const unsigned long long old = atomicCAS(res, (unsigned long long)r, mine);
        const unsigned long long verdict = (old == (unsigned long long)r) ? mine : old;
        if ((uint32_t)(verdict >> 32) != w.seq) continue;  // lost to a stale word: look again
        const uint32_t v = (uint32_t)verdict;
        if (v && (uint32_t)(f >> 32) != w.seq) (void)ld_acquire_sys(w.flags + i);
        return v;
    }
}

// =============================================================================
// phase trace (diagnostic builds only: -DMCEP_PHASE_TRACE)
// =============================================================================
// Thread 0 of every block stamps the SM cycle counter at the phase boundaries
// of the four bodies below (slot 0 also takes the global timer, so blocks can
// be lined up against each other). Compiled out of the normal library.
#ifdef MCEP_PHASE_TRACE
constexpr int kTraceBodies = 4, kTraceBlocks = 1024, kTraceSlots = 8;
__device__ unsigned long long g_phase_trace[kTraceBodies][kTraceBlocks][kTraceSlots];
#define MCEP_TRACE(body, slot)                                                     \
    do {                                                                           \
        if (threadIdx.x == 0 && blockIdx.x < kTraceBlocks) {                       \
            g_phase_trace[body][blockIdx.x][slot] = (unsigned long long)clock64(); \
            if ((slot) == 0) g_phase_trace[body][blockIdx.x][kTraceSlots - 1] = globaltimer_ns(); \
        }                                                                          \
    } while (0)
#define MCEP_TRACE_SYNC() __syncthreads()
#else
#define MCEP_TRACE(body, slot) \
    do {                       \
    } while (0)
#define MCEP_TRACE_SYNC() \
    do {                  \
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
            if (p.done) p.done[e] = 0;
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

// =============================================================================
// dispatch: send
// =============================================================================
// One block per token (blocks stride over the tokens), one warp per 512-channel
// tile of the row. The block reads the bf16 row once (32 bytes per lane),
// quantises it in registers when FP8 is on, and stores it to every selected
// expert's slot: in the staged mode a message
//   [32 B header: token index | payload | 16 B of scales per 512 channels]
// in the owner rank's receive staging (peer memory over NVLink, or local), in
// the direct mode (single rank) the packed outputs themselves.
//
// kFused: the slots are counted here instead of read from the layout kernel -
// every block histograms the whole (small) index matrix in shared memory and
// counts, for its own token, the earlier tokens that chose the same experts.
// The host uses it when one block per token fits the machine in one wave.
//
// Completion: messages are not fenced one by one. A block counts what it sent
// per expert in shared memory; when its tokens are done it issues ONE
// system-scope fence, then adds its counts to the per-expert totals. Whoever
// completes an expert's total publishes the (source, expert) flag.
__device__ __forceinline__ int topk_entry(const int64_t* topk_idx, int t, int K, int k, int E) {
    // expert of entry (t, k); -1 when masked, out of range, or a repeat of an
    // earlier entry of the same token
    const int e = (int)__ldg(topk_idx + (size_t)t * K + k);
    if (e < 0 || e >= E) return -1;
    for (int kk = 0; kk < k; ++kk)
        if ((int)__ldg(topk_idx + (size_t)t * K + kk) == e) return -1;
    return e;
}

template <bool kFP8, bool kDirect, bool kFused>
__device__ __forceinline__ void dispatch_send_body(const DispatchSendParams& p, int* smem_i32) {
    __shared__ char* s_dst[kMaxTopk];
    __shared__ int s_exp[kMaxTopk];
    __shared__ int s_slot[kMaxTopk];
    __shared__ int s_before[kMaxTopk];
    __shared__ int s_raw[kMaxTopk];
    __shared__ int s_active[kMaxRanks];
    __shared__ char* s_peer[kMaxRanks];

    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    const int L = p.E / p.R;
    const int RM = p.R * p.M;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    const int S = p.H / 128;
    const char* xb = reinterpret_cast<const char*>(p.x);
    int* hist = smem_i32;                              // [E] whole-batch counts (fused)
    int* kmap = smem_i32 + p.E;                        // [E] expert -> k of this block's token (fused)
    int* cta_cnt = smem_i32 + (kFused ? 2 * p.E : 0);  // [E] sent by this block (staged)

    pdl_wait();
    pdl_launch_dependents();
    MCEP_TRACE(0, 0);
    // everything the block needs from memory is requested before the first
    // barrier, so the routing work costs one memory round trip, not several
    if (kFused)
        for (int e = tid; e < p.E; e += nthr) hist[e] = 0, kmap[e] = -1;
    if (!kDirect) {
        for (int e = tid; e < p.E; e += nthr) cta_cnt[e] = 0;
        for (int r = tid; r < p.R; r += nthr) {  // a block may have as few as 32 threads
            s_active[r] = ld_volatile_s32(p.active_ranks + r);
            s_peer[r] = reinterpret_cast<char*>(p.peer_base[r]);
        }
    }
    // The tables above are read by other threads further down. The token loop
    // has barriers of its own before any such read (and its first loads should
    // not wait for this prologue), but a block without tokens skips the loop.
    if ((int)blockIdx.x >= p.T) __syncthreads();

    for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
        const char* xrow = xb + (size_t)t * p.H * 2;
        V32 first = {};
        if (warp < ntiles && warp * 32 + lane < nchunks)
            first = ld32_readonly(xrow + (size_t)(warp * 32 + lane) * 32);
        const bool scan_now = kFused && t == (int)blockIdx.x;
        // the scan below lets a warp take whole tokens: lane -> (token, k)
        const int tpw = 32 / p.K;            // tokens per warp pass (K <= 16)
        const int sk = lane % p.K, st = lane / p.K;
        const bool lane_used = st < tpw;
        // the first kScanAhead passes of the scan are requested here, together
        // with the row, so the scan does not pay a memory round trip per pass
        constexpr int kScanAhead = 4;
        int e_ahead[kScanAhead];
#pragma unroll
        for (int u = 0; u < kScanAhead; ++u) {
            const int t2 = (warp + u * nwarps) * tpw + st;
            e_ahead[u] = -1;
            if (scan_now && lane_used && t2 < p.T)
                e_ahead[u] = (int)__ldg(p.topk_idx + (size_t)t2 * p.K + sk);
        }
        int my_slot = -1;
        if (tid < kMaxTopk) {
            int e = tid < p.K ? (int)__ldg(p.topk_idx + (size_t)t * p.K + tid) : -1;
            if (!kFused && tid < p.K) my_slot = __ldg(p.slot + (size_t)t * p.K + tid);
            s_raw[tid] = (e >= 0 && e < p.E) ? e : -1;
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
            // One pass over the index matrix with every warp: whole-batch
            // histogram, and for this block's token the number of earlier tokens
            // per chosen expert. A repeated expert inside a token is counted once
            // (lanes holding the same (token, expert) elect the lowest lane).
            auto count_pass = [&](int base, int e) {
                const int t2 = base + st;
                const bool valid = lane_used && t2 < p.T;
                if (!valid || e >= p.E) e = -1;
                const unsigned key = e >= 0 ? (((unsigned)st << 16) | (unsigned)e) : (0x80000000u | lane);
                const unsigned grp = __match_any_sync(kFull, key);
                if (e >= 0 && (int)(__ffs(grp) - 1) == lane) {
                    atomicAdd(&hist[e], 1);
                    if (t2 < t) {
                        const int kk = kmap[e];
                        if (kk >= 0) atomicAdd(&s_before[kk], 1);
                    }
                }
            };
#pragma unroll
            for (int u = 0; u < kScanAhead; ++u) {
                const int base = (warp + u * nwarps) * tpw;
                if (base < p.T) count_pass(base, e_ahead[u]);
            }
            for (int base = (warp + kScanAhead * nwarps) * tpw; base < p.T; base += nwarps * tpw) {
                const int t2 = base + st;
                count_pass(base, (lane_used && t2 < p.T) ? (int)__ldg(p.topk_idx + (size_t)t2 * p.K + sk)
                                                         : -1);
            }
            __syncthreads();
        }
        if (tid < kMaxTopk) {
            char* dst = nullptr;
            int s = -1;
            const int e = s_exp[tid];
            if (e >= 0) {
                s = kFused ? s_before[tid] : my_slot;
                if (s >= p.M) {
                    atomicOr(p.status, kStatusSlotRange);
                } else if (s >= 0) {
                    if (kDirect) {
                        dst = reinterpret_cast<char*>(p.recv_x) +
                              ((size_t)e * RM + s) * (size_t)p.H * (kFP8 ? 1 : 2);
                    } else {
                        const int dr = e / L;
                        if (s_active[dr])
                            dst = s_peer[dr] + p.stage_off +
                                  ((size_t)((e - dr * L) * p.R + p.rank) * p.M + s) * p.msg_stride;
                    }
                }
            }
            s_dst[tid] = dst;
            s_slot[tid] = s;
        }
        __syncthreads();
        if (t == (int)blockIdx.x) MCEP_TRACE(0, 1);  // routing of the first token is known

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
                if (kDirect) {
#pragma unroll 4
                    for (int k = 0; k < p.K; ++k) {
                        char* d = s_dst[k];
                        if (d == nullptr || !act) continue;
                        st16(d + (size_t)c * 16, q);
                        if ((lane & 7) == 0)
                            p.recv_scales[((size_t)s_exp[k] * S + (c >> 3)) * RM + s_slot[k]] = sinv;
                    }
                } else {
                    float4 sc;
                    sc.x = __shfl_sync(kFull, sinv, 0);
                    sc.y = __shfl_sync(kFull, sinv, 8);
                    sc.z = __shfl_sync(kFull, sinv, 16);
                    sc.w = __shfl_sync(kFull, sinv, 24);
#pragma unroll 4
                    for (int k = 0; k < p.K; ++k) {
                        char* d = s_dst[k];
                        if (d == nullptr) continue;
                        if (act) st16(d + kHeaderBytes + (size_t)c * 16, q);
                        if (lane == 0)
                            st16(d + kHeaderBytes + p.H + (size_t)tile * 16,
                                 *reinterpret_cast<uint4*>(&sc));
                    }
                }
            } else {
#pragma unroll 4
                for (int k = 0; k < p.K; ++k) {
                    char* d = s_dst[k];
                    if (d == nullptr || !act) continue;
                    st32(d + (kDirect ? 0 : kHeaderBytes) + (size_t)c * 32, cur);
                }
            }
        }
        if (tid < p.K && s_dst[tid] != nullptr) {
            if (kDirect) {
                p.recv_src_info[(size_t)s_exp[tid] * RM + s_slot[tid]] = t;
            } else {
                st16(s_dst[tid], make_uint4((uint32_t)t, 0u, 0u, 0u));
                atomicAdd(&cta_cnt[s_exp[tid]], 1);
            }
        }
        __syncthreads();
    }

    MCEP_TRACE(0, 2);  // all payload stores are issued
    // per-expert duties, spread over the grid: the receive layout of a single
    // rank, or the flag of an expert this rank sends nothing to
    for (int e = blockIdx.x * nthr + tid; e < p.E; e += gridDim.x * nthr) {
        const int c = kFused ? hist[e] : __ldg(p.count + e);
        if (kDirect) {
            if (kFused) {
                p.recv_count[e] = c;
                p.layout_range[e] = c;  // begin 0 | count
            }
        } else if (c == 0) {
            const int dr = e / L;
            if (s_active[dr]) {
                uint64_t* f = reinterpret_cast<uint64_t*>(s_peer[dr] + p.flag_off) +
                              ((e - dr * L) * p.R + p.rank);
                st_relaxed_sys(f, ((uint64_t)p.seq << 32) | 1u);
            }
        }
    }
    if (!kDirect) {
        // ONE system-scope fence for everything this block stored (it costs
        // microseconds even when idle, so it is not paid per message), then the
        // bookkeeping. Whoever completes an expert's total has, through the
        // counter, observed every contributor's fence: all of that expert's
        // messages are performed system-wide, and the flag may follow with only
        // a device-scope fence in between.
        MCEP_TRACE(0, 3);
        if (tid == 0) __threadfence_system();
        MCEP_TRACE(0, 4);  // the fence has returned
        __syncthreads();
        for (int e = tid; e < p.E; e += nthr) {
            const int c = cta_cnt[e];
            if (c == 0) continue;
            const int total = kFused ? hist[e] : __ldg(p.count + e);
            const int old = atomicAdd(p.done + e, c);
            if (old + c == total) {
                p.done[e] = 0;
                __threadfence();
                const int dr = e / L;
                uint64_t* f = reinterpret_cast<uint64_t*>(s_peer[dr] + p.flag_off) +
                              ((e - dr * L) * p.R + p.rank);
                st_relaxed_sys(f, ((uint64_t)p.seq << 32) | (uint32_t)(total + 1));
            }
        }
    }
    MCEP_TRACE(0, 5);
}

// =============================================================================
// dispatch: receive - wait for the (source, expert) flags, fix the layout, pack
// =============================================================================
// Every block first learns all L*R counts - one flag per thread, so the wait
// costs one flag latency, and the verdict words make all blocks agree - and
// turns them into the receive layout in shared memory: begin offsets per
// (expert, source) and a global row prefix. Block 0 writes `layout_range` and
// `recv_count`. Then rows are spread evenly over all warps of the grid (one
// warp per row, loads batched ahead of stores), whatever the routing skew.
constexpr int kRowWarps = 8;

template <bool kFP8>
__device__ __forceinline__ void dispatch_recv_body(const DispatchRecvParams& p, int* smem_i32) {
    int* pre = smem_i32;                  // [L*R + 1] rows before each (expert, source)
    int* beg = smem_i32 + p.L * p.R + 1;  // [L*R] first output row of each (expert, source)
    __shared__ int s_wt[32];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int n = p.L * p.R;
    const int RM = p.R * p.M;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    const int S = p.H / 128;
    pdl_wait();
    pdl_launch_dependents();
    MCEP_TRACE(1, 0);
    for (int i = tid; i < n; i += nthr) {
        const uint32_t v = resolve_flag(p.w, i, i % p.R, (i % gridDim.x) == blockIdx.x);
        pre[i] = v ? (int)v - 1 : 0;
    }
    __syncthreads();
    MCEP_TRACE(1, 1);  // every flag has a verdict
    for (int le = tid; le < p.L; le += nthr) {
        int run = 0;
        for (int src = 0; src < p.R; ++src) {
            const int c = pre[le * p.R + src];
            beg[le * p.R + src] = run;
            if (blockIdx.x == 0)
                p.layout_range[le * p.R + src] = c ? (((int64_t)run << 32) | (int64_t)c) : 0;
            run += c;
        }
        if (blockIdx.x == 0) p.recv_count[le] = run;
    }
    __syncthreads();
    block_exclusive_scan(pre, n, s_wt);
    MCEP_TRACE(1, 2);  // layout done
    const int total = pre[n];
    const int nwarps = nthr >> 5;
    // rows are dealt to the blocks one at a time (warp w of block b takes row
    // w * grid + b, ...): a batch with fewer rows than the grid has warps still
    // spreads over every SM
    for (int g = warp * gridDim.x + blockIdx.x; g < total; g += gridDim.x * nwarps) {
        const int i = find_segment(pre, n, g);
        const int le = i / p.R;
        const int j = g - pre[i];
        const int row = beg[i] + j;
        if (j >= p.M || row >= RM) {
            if (lane == 0) atomicOr(p.w.status, kStatusSlotRange);
            continue;
        }
        const char* msg = p.stage + ((size_t)i * p.M + j) * p.msg_stride;
        const size_t out_row = (size_t)le * RM + row;
        const int tok = lane == 0 ? ld_s32_coherent(msg) : 0;
        if (kFP8) {
            constexpr int kB = 8;  // 8 x 16 B per lane in flight
            char* out = reinterpret_cast<char*>(p.recv_x) + out_row * p.H;
            float sc0 = 0.f, sc1 = 0.f;
            if (lane < S) sc0 = ld_f32_coherent(msg + kHeaderBytes + p.H + (size_t)lane * 4);
            if (lane + 32 < S) sc1 = ld_f32_coherent(msg + kHeaderBytes + p.H + (size_t)(lane + 32) * 4);
            for (int t0 = 0; t0 < ntiles; t0 += kB) {
                uint4 v[kB];
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks)
                        v[b] = ld16_coherent(msg + kHeaderBytes + (size_t)c * 16);
                }
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks) st16(out + (size_t)c * 16, v[b]);
                }
            }
            if (lane < S) p.recv_scales[((size_t)le * S + lane) * RM + row] = sc0;
            if (lane + 32 < S) p.recv_scales[((size_t)le * S + lane + 32) * RM + row] = sc1;
            for (int gi = lane + 64; gi < S; gi += 32)  // hidden > 8192
                p.recv_scales[((size_t)le * S + gi) * RM + row] =
                    ld_f32_coherent(msg + kHeaderBytes + p.H + (size_t)gi * 4);
        } else {
            constexpr int kB = 4;  // 4 x 32 B per lane in flight
            char* out = reinterpret_cast<char*>(p.recv_x) + out_row * p.H * 2;
            for (int t0 = 0; t0 < ntiles; t0 += kB) {
                V32 v[kB];
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks)
                        v[b] = ld32_coherent(msg + kHeaderBytes + (size_t)c * 32);
                }
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks) st32(out + (size_t)c * 32, v[b]);
                }
            }
        }
        if (lane == 0) p.recv_src_info[out_row] = tok;
    }
    MCEP_TRACE_SYNC();
    MCEP_TRACE(1, 3);
}

// =============================================================================
// combine: send expert outputs back to the token owners
// =============================================================================
// One warp per packed row (warps stride over the rows), loads batched ahead of
// the stores. Row r of local expert le that came from rank d's token t goes to
// d's combine staging slot [global expert][t] (the slot rule of
// mooncake-ep/src/mooncake_ep_kernel.cu:633-637). Completion is counted per
// (expert, destination) segment the same way dispatch counts per expert: one
// system fence per block, then the block's shared-memory counts are added to
// the global ones and whoever completes a segment publishes that expert's flag
// at d.
__device__ __forceinline__ void combine_send_body(const CombineSendParams& p, int* smem_i32) {
    int* pre = smem_i32;                      // [L*R + 1]
    int* cta_cnt = smem_i32 + p.L * p.R + 1;  // [L*R]
    __shared__ int s_wt[32];
    __shared__ int s_active[kMaxRanks];
    __shared__ char* s_peer[kMaxRanks];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int n = p.L * p.R;
    const int RM = p.R * p.M;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    pdl_wait();
    pdl_launch_dependents();
    MCEP_TRACE(2, 0);
    for (int i = tid; i < n; i += nthr) {
        pre[i] = (int)(__ldg(p.layout_range + i) & 0xffffffffll);
        cta_cnt[i] = 0;
    }
    for (int r = tid; r < p.R; r += nthr) {
        s_active[r] = ld_volatile_s32(p.active_ranks + r);
        s_peer[r] = reinterpret_cast<char*>(p.peer_base[r]);
    }
    __syncthreads();
    // empty segments: flag right away
    for (int i = blockIdx.x * nthr + tid; i < n; i += gridDim.x * nthr) {
        if (pre[i] == 0) {
            const int d = i % p.R, le = i / p.R;
            if (s_active[d]) {
                uint64_t* f = reinterpret_cast<uint64_t*>(s_peer[d] + p.flag_off) + (p.rank * p.L + le);
                st_relaxed_sys(f, ((uint64_t)p.seq << 32) | 1u);
            }
        }
    }
    __syncthreads();
    block_exclusive_scan(pre, n, s_wt);
    MCEP_TRACE(2, 1);  // layout read and scanned
    const int total = pre[n];
    const char* xb = reinterpret_cast<const char*>(p.x);
    constexpr int kB = 8;  // 8 x 32 B per lane in flight: a 7168-wide row takes two round trips
    const int nwarps = nthr >> 5;
    // rows dealt to the blocks one at a time, as in the dispatch receive phase
    for (int g = warp * gridDim.x + blockIdx.x; g < total; g += gridDim.x * nwarps) {
        const int i = find_segment(pre, n, g);
        const int le = i / p.R, d = i - le * p.R;
        const int j = g - pre[i];
        const int row = (int)(__ldg(p.layout_range + i) >> 32) + j;
        const bool live = s_active[d] != 0;
        const bool row_ok = row < RM;
        // the source row does not depend on the token index: request it together
        // with the index so the two loads overlap
        int t = -1;
        if (row_ok) t = __ldg(p.src_info + (size_t)le * RM + row);
        const char* src = xb + ((size_t)le * RM + (row_ok ? row : 0)) * p.H * 2;
        V32 v[kB];
#pragma unroll
        for (int b = 0; b < kB; ++b) {
            const int c = b * 32 + lane;
            if (live && row_ok && b < ntiles && c < nchunks) v[b] = ld32_readonly(src + (size_t)c * 32);
        }
        if (t < 0 || t >= p.M) {
            if (lane == 0) atomicOr(p.status, kStatusBadSource);
        } else if (live) {
            char* dst = s_peer[d] + p.stage_off + ((size_t)(p.rank * p.L + le) * p.M + t) * p.H * 2;
#pragma unroll
            for (int b = 0; b < kB; ++b) {
                const int c = b * 32 + lane;
                if (b < ntiles && c < nchunks) st32(dst + (size_t)c * 32, v[b]);
            }
            for (int t0 = kB; t0 < ntiles; t0 += kB) {
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks) v[b] = ld32_readonly(src + (size_t)c * 32);
                }
#pragma unroll
                for (int b = 0; b < kB; ++b) {
                    const int c = (t0 + b) * 32 + lane;
                    if (t0 + b < ntiles && c < nchunks) st32(dst + (size_t)c * 32, v[b]);
                }
            }
        }
        if (lane == 0) atomicAdd(&cta_cnt[i], 1);
    }
    __syncthreads();
    MCEP_TRACE(2, 2);  // all rows are issued
    if (tid == 0) __threadfence_system();
    MCEP_TRACE(2, 3);  // the fence has returned
    __syncthreads();
    for (int i = tid; i < n; i += nthr) {
        const int c = cta_cnt[i];
        if (c == 0) continue;
        const int cnt = (int)(__ldg(p.layout_range + i) & 0xffffffffll);
        const int old = atomicAdd(p.done + i, c);
        if (old + c == cnt) {
            p.done[i] = 0;
            const int d = i % p.R, le = i / p.R;
            if (s_active[d]) {
                __threadfence();  // see the dispatch send kernel: one system fence per block
                uint64_t* f = reinterpret_cast<uint64_t*>(s_peer[d] + p.flag_off) + (p.rank * p.L + le);
                st_relaxed_sys(f, ((uint64_t)p.seq << 32) | 1u);
            }
        }
    }
    MCEP_TRACE(2, 4);
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
// combine: weighted top-k reduction
// =============================================================================
// One block per token, one warp per 512-channel tile; each lane owns 16
// channels: up to K 32-byte loads in flight, fp32 FMA accumulation in k order,
// one bf16 rounding, one 32-byte store (mooncake_ep_kernel.cu:715-752).
// kDepth rows are requested before the first of them is used: 8 when there is
// one block per SM anyway (small batches), 4 when several blocks share an SM.
template <bool kDirect, int kDepth>
__device__ __forceinline__ void combine_reduce_body(const CombineReduceParams& p) {
    __shared__ const char* s_ptr[kMaxTopk];
    __shared__ float s_w[kMaxTopk];
    __shared__ int s_row[kMaxTopk];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int lane = tid & 31, warp = tid >> 5, nwarps = nthr >> 5;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    pdl_wait();
    pdl_launch_dependents();
    MCEP_TRACE(3, 0);
    for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
        int e = -1, r = 0;
        float w = 0.f;
        if (tid < p.K) {
            e = (int)__ldg(p.topk_idx + (size_t)t * p.K + tid);
            w = __ldg(p.topk_weights + (size_t)t * p.K + tid);
            if (kDirect && !p.search) r = __ldcg(p.rowmap + (size_t)t * p.K + tid);
        }
        if (kDirect && p.search) {
            // Small batches: no separate inversion pass. Warp k looks the token
            // up in the handle itself - the segment of expert topk[t][k] that
            // came from this (only) rank - 32 entries of src_info at a time.
            for (int k = warp; k < p.K; k += nwarps) {
                const int ek = (int)__ldg(p.topk_idx + (size_t)t * p.K + k);
                int row = -1;
                if (ek >= 0 && ek < p.E) {
                    const long long lr = __ldg(p.layout_range + ek);
                    const int cnt = (int)(lr & 0xffffffffll), begin = (int)(lr >> 32);
                    for (int j0 = 0; j0 < cnt; j0 += 32) {
                        const int j = begin + j0 + lane;
                        const bool hit = j0 + lane < cnt && j < p.RM &&
                                         __ldg(p.src_info + (size_t)ek * p.RM + j) == t;
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
            if (kDirect && p.search && tid < p.K) r = s_row[tid];
            if (tid < p.K && e >= 0 && e < p.E) {
                const int owner = e / p.L;
                if (kDirect) {
                    if (ld_volatile_s32(p.active_ranks + owner) && r >= 0 && r < p.RM)
                        ptr = reinterpret_cast<const char*>(p.x) + ((size_t)e * p.RM + r) * p.H * 2;
                } else {
                    // wait for this expert's rows (mooncake_ep_kernel.cu:685-699), then the
                    // mask decides (an owner that timed out is skipped, :728-732)
                    const uint32_t v = resolve_flag(p.w, e, owner);
                    if (v && ld_volatile_s32(p.active_ranks + owner))
                        ptr = p.stage + ((size_t)e * p.M + t) * p.H * 2;
                }
            }
            s_ptr[tid] = ptr;
            s_w[tid] = w;
        }
        __syncthreads();
        if (t == (int)blockIdx.x) MCEP_TRACE(3, 1);  // the first token's rows are located / have arrived
        for (int tile = warp; tile < ntiles; tile += nwarps) {
            const int c = tile * 32 + lane;
            if (c >= nchunks) continue;
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = 0.f;
            // s_ptr has kMaxTopk entries, null from K on
            for (int k0 = 0; k0 < p.K; k0 += kDepth) {
                V32 v[kDepth];
#pragma unroll
                for (int b = 0; b < kDepth; ++b) {
                    const char* rp = s_ptr[k0 + b];
                    if (rp != nullptr)
                        v[b] = kDirect ? ld32_readonly(rp + (size_t)c * 32)
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
            st32(reinterpret_cast<char*>(p.combined_x) + ((size_t)t * p.H + (size_t)c * 16) * 2,
                 pack_bf16x16(acc));
        }
    }
    MCEP_TRACE_SYNC();
    MCEP_TRACE(3, 2);
}

// =============================================================================
// kernels
// =============================================================================
// The phases above as kernels of their own (hook mode, large batches), and the
// two phases of a call as ONE kernel for small batches in a group: every block
// first does its share of the send phase, then turns to the receive phase. The
// receive phase waits for flags that this rank's own blocks publish at the end
// of their send phase, so the grid is never larger than what is resident at
// once (the launchers see to that); a block that has started never depends on a
// block that has not.
template <bool kFP8, bool kDirect, bool kFused>
__global__ void __launch_bounds__(512) ep_dispatch_send_kernel(DispatchSendParams p) {
    extern __shared__ int smem_i32[];
    dispatch_send_body<kFP8, kDirect, kFused>(p, smem_i32);
}

template <bool kFP8>
__global__ void __launch_bounds__(kRowWarps * 32, 4) ep_dispatch_recv_kernel(DispatchRecvParams p) {
    extern __shared__ int smem_i32[];
    dispatch_recv_body<kFP8>(p, smem_i32);
}

template <bool kFP8>
__global__ void __launch_bounds__(512) ep_dispatch_kernel(DispatchSendParams sp, DispatchRecvParams rp) {
    extern __shared__ int smem_i32[];
    dispatch_send_body<kFP8, false, true>(sp, smem_i32);
    __syncthreads();
    dispatch_recv_body<kFP8>(rp, smem_i32);
}

__global__ void __launch_bounds__(kRowWarps * 32) ep_combine_send_kernel(CombineSendParams p) {
    extern __shared__ int smem_i32[];
    combine_send_body(p, smem_i32);
}

template <bool kDirect, int kDepth>
__global__ void __launch_bounds__(512) ep_combine_reduce_kernel(CombineReduceParams p) {
    static_assert(kMaxTopk % kDepth == 0, "the row batches must tile the top-k table");
    combine_reduce_body<kDirect, kDepth>(p);
}

__global__ void __launch_bounds__(512) ep_combine_kernel(CombineSendParams sp, CombineReduceParams rp) {
    extern __shared__ int smem_i32[];
    combine_send_body(sp, smem_i32);
    __syncthreads();
    combine_reduce_body<false, 8>(rp);
}

// threads per block: one warp per tile, at most 16 warps
inline int block_threads(int H) {
    int ntiles = (H + kTileChannels - 1) / kTileChannels;
    if (ntiles > 16) ntiles = 16;
    if (ntiles < 1) ntiles = 1;
    return ntiles * 32;
}
// a grid that fills the machine once (blocks stride over the work items):
// as many blocks as are resident at a time for this kernel, block size and
// shared memory
template <typename K>
inline int persistent_grid(long long items, K kernel, int threads, size_t smem, const LaunchCtx& ctx) {
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
    long long cap = (long long)ctx.num_sms * per_sm;
    long long g = items < cap ? items : cap;
    return (int)(g < 1 ? 1 : g);
}

}  // namespace kernels
using namespace kernels;

// =============================================================================
// launchers
// =============================================================================
cudaError_t launch_layout(const LayoutParams& p, const LaunchCtx& ctx) {
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

bool dispatch_send_can_fuse_layout(int T, int K, int H, int num_sms) {
    // one block per token in a single wave, and an index matrix small enough to
    // be scanned by every block
    (void)H;
    // one block per token, all resident at once even at two blocks per SM
    return (long long)T * K <= 4096 && T <= num_sms * 2;
}

cudaError_t launch_dispatch_send(const DispatchSendParams& p, const LaunchCtx& ctx) {
    const int threads = block_threads(p.H);
    const size_t smem = (size_t)((p.fused ? 2 * p.E : 0) + (p.direct ? 0 : p.E)) * sizeof(int);
    void (*k)(DispatchSendParams) = nullptr;
    const int sel = (p.use_fp8 ? 4 : 0) | (p.direct ? 2 : 0) | (p.fused ? 1 : 0);
    switch (sel) {
        case 0: k = ep_dispatch_send_kernel<false, false, false>; break;
        case 1: k = ep_dispatch_send_kernel<false, false, true>; break;
        case 2: k = ep_dispatch_send_kernel<false, true, false>; break;
        case 3: k = ep_dispatch_send_kernel<false, true, true>; break;
        case 4: k = ep_dispatch_send_kernel<true, false, false>; break;
        case 5: k = ep_dispatch_send_kernel<true, false, true>; break;
        case 6: k = ep_dispatch_send_kernel<true, true, false>; break;
        default: k = ep_dispatch_send_kernel<true, true, true>; break;
    }
    const int grid = p.fused ? (p.T > 0 ? p.T : 1) : persistent_grid(p.T, k, threads, smem, ctx);
    return launch(p.direct ? "ep_dispatch_send_direct" : "ep_dispatch_send", k, dim3(grid),
                  dim3(threads), smem, ctx, p);
}

cudaError_t launch_dispatch_recv(const DispatchRecvParams& p, const LaunchCtx& ctx) {
    const int threads = kRowWarps * 32;
    const size_t smem = (size_t)(2 * p.L * p.R + 1) * sizeof(int);
    auto k = p.use_fp8 ? ep_dispatch_recv_kernel<true> : ep_dispatch_recv_kernel<false>;
    // The row count is only known on the device. Under even routing a rank
    // receives about what it sends (`expected_rows`); the grid is sized for
    // twice that - blocks stride, so a skewed or larger load is still covered -
    // and never beyond one resident wave.
    long long rows = 2ll * p.expected_rows;
    const long long worst = (long long)p.L * p.R * p.M;
    if (rows > worst) rows = worst;
    const int grid = persistent_grid((rows + kRowWarps - 1) / kRowWarps, k, threads, smem, ctx);
    return launch("ep_dispatch_recv", k, dim3(grid), dim3(threads), smem, ctx, p);
}

cudaError_t launch_combine_send(const CombineSendParams& p, const LaunchCtx& ctx) {
    const int threads = kRowWarps * 32;
    const long long rows = (long long)p.L * p.R * p.M;
    const size_t smem = (size_t)(2 * p.L * p.R + 1) * sizeof(int);
    const int grid = persistent_grid((rows + kRowWarps - 1) / kRowWarps, ep_combine_send_kernel,
                                     threads, smem, ctx);
    return launch("ep_combine_send", ep_combine_send_kernel, dim3(grid), dim3(threads), smem, ctx, p);
}

bool call_can_be_one_kernel(int T, int K, int H, int num_sms) {
    // small batch, one block per token resident at two blocks per SM (dispatch) and
    // at one block per SM for the register-heavier combine
    (void)H;
    return (long long)T * K <= 4096 && T <= num_sms;
}

cudaError_t launch_dispatch_one_kernel(const DispatchSendParams& sp, const DispatchRecvParams& rp,
                                       const LaunchCtx& ctx) {
    const int threads = block_threads(sp.H);
    size_t smem = (size_t)3 * sp.E * sizeof(int);
    const size_t smem_recv = (size_t)(2 * rp.L * rp.R + 1) * sizeof(int);
    if (smem_recv > smem) smem = smem_recv;
    auto k = sp.use_fp8 ? ep_dispatch_kernel<true> : ep_dispatch_kernel<false>;
    const int grid = sp.T > 0 ? sp.T : 1;
    if (grid > persistent_grid(grid, k, threads, smem, ctx)) return cudaErrorInvalidConfiguration;
    return launch("ep_dispatch", k, dim3(grid), dim3(threads), smem, ctx, sp, rp);
}

cudaError_t launch_combine_one_kernel(const CombineSendParams& sp, const CombineReduceParams& rp,
                                      const LaunchCtx& ctx) {
    const int threads = block_threads(sp.H);
    const size_t smem = (size_t)(2 * sp.L * sp.R + 1) * sizeof(int);
    // enough blocks for one token each in the reduce phase; the send phase strides
    const int want = rp.T > 0 ? rp.T : 1;
    const int grid = persistent_grid(want, ep_combine_kernel, threads, smem, ctx);
    return launch("ep_combine", ep_combine_kernel, dim3(grid), dim3(threads), smem, ctx, sp, rp);
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

cudaError_t launch_combine_reduce(const CombineReduceParams& p, const LaunchCtx& ctx) {
    const int threads = block_threads(p.H);
    const bool deep = p.T <= ctx.num_sms;  // one block per SM at most: spend registers on loads in flight
    auto k = p.direct ? (deep ? ep_combine_reduce_kernel<true, 8> : ep_combine_reduce_kernel<true, 4>)
                      : (deep ? ep_combine_reduce_kernel<false, 8> : ep_combine_reduce_kernel<false, 4>);
    const int grid = persistent_grid(p.T, k, threads, 0, ctx);
    return launch(p.direct ? "ep_combine_reduce_direct" : "ep_combine_reduce", k, dim3(grid),
                  dim3(threads), 0, ctx, p);
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
