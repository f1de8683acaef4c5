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

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;
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

// Spin until the flag carries this call's sequence number. Leaves early when
// the source is, or becomes, inactive: the rule of
// mooncake-ep/src/mooncake_ep_kernel.cu:417-429 (timeout -> the waiter clears
// active_ranks[src]; anyone who sees it cleared stops waiting). Returns the
// flag's low word, or 0 when the wait was given up.
__device__ __forceinline__ uint32_t wait_flag(const uint64_t* flag, uint32_t seq,
                                              int32_t* active_ranks, int src,
                                              int64_t timeout_ns, int64_t hard_ns,
                                              int32_t* status) {
    uint64_t v = ld_acquire_sys(flag);
    if ((uint32_t)(v >> 32) == seq) return (uint32_t)v;
    const uint64_t start = globaltimer_ns();
    while (true) {
        v = ld_acquire_sys(flag);
        if ((uint32_t)(v >> 32) == seq) return (uint32_t)v;
        const int64_t waited = (int64_t)(globaltimer_ns() - start);
        if (timeout_ns >= 0 && waited > timeout_ns) st_volatile_s32(active_ranks + src, 0);
        if (waited > hard_ns) {
            st_volatile_s32(active_ranks + src, 0);
            atomicOr(status, kStatusHardTimeout);
        }
        if (!ld_volatile_s32(active_ranks + src)) return 0;
    }
}

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
    for (int i = tid; i < n; i += nthr) {
        const int e = (int)__ldg(p.topk_idx + i);
        if (e >= e0 && e < e1) {
            const int t = i / p.K;
            atomicOr(&mask[(e - e0) * words + (t >> 5)], 1u << (t & 31));
        }
    }
    __syncthreads();
    pdl_launch_dependents();
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
    for (int i = tid; i < n; i += nthr) {
        const int e = (int)__ldg(p.topk_idx + i);
        if (e >= e0 && e < e1) {
            const int t = i / p.K, k = i - t * p.K;
            bool dup = false;
            for (int kk = 0; kk < k; ++kk) dup |= ((int)__ldg(p.topk_idx + t * p.K + kk) == e);
            const int o = (e - e0) * words + (t >> 5);
            p.slot[i] = dup ? -1 : (int)(wpre[o] + __popc(mask[o] & ((1u << (t & 31)) - 1u)));
        } else if (e < 0 && blockIdx.x == 0) {
            p.slot[i] = -1;
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
// Warp item = (token, part of the row). The warp reads its part of the bf16 row
// once (32 bytes per lane and pass), quantises it in registers when FP8 is on,
// and stores it to every selected expert's slot: in the staged mode a message
//   [32 B header: token index | payload | 16 B of scales per 512 channels]
// in the owner rank's receive staging (peer memory over NVLink or local), in the
// direct mode (single rank) the packed outputs themselves. The warp that
// completes an expert's last message publishes the (source, expert) flag.
template <bool kFP8, bool kDirect>
__global__ void __launch_bounds__(kThreads) ep_dispatch_send_kernel(DispatchSendParams p) {
    __shared__ char* s_dst[kWarpsPerBlock][kMaxTopk];
    __shared__ int s_exp[kWarpsPerBlock][kMaxTopk];
    __shared__ int s_slot[kWarpsPerBlock][kMaxTopk];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gwarp = blockIdx.x * kWarpsPerBlock + warp;
    const int nwarps = gridDim.x * kWarpsPerBlock;
    const int L = p.E / p.R;
    const int RM = p.R * p.M;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    const int S = p.H / 128;
    const char* xb = reinterpret_cast<const char*>(p.x);

    pdl_wait();  // slot[] and count[] come from the layout kernel

    if (!kDirect) {
        // experts this rank sends nothing to still get their flag
        for (int e = blockIdx.x * kThreads + threadIdx.x; e < p.E; e += gridDim.x * kThreads) {
            if (__ldg(p.count + e) == 0) {
                const int dr = e / L;
                if (ld_volatile_s32(p.active_ranks + dr)) {
                    uint64_t* f = reinterpret_cast<uint64_t*>(
                                      reinterpret_cast<char*>(p.peer_base[dr]) + p.flag_off) +
                                  ((e - dr * L) * p.R + p.rank);
                    st_release_sys(f, ((uint64_t)p.seq << 32) | 1u);
                }
            }
        }
    }

    const int items = p.T * p.parts;
    for (int item = gwarp; item < items; item += nwarps) {
        const int t = item / p.parts, part = item - t * p.parts;
        char* my_dst = nullptr;
        int my_e = -1, my_s = -1;
        if (lane < p.K) {
            const int e = (int)__ldg(p.topk_idx + t * p.K + lane);
            const int s = __ldg(p.slot + t * p.K + lane);
            if (e >= 0 && s >= 0) {
                if (s >= p.M) {
                    atomicOr(p.status, kStatusSlotRange);
                } else if (kDirect) {
                    my_dst = reinterpret_cast<char*>(p.recv_x) +
                             ((size_t)e * RM + s) * (size_t)p.H * (kFP8 ? 1 : 2);
                    my_e = e, my_s = s;
                } else {
                    const int dr = e / L;
                    if (ld_volatile_s32(p.active_ranks + dr)) {
                        my_dst = reinterpret_cast<char*>(p.peer_base[dr]) + p.stage_off +
                                 ((size_t)((e - dr * L) * p.R + p.rank) * p.M + s) * p.msg_stride;
                        my_e = e, my_s = s;
                    }
                }
            }
        }
        if (lane < kMaxTopk) {
            s_dst[warp][lane] = my_dst;
            s_exp[warp][lane] = my_e;
            s_slot[warp][lane] = my_s;
        }
        __syncwarp();

        const int tile0 = part * p.tiles_per_part;
        const int tile1 = min(ntiles, tile0 + p.tiles_per_part);
        const char* xrow = xb + (size_t)t * p.H * 2;
        V32 cur = {};
        if (tile0 < tile1 && tile0 * 32 + lane < nchunks)
            cur = ld32_readonly(xrow + (size_t)(tile0 * 32 + lane) * 32);
        for (int tile = tile0; tile < tile1; ++tile) {
            const int c = tile * 32 + lane;
            const bool act = c < nchunks;
            V32 nxt = {};
            if (tile + 1 < tile1 && c + 32 < nchunks) nxt = ld32_readonly(xrow + (size_t)(c + 32) * 32);
            if (kFP8) {
                float sinv;
                const uint4 q = quantize16(cur, sinv);
                if (kDirect) {
#pragma unroll 4
                    for (int k = 0; k < p.K; ++k) {
                        char* d = s_dst[warp][k];
                        if (d == nullptr) continue;
                        if (act) {
                            st16(d + (size_t)c * 16, q);
                            if ((lane & 7) == 0)
                                p.recv_scales[((size_t)s_exp[warp][k] * S + (c >> 3)) * RM +
                                              s_slot[warp][k]] = sinv;
                        }
                    }
                } else {
                    float4 sc;
                    sc.x = __shfl_sync(kFull, sinv, 0);
                    sc.y = __shfl_sync(kFull, sinv, 8);
                    sc.z = __shfl_sync(kFull, sinv, 16);
                    sc.w = __shfl_sync(kFull, sinv, 24);
#pragma unroll 4
                    for (int k = 0; k < p.K; ++k) {
                        char* d = s_dst[warp][k];
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
                    char* d = s_dst[warp][k];
                    if (d == nullptr) continue;
                    if (act) st32(d + (kDirect ? 0 : kHeaderBytes) + (size_t)c * 32, cur);
                }
            }
            cur = nxt;
        }
        if (part == 0 && my_dst != nullptr) {
            if (kDirect)
                p.recv_src_info[(size_t)my_e * RM + my_s] = t;
            else
                st16(my_dst, make_uint4((uint32_t)t, 0u, 0u, 0u));
        }
        __syncwarp();
        if (!kDirect && my_dst != nullptr) {
            const int n = __ldg(p.count + my_e);
            const int old = atom_add_acq_rel_sys(p.done + my_e, 1);
            if (old + 1 == n * p.parts) {
                const int dr = my_e / L;
                uint64_t* f = reinterpret_cast<uint64_t*>(
                                  reinterpret_cast<char*>(p.peer_base[dr]) + p.flag_off) +
                              ((my_e - dr * L) * p.R + p.rank);
                st_release_sys(f, ((uint64_t)p.seq << 32) | (uint32_t)(n + 1));
            }
        }
        __syncwarp();
    }
    pdl_launch_dependents();
}

// =============================================================================
// dispatch: wait for the (source, expert) flags and fix the receive layout
// =============================================================================
// One block. Thread i waits for flag i = expert * R + source, then the block
// turns the counts into `layout_range`, `recv_count` and the row prefix the
// pack kernel partitions its work by.
__global__ void __launch_bounds__(1024) ep_dispatch_wait_kernel(DispatchWaitParams p) {
    extern __shared__ int smem_i32[];
    int* cnt = smem_i32;            // [L*R]
    int* tot = smem_i32 + p.L * p.R;  // [L + 1]
    __shared__ int s_wt[32];
    const int tid = threadIdx.x, nthr = blockDim.x;
    const int n = p.L * p.R;
    pdl_wait();
    for (int i = tid; i < n; i += nthr) {
        const int src = i % p.R;
        const uint32_t v = wait_flag(p.flags + i, p.seq, p.active_ranks, src, p.timeout_ns,
                                     p.hard_timeout_ns, p.status);
        cnt[i] = v ? (int)v - 1 : 0;
    }
    __syncthreads();
    pdl_launch_dependents();
    for (int le = tid; le < p.L; le += nthr) {
        int begin = 0;
        for (int src = 0; src < p.R; ++src) {
            const int c = cnt[le * p.R + src];
            p.layout_range[le * p.R + src] = c ? (((int64_t)begin << 32) | (int64_t)c) : 0;
            begin += c;
        }
        p.recv_count[le] = begin;
        tot[le] = begin;
    }
    __syncthreads();
    block_exclusive_scan(tot, p.L, s_wt);
    for (int le = tid; le < p.L; le += nthr) {
        int run = tot[le];
        for (int src = 0; src < p.R; ++src) {
            p.pack_prefix[le * p.R + src] = run;
            run += cnt[le * p.R + src];
        }
    }
    if (tid == 0) p.pack_prefix[n] = tot[p.L];
}

// =============================================================================
// dispatch: pack the staged messages into the caller's tensors
// =============================================================================
template <bool kFP8>
__global__ void __launch_bounds__(kThreads) ep_dispatch_pack_kernel(DispatchPackParams p) {
    extern __shared__ int smem_i32[];
    int* pre = smem_i32;  // [L*R + 1]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = p.L * p.R;
    const int RM = p.R * p.M;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    const int S = p.H / 128;
    pdl_wait();
    for (int i = threadIdx.x; i <= n; i += kThreads) pre[i] = __ldcg(p.pack_prefix + i);
    __syncthreads();
    pdl_launch_dependents();
    const int total = pre[n];
    const long long items = (long long)total * p.parts;
    for (long long item = (long long)blockIdx.x * kWarpsPerBlock + warp; item < items;
         item += (long long)gridDim.x * kWarpsPerBlock) {
        const int g = (int)(item / p.parts), part = (int)(item - (long long)g * p.parts);
        const int i = find_segment(pre, n, g);
        const int le = i / p.R;
        const int j = g - pre[i];
        const int row = (int)(__ldcg(p.layout_range + i) >> 32) + j;
        if (j >= p.M || row >= RM) {
            if (lane == 0) atomicOr(p.status, kStatusSlotRange);
            continue;
        }
        const char* msg = p.stage + ((size_t)i * p.M + j) * p.msg_stride;
        const size_t out_row = (size_t)le * RM + row;
        const int tile0 = part * p.tiles_per_part;
        const int tile1 = min(ntiles, tile0 + p.tiles_per_part);
        for (int tile = tile0; tile < tile1; ++tile) {
            const int c = tile * 32 + lane;
            if (kFP8) {
                if (c < nchunks)
                    st16(reinterpret_cast<char*>(p.recv_x) + out_row * p.H + (size_t)c * 16,
                         ld16_coherent(msg + kHeaderBytes + (size_t)c * 16));
                const int gi = tile * 4 + lane;
                if (lane < 4 && gi < S)
                    p.recv_scales[((size_t)le * S + gi) * RM + row] =
                        ld_f32_coherent(msg + kHeaderBytes + p.H + (size_t)gi * 4);
            } else {
                if (c < nchunks)
                    st32(reinterpret_cast<char*>(p.recv_x) + (out_row * p.H + (size_t)c * 16) * 2,
                         ld32_coherent(msg + kHeaderBytes + (size_t)c * 32));
            }
        }
        if (part == 0 && lane == 0) p.recv_src_info[out_row] = ld_s32_coherent(msg);
    }
}

// =============================================================================
// combine: send expert outputs back to the token owners
// =============================================================================
// Warp item = (packed row, part). Row r of local expert le that came from rank
// d's token t goes to d's combine staging slot [global expert][t]
// (the slot rule of mooncake-ep/src/mooncake_ep_kernel.cu:633-637). The warp that
// completes a (expert, destination) segment publishes that expert's flag at d.
__global__ void __launch_bounds__(kThreads) ep_combine_send_kernel(CombineSendParams p) {
    extern __shared__ int smem_i32[];
    int* pre = smem_i32;  // [L*R + 1]
    __shared__ int s_wt[32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = p.L * p.R;
    const int RM = p.R * p.M;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    pdl_wait();
    for (int i = threadIdx.x; i < n; i += kThreads)
        pre[i] = (int)(__ldg(p.layout_range + i) & 0xffffffffll);
    __syncthreads();
    // empty segments: flag right away
    for (int i = blockIdx.x * kThreads + threadIdx.x; i < n; i += gridDim.x * kThreads) {
        if (pre[i] == 0) {
            const int d = i % p.R, le = i / p.R;
            if (ld_volatile_s32(p.active_ranks + d)) {
                uint64_t* f = reinterpret_cast<uint64_t*>(
                                  reinterpret_cast<char*>(p.peer_base[d]) + p.flag_off) +
                              (p.rank * p.L + le);
                st_release_sys(f, ((uint64_t)p.seq << 32) | 1u);
            }
        }
    }
    __syncthreads();
    block_exclusive_scan(pre, n, s_wt);
    const int total = pre[n];
    const long long items = (long long)total * p.parts;
    const char* xb = reinterpret_cast<const char*>(p.x);
    for (long long item = (long long)blockIdx.x * kWarpsPerBlock + warp; item < items;
         item += (long long)gridDim.x * kWarpsPerBlock) {
        const int g = (int)(item / p.parts), part = (int)(item - (long long)g * p.parts);
        const int i = find_segment(pre, n, g);
        const int le = i / p.R, d = i - le * p.R;
        const int j = g - pre[i];
        const long long lr = __ldg(p.layout_range + i);
        const int cnt = (int)(lr & 0xffffffffll);
        const int row = (int)(lr >> 32) + j;
        const bool live = ld_volatile_s32(p.active_ranks + d) != 0;
        int t = -1;
        if (row < RM) t = __ldg(p.src_info + (size_t)le * RM + row);
        if (t < 0 || t >= p.M) {
            if (lane == 0) atomicOr(p.status, kStatusBadSource);
        } else if (live) {
            const char* src = xb + ((size_t)le * RM + row) * p.H * 2;
            char* dst = reinterpret_cast<char*>(p.peer_base[d]) + p.stage_off +
                        ((size_t)(p.rank * p.L + le) * p.M + t) * p.H * 2;
            const int tile0 = part * p.tiles_per_part;
            const int tile1 = min(ntiles, tile0 + p.tiles_per_part);
            V32 cur = {};
            if (tile0 < tile1 && tile0 * 32 + lane < nchunks)
                cur = ld32_readonly(src + (size_t)(tile0 * 32 + lane) * 32);
            for (int tile = tile0; tile < tile1; ++tile) {
                const int c = tile * 32 + lane;
                V32 nxt = {};
                if (tile + 1 < tile1 && c + 32 < nchunks)
                    nxt = ld32_readonly(src + (size_t)(c + 32) * 32);
                if (c < nchunks) st32(dst + (size_t)c * 32, cur);
                cur = nxt;
            }
        }
        __syncwarp();
        if (lane == 0) {
            const int old = atom_add_acq_rel_sys(p.done + i, 1);
            if (old + 1 == cnt * p.parts) {
                p.done[i] = 0;
                if (live) {
                    uint64_t* f = reinterpret_cast<uint64_t*>(
                                      reinterpret_cast<char*>(p.peer_base[d]) + p.flag_off) +
                                  (p.rank * p.L + le);
                    st_release_sys(f, ((uint64_t)p.seq << 32) | 1u);
                }
            }
        }
    }
    pdl_launch_dependents();
}

// One block; thread e waits for expert e's flag
// (mooncake-ep/src/mooncake_ep_kernel.cu:685-699).
__global__ void __launch_bounds__(1024) ep_combine_wait_kernel(CombineWaitParams p) {
    pdl_wait();
    for (int e = threadIdx.x; e < p.E; e += blockDim.x)
        (void)wait_flag(p.flags + e, p.seq, p.active_ranks, e / p.L, p.timeout_ns,
                        p.hard_timeout_ns, p.status);
    pdl_launch_dependents();
}

// Single rank: rowmap[t][k] = packed row of (token t, expert topk[t][k]) as the
// handle records it.
__global__ void __launch_bounds__(256) ep_combine_invert_kernel(CombineInvertParams p) {
    const int RM = p.R * p.M;
    const long long total = (long long)p.L * p.M;
    pdl_wait();
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
    pdl_launch_dependents();
}

// =============================================================================
// combine: weighted top-k reduction
// =============================================================================
// Warp item = (token, 512-channel tile); each lane owns 16 channels: up to K
// 32-byte loads in flight, fp32 FMA accumulation in k order, one bf16 rounding,
// one 32-byte store (the arithmetic of mooncake_ep_kernel.cu:715-752).
template <bool kDirect>
__global__ void __launch_bounds__(kThreads) ep_combine_reduce_kernel(CombineReduceParams p) {
    __shared__ const char* s_ptr[kWarpsPerBlock][kMaxTopk];
    __shared__ float s_w[kWarpsPerBlock][kMaxTopk];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nchunks = p.H / 16;
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    const long long items = (long long)p.T * ntiles;
    pdl_wait();
    for (long long item = (long long)blockIdx.x * kWarpsPerBlock + warp; item < items;
         item += (long long)gridDim.x * kWarpsPerBlock) {
        const int t = (int)(item / ntiles), tile = (int)(item - (long long)t * ntiles);
        const char* ptr = nullptr;
        float w = 0.f;
        if (lane < p.K) {
            const int e = (int)__ldg(p.topk_idx + (size_t)t * p.K + lane);
            w = __ldg(p.topk_weights + (size_t)t * p.K + lane);
            if (e >= 0 && e < p.E && ld_volatile_s32(p.active_ranks + e / p.L)) {
                if (kDirect) {
                    const int r = __ldcg(p.rowmap + (size_t)t * p.K + lane);
                    if (r >= 0 && r < p.RM)
                        ptr = reinterpret_cast<const char*>(p.x) + ((size_t)e * p.RM + r) * p.H * 2;
                } else {
                    ptr = p.stage + ((size_t)e * p.M + t) * p.H * 2;
                }
            }
        }
        if (lane < kMaxTopk) {
            s_ptr[warp][lane] = ptr;
            s_w[warp][lane] = w;
        }
        __syncwarp();
        const int c = tile * 32 + lane;
        if (c < nchunks) {
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll 4
            for (int k = 0; k < p.K; ++k) {
                const char* rp = s_ptr[warp][k];
                if (rp == nullptr) continue;
                const V32 v = kDirect ? ld32_readonly(rp + (size_t)c * 32)
                                      : ld32_coherent(rp + (size_t)c * 32);
                const float wk = s_w[warp][k];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    acc[2 * i] = fmaf(bf16lo(v.w[i]), wk, acc[2 * i]);
                    acc[2 * i + 1] = fmaf(bf16hi(v.w[i]), wk, acc[2 * i + 1]);
                }
            }
            st32(reinterpret_cast<char*>(p.combined_x) + ((size_t)t * p.H + (size_t)c * 16) * 2,
                 pack_bf16x16(acc));
        }
        __syncwarp();
    }
}

inline int grid_for_warp_items(long long items, const LaunchCtx& ctx, int blocks_per_sm) {
    long long blocks = (items + kWarpsPerBlock - 1) / kWarpsPerBlock;
    long long cap = (long long)ctx.num_sms * blocks_per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace kernels
using namespace kernels;

// =============================================================================
// launchers
// =============================================================================
cudaError_t launch_layout(const LayoutParams& p, const LaunchCtx& ctx) {
    const int words = (p.T + 31) / 32 > 0 ? (p.T + 31) / 32 : 1;
    // experts per block: spread over the SMs, bounded by shared memory
    int epc = (p.E + ctx.num_sms - 1) / ctx.num_sms;
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
    const int n = p.T * p.K;
    int threads = 128;
    while (threads < 1024 && threads * 4 < n) threads <<= 1;
    const int grid = (p.E + epc - 1) / epc;
    return launch("ep_routing_layout", ep_routing_layout_kernel, dim3(grid), dim3(threads), smem, ctx, p, epc, words);
}

cudaError_t launch_dispatch_send(const DispatchSendParams& p, const LaunchCtx& ctx) {
    const long long items = (long long)p.T * p.parts;
    int grid = grid_for_warp_items(items, ctx, 8);
    // enough threads to cover the zero-count flag loop in one pass when cheap
    const int min_grid = (p.E + kThreads - 1) / kThreads;
    if (!p.direct && grid < min_grid) grid = min_grid;
    auto k = p.use_fp8 ? (p.direct ? ep_dispatch_send_kernel<true, true>
                                   : ep_dispatch_send_kernel<true, false>)
                       : (p.direct ? ep_dispatch_send_kernel<false, true>
                                   : ep_dispatch_send_kernel<false, false>);
    return launch(p.direct ? "ep_dispatch_send_direct" : "ep_dispatch_send", k, dim3(grid), dim3(kThreads), 0, ctx, p);
}

cudaError_t launch_dispatch_wait(const DispatchWaitParams& p, const LaunchCtx& ctx) {
    const int n = p.L * p.R;
    int threads = 32;
    while (threads < 1024 && threads < n) threads <<= 1;
    const size_t smem = (size_t)(n + p.L + 1) * sizeof(int);
    return launch("ep_dispatch_wait", ep_dispatch_wait_kernel, dim3(1), dim3(threads), smem, ctx, p);
}

cudaError_t launch_dispatch_pack(const DispatchPackParams& p, const LaunchCtx& ctx) {
    // the row count is only known on the device: size for the worst case the
    // machine can hold at once and let the blocks stride
    const long long worst = (long long)p.L * p.R * p.M * p.parts;
    const int grid = grid_for_warp_items(worst, ctx, 8);
    const size_t smem = (size_t)(p.L * p.R + 1) * sizeof(int);
    auto k = p.use_fp8 ? ep_dispatch_pack_kernel<true> : ep_dispatch_pack_kernel<false>;
    return launch("ep_dispatch_pack", k, dim3(grid), dim3(kThreads), smem, ctx, p);
}

cudaError_t launch_combine_send(const CombineSendParams& p, const LaunchCtx& ctx) {
    const long long worst = (long long)p.L * p.R * p.M * p.parts;
    int grid = grid_for_warp_items(worst, ctx, 8);
    const size_t smem = (size_t)(p.L * p.R + 1) * sizeof(int);
    return launch("ep_combine_send", ep_combine_send_kernel, dim3(grid), dim3(kThreads), smem, ctx, p);
}

cudaError_t launch_combine_wait(const CombineWaitParams& p, const LaunchCtx& ctx) {
    int threads = 32;
    while (threads < 1024 && threads < p.E) threads <<= 1;
    return launch("ep_combine_wait", ep_combine_wait_kernel, dim3(1), dim3(threads), 0, ctx, p);
}

cudaError_t launch_combine_invert(const CombineInvertParams& p, const LaunchCtx& ctx) {
    const long long total = (long long)p.L * p.M;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)ctx.num_sms * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return launch("ep_combine_invert", ep_combine_invert_kernel, dim3((int)blocks), dim3(256), 0, ctx, p);
}

cudaError_t launch_combine_reduce(const CombineReduceParams& p, const LaunchCtx& ctx) {
    const int ntiles = (p.H + kTileChannels - 1) / kTileChannels;
    const int grid = grid_for_warp_items((long long)p.T * ntiles, ctx, 8);
    auto k = p.direct ? ep_combine_reduce_kernel<true> : ep_combine_reduce_kernel<false>;
    return launch(p.direct ? "ep_combine_reduce_direct" : "ep_combine_reduce", k, dim3(grid), dim3(kThreads), 0, ctx, p);
}

}  // namespace mcep
