// Kernels of the elastic-style calls: see ep_elastic.cuh. None of them waits for
// another GPU; the exchange between the ranks is the group dispatch / combine.
#include "ep_elastic.cuh"

#include "ep_device.cuh"
#include "ep_kernels.cuh"

namespace mcep {
namespace {

constexpr unsigned kAll = 0xffffffffu;
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

__device__ __forceinline__ int rows_received(const int64_t* layout_range, int R, int* s_begin,
                                             int* s_end) {
    // (begin << 32) | count per source rank; the rows of all sources are [0, n)
    __shared__ int s_n;
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        const int64_t v = layout_range[r];
        const int begin = (int)(v >> 32), cnt = (int)(v & 0xffffffffll);
        if (s_begin) s_begin[r] = begin;
        if (s_end) s_end[r] = begin + cnt;
    }
    if (threadIdx.x < 32) {
        int n = 0;
        for (int r = threadIdx.x; r < R; r += 32) {
            const int64_t v = layout_range[r];
            n = max(n, (int)(v >> 32) + (int)(v & 0xffffffffll));
        }
        for (int d = 16; d > 0; d >>= 1) n = max(n, __shfl_xor_sync(kAll, n, d));
        if (threadIdx.x == 0) s_n = n;
    }
    __syncthreads();
    return s_n;
}

// Block-wide exclusive position of the threads whose `flag` is set, continuing
// from the positions earlier rounds handed out. All threads of the block call it.
__device__ __forceinline__ int block_position(bool flag, int* s_warp, int* s_base) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned bal = __ballot_sync(kAll, flag);
    if (lane == 0) s_warp[warp] = __popc(bal);
    __syncthreads();
    int before = *s_base;
    for (int i = 0; i < warp; ++i) before += s_warp[i];
    const int pos = before + __popc(bal & ((1u << lane) - 1u));
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int i = 0; i < kWarps; ++i) s += s_warp[i];
        *s_base += s;
    }
    __syncthreads();
    return pos;
}

// One block per destination rank r and 256 tokens: which tokens go to r, at which lane of their
// top-k list (the last one that names an expert of r, as `deduplicate` of
// mooncake_ep_elastic_ptx.cuh:690-693 elects), and in which position (token
// order, as the deterministic prologue of the reference assigns them:
// mooncake_ep_elastic_dispatch_deterministic_prologue.cuh:134-166). The block
// also stores, in rank r's memory, the record of every row r is about to get.
__global__ void __launch_bounds__(kThreads) ep_elastic_route_kernel(ElasticRouteParams p) {
    const int r = blockIdx.x;                 // destination rank
    const int first = blockIdx.y * kThreads;  // this block's 256 tokens
    const int L = p.E / p.R;
    pdl_launch_dependents();  // the exchange's first kernel may take its place; it waits for this one at its top
    __shared__ int s_warp[kWarps];
    __shared__ int s_base;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    {
        // tokens of the earlier blocks that go to rank r: counted again here (the index matrix
        // sits in L2) rather than waited for, so no block of this kernel depends on another
        int before = 0;
        for (int t = threadIdx.x; t < first; t += kThreads) {
            bool hit = false;
#pragma unroll
            for (int k = 0; k < kMaxTopk; ++k) {
                if (k >= p.K) break;
                const int64_t e = __ldg(p.topk_idx + (size_t)t * p.K + k);
                hit = hit || (e >= 0 && e < p.E && (int)e / L == r);
            }
            before += hit ? 1 : 0;
        }
        for (int d = 16; d > 0; d >>= 1) before += __shfl_xor_sync(kAll, before, d);
        if (lane == 0) s_warp[warp] = before;
        __syncthreads();
        if (threadIdx.x == 0) {
            int sum = 0;
            for (int i = 0; i < kWarps; ++i) sum += s_warp[i];
            s_base = sum;
        }
        __syncthreads();
    }
    {
        const int t = first + threadIdx.x;
        // the token's choices, all loaded before anything is stored
        int64_t raw[kMaxTopk];
        int rk[kMaxTopk];
        int master = -1;
        if (t < p.T) {
#pragma unroll
            for (int k = 0; k < kMaxTopk; ++k) raw[k] = k < p.K ? __ldg(p.topk_idx + (size_t)t * p.K + k) : -1;
#pragma unroll
            for (int k = 0; k < kMaxTopk; ++k) {
                rk[k] = (raw[k] >= 0 && raw[k] < p.E) ? (int)raw[k] / L : -1;
                if (rk[k] == r) master = k;
            }
        }
        const int slot = block_position(master >= 0, s_warp, &s_base);
        if (t >= p.T) return;
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
            if (k >= p.K) break;
            const size_t at = (size_t)t * p.K + k;
            if (rk[k] == r) {
                p.rank_topk[at] = (k == master) ? r : -1;
                p.dst_slot[at] = (k == master) ? p.rank * p.M + slot : -1;
            } else if (rk[k] < 0 && r == 0) {
                p.rank_topk[at] = -1;
                p.dst_slot[at] = -1;
            }
        }
        // what the receiver needs to know about the row, stored where it will look for it:
        // in rank r's memory, at this rank's region, at the row's position
        char* base = static_cast<char*>(p.record_base[r]);
        if (master >= 0 && base != nullptr) {
            char* rec = base + ((size_t)p.rank * p.M + slot) * p.record_stride;
#pragma unroll
            for (int k = 0; k < kMaxTopk; ++k) {
                if (k >= p.K) break;
                reinterpret_cast<int32_t*>(rec)[k] = rk[k] >= 0 ? (int32_t)raw[k] : -1;
                reinterpret_cast<float*>(rec)[p.K + k] =
                    p.topk_weights ? __ldg(p.topk_weights + (size_t)t * p.K + k) : 0.f;
            }
            reinterpret_cast<int32_t*>(rec)[2 * p.K] = t;
        }
        if (r != 0 || p.copied_topk_idx == nullptr) return;
#pragma unroll
        for (int k = 0; k < kMaxTopk; ++k) {
            if (k >= p.K) break;
            p.copied_topk_idx[(size_t)t * p.K + k] = raw[k];
        }
    }
}

// Receiver side, after the exchange: per received row the record its source
// stored here is turned into the row's local expert choices,
// weights and source metadata (mooncake_ep_elastic_dispatch_copy_epilogue.cuh:
// 114-132, 212-248); the last block to finish turns the per-expert hit counts
// into the aligned exclusive prefix sum of
// mooncake_ep_elastic_dispatch_official.cuh:255-310.
__global__ void __launch_bounds__(kThreads) ep_elastic_epilogue_kernel(ElasticEpilogueParams p) {
    __shared__ int s_begin[kMaxRanks], s_end[kMaxRanks];
    __shared__ bool s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();  // the exchange's kernels wrote the layout
    const int n = rows_received(p.layout_range, p.R, s_begin, s_end);
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        int run = 0;
        for (int r = 0; r < p.R; ++r) {
            run += s_end[r] - s_begin[r];
            p.psum_rank[r] = run;
        }
    }
    const int lo = p.rank * p.L;
    const int md_stride = p.K + 2;
    for (int i = blockIdx.x * kWarps + warp; i < n; i += gridDim.x * kWarps) {
        int src = -1;
        for (int r0 = 0; r0 < p.R && src < 0; r0 += 32) {
            const int r = r0 + lane;
            const unsigned b = __ballot_sync(kAll, r < p.R && i >= s_begin[r] && i < s_end[r]);
            if (b) src = r0 + __ffs(b) - 1;
        }
        if (src < 0) continue;
        // the record the source stored for its (i - begin)-th row, in this rank's memory
        const char* rec = p.records + ((size_t)src * p.M + (i - s_begin[src])) * p.record_stride;
        int e = -1;
        float w = 0.f;
        if (lane < p.K) {
            e = ld_s32_coherent(rec + 4 * lane);
            w = ld_f32_coherent(rec + 4 * (p.K + lane));
        }
        const int tok = ld_s32_coherent(rec + 8 * p.K);
        if (tok < 0 || tok >= p.M) {
            if (lane == 0) atomicOr(p.status, kStatusBadSource);
            continue;
        }
        const int local = (e >= lo && e < lo + p.L) ? e - lo : -1;
        const unsigned hit = __ballot_sync(kAll, local >= 0);
        const int master = hit ? 31 - __clz(hit) : 0;
        if (lane < p.K) {
            p.recv_topk_idx[(size_t)i * p.K + lane] = local;
            if (p.recv_topk_weights) p.recv_topk_weights[(size_t)i * p.K + lane] = w;
            if (local >= 0) atomicAdd(p.hist + local, 1);
            if (p.expand) p.recv_src_metadata[(size_t)i * md_stride + 2 + lane] = -1;
        }
        if (lane == 0) {
            p.recv_src_metadata[(size_t)i * md_stride] = src * p.M + tok;
            p.recv_src_metadata[(size_t)i * md_stride + 1] = src * p.K + master;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(p.ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (warp == 0) {
        int run = 0;
        for (int e0 = 0; e0 < p.L + 1; e0 += 32) {
            const int e = e0 + lane;
            // entry e of the exclusive sum adds the aligned count of expert e - 1
            int c = 0;
            if (e >= 1 && e <= p.L) {
                c = __ldcg(p.hist + e - 1);
                c = (c + p.alignment - 1) / p.alignment * p.alignment;
            }
            int v = c;
            for (int d = 1; d < 32; d <<= 1) {
                const int u = __shfl_up_sync(kAll, v, d);
                if (lane >= d) v += u;
            }
            if (e <= p.L) {
                p.psum_expert[e] = run + v;
                if (p.psum_start) p.psum_start[e] = run + v;
            }
            run += __shfl_sync(kAll, v, 31);
        }
        __syncwarp();
        for (int e = lane; e < p.L; e += 32) p.hist[e] = 0;
        if (lane == 0) *p.ticket = 0;
    }
}

// Expanded layout: one block per local expert numbers the rows that chose it, in
// receive order (the reference hands the positions out with an atomic, in
// arrival order: mooncake_ep_elastic_dispatch_copy_epilogue.cuh:138-141).
__global__ void __launch_bounds__(kThreads) ep_elastic_expand_scan_kernel(ElasticExpandParams p) {
    const int e = blockIdx.x;
    __shared__ int s_warp[kWarps];
    __shared__ int s_base;
    const int n = rows_received(p.layout_range, p.R, nullptr, nullptr);
    if (threadIdx.x == 0) s_base = 0;
    __syncthreads();
    const int start = p.psum_start[e];
    const int md_stride = p.K + 2;
    for (int i0 = 0; i0 < n; i0 += kThreads) {
        const int i = i0 + threadIdx.x;
        int k_hit = -1;
        if (i < n)
            for (int k = 0; k < p.K; ++k)
                if (p.recv_topk_idx[(size_t)i * p.K + k] == e) k_hit = k;
        const int pos = block_position(k_hit >= 0, s_warp, &s_base);
        if (k_hit >= 0) p.recv_src_metadata[(size_t)i * md_stride + 2 + k_hit] = start + pos;
    }
    if (threadIdx.x == 0) p.psum_expert[e] = start + s_base;
}

__device__ __forceinline__ void copy_row(void* dst, const void* src, int row_bytes, int lane) {
    for (int c = lane * 32; c < row_bytes; c += 32 * 32)
        st32(static_cast<char*>(dst) + c, ld32_coherent(static_cast<const char*>(src) + c));
}

__global__ void __launch_bounds__(kThreads) ep_elastic_expand_copy_kernel(ElasticExpandParams p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = rows_received(p.layout_range, p.R, nullptr, nullptr);
    const int md_stride = p.K + 2;
    for (int i = blockIdx.x * kWarps + warp; i < n; i += gridDim.x * kWarps) {
        const int slot = lane < p.K ? p.recv_src_metadata[(size_t)i * md_stride + 2 + lane] : -1;
        unsigned todo = __ballot_sync(kAll, slot >= 0);
        const char* src = static_cast<const char*>(p.flat_x) + (size_t)i * p.row_bytes;
        while (todo) {
            const int k = __ffs(todo) - 1;
            todo &= todo - 1;
            const int dst = __shfl_sync(kAll, slot, k);
            copy_row(static_cast<char*>(p.recv_x) + (size_t)dst * p.row_bytes, src, p.row_bytes, lane);
            if (p.recv_topk_weights && lane == 0)
                p.recv_topk_weights[dst] = p.flat_weights[(size_t)i * p.K + k];
        }
    }
}

// mooncake_ep_elastic_combine_official.cuh:146-216 with multiple reduction: one
// row is copied; two rows are added as the reference's bf16 add does (the exact
// sum rounded once, which an fp32 add followed by the bf16 rounding also gives);
// more are accumulated in fp32 from zero in listing order and rounded once.
__global__ void __launch_bounds__(kThreads) ep_elastic_local_reduce_kernel(ElasticLocalReduceParams p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = rows_received(p.layout_range, p.R, nullptr, nullptr);
    const int md_stride = p.K + 2;
    const int row_bytes = p.H * 2;
    for (int i = blockIdx.x * kWarps + warp; i < n; i += gridDim.x * kWarps) {
        const int slot = lane < p.K ? p.recv_src_metadata[(size_t)i * md_stride + 2 + lane] : -1;
        const unsigned valid = __ballot_sync(kAll, slot >= 0);
        const int cnt = __popc(valid);
        char* dst = static_cast<char*>(p.y) + (size_t)i * row_bytes;
        if (cnt == 0) continue;
        if (cnt == 1) {
            const int s = __shfl_sync(kAll, slot, __ffs(valid) - 1);
            for (int c = lane * 32; c < row_bytes; c += 32 * 32)
                st32(dst + c, ld32_readonly(static_cast<const char*>(p.x) + (size_t)s * row_bytes + c));
            continue;
        }
        // the rows to add, in listing order (gathered before the lanes' loops part ways)
        int rows[kMaxTopk];
        {
            unsigned todo = valid;
#pragma unroll
            for (int j = 0; j < kMaxTopk; ++j) {
                const int k = todo ? __ffs(todo) - 1 : 0;
                const int s = __shfl_sync(kAll, slot, k);
                rows[j] = todo ? s : -1;
                todo &= todo - 1;
            }
        }
        for (int c = lane * 32; c < row_bytes; c += 32 * 32) {
            float acc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[j] = 0.f;
#pragma unroll
            for (int m = 0; m < kMaxTopk; ++m) {
                if (m >= cnt) break;
                const V32 v = ld32_readonly(static_cast<const char*>(p.x) + (size_t)rows[m] * row_bytes + c);
                // two rows: a + b, not 0 + a + b (the sign of a zero sum differs)
                const bool first = m == 0 && cnt == 2;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    acc[2 * j] = first ? bf16lo(v.w[j]) : __fadd_rn(acc[2 * j], bf16lo(v.w[j]));
                    acc[2 * j + 1] = first ? bf16hi(v.w[j]) : __fadd_rn(acc[2 * j + 1], bf16hi(v.w[j]));
                }
            }
            st32(dst + c, pack_bf16x16(acc));
        }
    }
}

__global__ void ep_elastic_fill_ones_kernel(float* w, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        w[i] = 1.0f;
}

}  // namespace

cudaError_t launch_elastic_route(const ElasticRouteParams& p, cudaStream_t stream) {
    LaunchScope scope("ep_elastic_route", stream);
    const int chunks = p.T > 0 ? (p.T + kThreads - 1) / kThreads : 1;
    ep_elastic_route_kernel<<<dim3(p.R, chunks), kThreads, 0, stream>>>(p);
    return scope.done(cudaGetLastError());
}

cudaError_t launch_elastic_epilogue(const ElasticEpilogueParams& p, int num_sms, cudaStream_t stream,
                                    bool pdl) {
    const int cap_blocks = (p.R * p.M + kWarps - 1) / kWarps;
    const int grid = max(1, min(2 * num_sms, cap_blocks));
    LaunchScope scope("ep_elastic_epilogue", stream);
    // with `pdl` the blocks may become resident while the exchange's last kernel drains;
    // they wait for its completion before they read anything
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kThreads), cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr, cfg.numAttrs = 1;
    }
    return scope.done(cudaLaunchKernelEx(&cfg, ep_elastic_epilogue_kernel, p));
}

cudaError_t launch_elastic_expand_scan(const ElasticExpandParams& p, cudaStream_t stream) {
    LaunchScope scope("ep_elastic_expand_scan", stream);
    ep_elastic_expand_scan_kernel<<<p.L, kThreads, 0, stream>>>(p);
    return scope.done(cudaGetLastError());
}

cudaError_t launch_elastic_expand_copy(const ElasticExpandParams& p, int num_sms, cudaStream_t stream) {
    LaunchScope scope("ep_elastic_expand_copy", stream);
    ep_elastic_expand_copy_kernel<<<4 * num_sms, kThreads, 0, stream>>>(p);
    return scope.done(cudaGetLastError());
}

cudaError_t launch_elastic_local_reduce(const ElasticLocalReduceParams& p, int num_sms,
                                        cudaStream_t stream) {
    LaunchScope scope("ep_elastic_local_reduce", stream);
    ep_elastic_local_reduce_kernel<<<4 * num_sms, kThreads, 0, stream>>>(p);
    return scope.done(cudaGetLastError());
}

cudaError_t launch_elastic_fill_ones(float* w, size_t n, cudaStream_t stream) {
    LaunchScope scope("ep_elastic_fill_ones", stream);
    ep_elastic_fill_ones_kernel<<<64, 256, 0, stream>>>(w, n);
    return scope.done(cudaGetLastError());
}

}  // namespace mcep
