// Elastic-style entry points of the C ABI (include/mcep.h): flat receive layout,
// one copy of a token per destination rank.
//
// Counterpart of mooncake-ep/src/mooncake_ep_elastic_buffer.cpp:230-426. The
// exchange between the ranks is mcep_dispatch / mcep_combine with num_experts =
// num_ranks (every rank one "expert", a token listed once per rank it has to
// reach); the kernels of ep_elastic_kernels.cu prepare that routing and turn the
// exchange's outputs into the tensors of the elastic interface. What the
// receiver needs to know about a row beyond its payload (the token's expert
// choices, weights and index) travels ahead of it: before the exchange starts,
// the source stores a record per row in the receiver's symmetric memory, at the
// position the row will take inside the source's segment.
#include "ep_elastic.cuh"

#include <cstdio>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "../../include/mcep.h"
#include "ep_kernels.cuh"
#include "ep_runtime_internal.h"

namespace {

using mcep::report_failure;

#define EL_CUDA(expr)                                                                       \
    do {                                                                                    \
        cudaError_t e_ = (expr);                                                            \
        if (e_ != cudaSuccess) {                                                            \
            char m_[512];                                                                   \
            snprintf(m_, sizeof(m_), "Failed: CUDA error %s:%d '%s' (%s)", __FILE__, __LINE__, \
                     cudaGetErrorString(e_), #expr);                                        \
            return report_failure(MCEP_ERR_CUDA, m_);                                       \
        }                                                                                   \
    } while (0)

#define EL_REQUIRE(cond)                                                                    \
    do {                                                                                    \
        if (!(cond)) {                                                                      \
            char m_[512];                                                                   \
            snprintf(m_, sizeof(m_), "Failed: Assertion error %s:%d '%s'", __FILE__, __LINE__, #cond); \
            return report_failure(MCEP_ERR_INVALID, m_);                                    \
        }                                                                                   \
    } while (0)

size_t up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// The record areas end where the data area ends, rounded down so that they stay
// 16-byte aligned whatever size the caller gave the buffer.
size_t usable_bytes(int64_t num_bytes) { return num_bytes > 0 ? (size_t)num_bytes / 16 * 16 : 0; }

int record_stride(int K) { return (int)up(8 * (size_t)K + 4, 16); }
size_t record_bytes(int R, int M, int K) { return up((size_t)R * M * record_stride(K), 256); }

// What the entry points keep per buffer between calls.
struct ElasticState {
    int R = 0, M = 0, K = 0, L = 0, H = 0;  // capacities of the carve-up below
    bool group = false;
    char* blob = nullptr;
    int32_t* src_info[2] = {};
    int64_t* layout_range[2] = {};
    int32_t* recv_count[2] = {};
    int64_t* rank_topk[2] = {};
    char* own_records[2] = {};  // a single rank without symmetric memory keeps its records here
    float* ones = nullptr;
    float* flat_weights = nullptr;
    int32_t* psum_start = nullptr;
    int32_t* hist = nullptr;
    unsigned* ticket = nullptr;
    void** record_table = nullptr;  // device [2][R]
    void* flat_x = nullptr;         // single rank: flat rows before they are expanded / after the local sums
    std::vector<void*> table_host;
    cudaEvent_t ev = nullptr;
    struct Record {
        const void* key = nullptr;  // the handle's recv_src_metadata tensor
        int par = 0, T = 0, K = 0, E = 0, M = 0, H = 0, expand = 0;
        uint64_t stamp = 0;
    } rec[2];
    uint64_t clock = 0;
    uint32_t calls = 0;
    // The record areas sit at fixed places for the life of the buffer (fixed by its first
    // elastic call): a peer may still be reading one call's records while the next call's are
    // being stored, so the two areas must not move with the shapes of the calls.
    size_t record_area_bytes = 0;
    bool comm_stream_busy = false;  // a call was queued on the communication stream and not yet waited for here
};

std::mutex g_mu;
std::unordered_map<mcep_buffer*, ElasticState*> g_states;

ElasticState* state_of(mcep_buffer* b) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_states.find(b);
    if (it != g_states.end()) return it->second;
    auto* s = new ElasticState();
    g_states[b] = s;
    return s;
}

void free_blob(ElasticState* s) {
    if (s->blob) cudaFree(s->blob);
    s->blob = nullptr;
}

// (Re)allocates the scratch when a call needs more than the last ones did.
int ensure(ElasticState* s, const mcep::BufferView& v, int M, int K, int L, int H, cudaStream_t stream) {
    const int R = v.num_ranks;
    if (s->blob && R == s->R && M <= s->M && K <= s->K && L <= s->L && H <= s->H && v.group == s->group)
        return MCEP_OK;
    EL_CUDA(cudaDeviceSynchronize());
    free_blob(s);
    M = M > s->M ? M : s->M, K = K > s->K ? K : s->K, L = L > s->L ? L : s->L, H = H > s->H ? H : s->H;
    const size_t RM = (size_t)R * M;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off += up(bytes, 256);
        return at;
    };
    size_t o_src[2], o_lr[2], o_cnt[2], o_topk[2], o_rec[2];
    for (int p = 0; p < 2; ++p) {
        o_src[p] = take(RM * 4), o_lr[p] = take((size_t)R * 8), o_cnt[p] = take(64);
        o_topk[p] = take((size_t)M * K * 8);
        o_rec[p] = v.group ? 0 : take(record_bytes(R, M, K));
    }
    const size_t o_ones = take((size_t)M * K * 4), o_fw = take(RM * K * 4);
    const size_t o_ps = take((size_t)(L + 1) * 4), o_hist = take((size_t)L * 4 + 4), o_tick = take(64);
    const size_t o_tab = take(2 * (size_t)R * sizeof(void*));
    const size_t o_flat = v.group ? 0 : take(RM * 2 * (size_t)H);
    EL_CUDA(cudaMalloc(&s->blob, off));
    EL_CUDA(cudaMemsetAsync(s->blob, 0, off, stream));
    for (int p = 0; p < 2; ++p) {
        s->src_info[p] = reinterpret_cast<int32_t*>(s->blob + o_src[p]);
        s->layout_range[p] = reinterpret_cast<int64_t*>(s->blob + o_lr[p]);
        s->recv_count[p] = reinterpret_cast<int32_t*>(s->blob + o_cnt[p]);
        s->rank_topk[p] = reinterpret_cast<int64_t*>(s->blob + o_topk[p]);
        s->own_records[p] = v.group ? nullptr : s->blob + o_rec[p];
    }
    s->ones = reinterpret_cast<float*>(s->blob + o_ones);
    s->flat_weights = reinterpret_cast<float*>(s->blob + o_fw);
    s->psum_start = reinterpret_cast<int32_t*>(s->blob + o_ps);
    s->hist = reinterpret_cast<int32_t*>(s->blob + o_hist);
    s->ticket = reinterpret_cast<unsigned*>(s->blob + o_tick);
    s->record_table = reinterpret_cast<void**>(s->blob + o_tab);
    s->flat_x = v.group ? nullptr : s->blob + o_flat;
    s->table_host.assign(2 * (size_t)R, nullptr);
    s->R = R, s->M = M, s->K = K, s->L = L, s->H = H, s->group = v.group;
    for (auto& r : s->rec) r = ElasticState::Record();
    EL_CUDA(mcep::launch_elastic_fill_ones(s->ones, (size_t)M * K, stream));
    if (!s->ev) EL_CUDA(cudaEventCreateWithFlags(&s->ev, cudaEventDisableTiming));
    return MCEP_OK;
}

// Where every rank keeps the records of the call with this parity. In a group:
// at the end of the data area of the symmetric allocation, same offset on every
// rank.
int refresh_record_table(ElasticState* s, const mcep::BufferView& v, int par, size_t rec_bytes) {
    const int R = v.num_ranks;
    std::vector<void*> want(R, nullptr);
    for (int r = 0; r < R; ++r) {
        if (!v.group)
            want[r] = s->own_records[par];
        else if (v.peer_host[r] != nullptr)
            want[r] = static_cast<char*>(v.peer_host[r]) + v.data_off + usable_bytes(v.num_bytes) -
                      (size_t)(par + 1) * rec_bytes;
    }
    bool same = true;
    for (int r = 0; r < R; ++r) same = same && s->table_host[(size_t)par * R + r] == want[r];
    if (same) return MCEP_OK;
    EL_CUDA(cudaMemcpy(s->record_table + (size_t)par * R, want.data(), sizeof(void*) * R,
                       cudaMemcpyHostToDevice));
    for (int r = 0; r < R; ++r) s->table_host[(size_t)par * R + r] = want[r];
    return MCEP_OK;
}

int pick_stream(ElasticState* s, const mcep::BufferView& v, bool async, uint64_t compute_stream,
                cudaStream_t* out) {
    cudaStream_t compute = reinterpret_cast<cudaStream_t>(compute_stream);
    *out = compute;
    if (!async) {
        // the calls of a buffer share scratch: one that runs on the caller's stream waits for
        // what earlier calls left on the communication stream
        if (s->comm_stream_busy) {
            EL_CUDA(cudaEventRecord(s->ev, v.comm_stream));
            EL_CUDA(cudaStreamWaitEvent(compute, s->ev, 0));
            s->comm_stream_busy = false;
        }
        return MCEP_OK;
    }
    // as the reference: the communication stream, behind everything queued on the caller's
    EL_CUDA(cudaEventRecord(s->ev, compute));
    EL_CUDA(cudaStreamWaitEvent(v.comm_stream, s->ev, 0));
    s->comm_stream_busy = true;
    *out = v.comm_stream;
    return MCEP_OK;
}

}  // namespace

namespace mcep {

void elastic_release(mcep_buffer* b) {
    ElasticState* s = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_states.find(b);
        if (it == g_states.end()) return;
        s = it->second;
        g_states.erase(it);
    }
    free_blob(s);
    if (s->ev) cudaEventDestroy(s->ev);
    delete s;
}

}  // namespace mcep

extern "C" {

uint64_t mcep_elastic_buffer_size_hint(int M, int hidden, int num_ranks, int num_topk) {
    if (M <= 0 || hidden <= 0 || num_ranks <= 0 || num_topk <= 0) return 0;
    return up(mcep::exchange_bytes(num_ranks, num_ranks, M, hidden) + 2 * record_bytes(num_ranks, M, num_topk), 256);
}

int mcep_elastic_dispatch(mcep_buffer* b, const mcep_elastic_dispatch_args* a, mcep_event** out_event) {
    EL_REQUIRE(b != nullptr && a != nullptr && out_event != nullptr);
    *out_event = nullptr;
    const mcep::BufferView v = mcep::view_of(b);
    const int R = v.num_ranks, E = a->num_experts, M = a->num_max_tokens_per_rank;
    const int T = a->num_tokens, H = a->hidden, K = a->num_topk;
    // checks of mooncake_ep_elastic_buffer.cpp:241-271
    EL_REQUIRE(E > 0 && E % R == 0);
    EL_REQUIRE(a->x_element_size == 2 && a->sf == nullptr && a->num_sf_packs == 0 &&
               a->recv_x_scales == nullptr);
    EL_REQUIRE(T >= 0 && T <= M && H > 0 && K >= 1 && K <= MCEP_MAX_TOPK);
    EL_REQUIRE(a->expert_alignment >= 1);
    EL_REQUIRE(a->active_ranks != nullptr && (T == 0 || (a->x != nullptr && a->topk_idx != nullptr)));
    EL_REQUIRE(a->psum_num_recv_tokens_per_scaleup_rank != nullptr);
    EL_REQUIRE(a->psum_num_recv_tokens_per_expert != nullptr && (T == 0 || a->dst_buffer_slot_idx != nullptr));
    EL_REQUIRE(a->recv_x != nullptr && a->recv_topk_idx != nullptr && a->recv_src_metadata != nullptr);
    const int L = E / R;
    ElasticState* s = state_of(b);
    const size_t rec_want = record_bytes(R, M, K);
    const size_t rec_bytes = (v.group && s->record_area_bytes != 0) ? s->record_area_bytes : rec_want;
    if (rec_want > rec_bytes)
        return report_failure(MCEP_ERR_INVALID,
                              "Failed: Assertion error 'elastic calls of one buffer need no more record "
                              "space (num_max_tokens_per_rank, num_topk) than its first elastic call'");
    if (v.group && mcep::exchange_bytes(R, R, M, H) + 2 * rec_bytes > usable_bytes(v.num_bytes)) {
        char m[256];
        snprintf(m, sizeof(m),
                 "Failed: Assertion error %s:%d 'elastic layout fits num_ep_buffer_bytes' (need %zu, have %lld)",
                 __FILE__, __LINE__, mcep::exchange_bytes(R, R, M, H) + 2 * rec_bytes, (long long)v.num_bytes);
        return report_failure(MCEP_ERR_INVALID, m);
    }

    cudaStream_t stream = nullptr;
    // the scratch is set up on the caller's stream, ahead of everything this call queues
    if (int rc = ensure(s, v, M, K, L, H, reinterpret_cast<cudaStream_t>(a->compute_stream))) return rc;
    if (int rc = pick_stream(s, v, a->async_with_compute_stream != 0, a->compute_stream, &stream)) return rc;
    if (v.group) s->record_area_bytes = rec_bytes;
    const int par = (int)(++s->calls & 1u);
    if (int rc = refresh_record_table(s, v, par, rec_bytes)) return rc;

    mcep::ElasticRouteParams rp = {};
    rp.topk_idx = a->topk_idx, rp.topk_weights = a->topk_weights;
    rp.T = T, rp.K = K, rp.E = E, rp.R = R, rp.M = M, rp.rank = v.rank;
    rp.rank_topk = s->rank_topk[par], rp.dst_slot = a->dst_buffer_slot_idx;
    rp.copied_topk_idx = a->copied_topk_idx;
    rp.record_base = s->record_table + (size_t)par * R;
    rp.record_stride = record_stride(K);
    EL_CUDA(mcep::launch_elastic_route(rp, stream));

    // the exchange: ranks as experts
    void* flat = a->recv_x;
    if (a->do_expand) {
        flat = s->flat_x;
        if (v.group) {
            size_t bytes = 0;
            if (int rc = mcep_buffer_next_recv_x(b, M, H, R, 0, &flat, &bytes)) return rc;
            EL_REQUIRE(flat != nullptr);
        }
    }
    mcep_dispatch_args da = {};
    da.x = a->x, da.topk_idx = s->rank_topk[par], da.active_ranks = a->active_ranks;
    da.num_tokens = T, da.hidden = H, da.num_topk = K, da.num_max_dispatch_tokens_per_rank = M;
    da.num_experts = R, da.use_fp8 = 0, da.timeout_us = a->timeout_us;
    da.packed_recv_x = flat, da.packed_recv_x_scales = nullptr;
    da.packed_recv_count = s->recv_count[par], da.packed_recv_src_info = s->src_info[par];
    da.packed_recv_layout_range = s->layout_range[par];
    da.async_finish = 0, da.return_recv_hook = 0;
    da.compute_stream = reinterpret_cast<uint64_t>(stream);
    mcep_event* ev = nullptr;
    mcep_hook* hook = nullptr;
    // the route kernel lets its dependents start early; the exchange's first kernel waits for it
    mcep::allow_chained_first_launch(b);
    if (int rc = mcep_dispatch(b, &da, &ev, &hook)) return rc;

    auto& rec = s->rec[par];
    rec.key = a->recv_src_metadata, rec.par = par, rec.T = T, rec.K = K, rec.E = E, rec.M = M, rec.H = H;
    rec.expand = a->do_expand != 0, rec.stamp = ++s->clock;

    mcep::ElasticEpilogueParams ep = {};
    ep.layout_range = s->layout_range[par];
    ep.records = static_cast<const char*>(s->table_host[(size_t)par * R + v.rank]);
    ep.record_stride = rp.record_stride;
    ep.R = R, ep.M = M, ep.K = K, ep.L = L, ep.rank = v.rank;
    ep.alignment = a->expert_alignment, ep.expand = a->do_expand != 0;
    ep.recv_topk_idx = a->recv_topk_idx;
    ep.recv_topk_weights = a->do_expand ? s->flat_weights : a->recv_topk_weights;
    ep.recv_src_metadata = a->recv_src_metadata;
    ep.psum_rank = a->psum_num_recv_tokens_per_scaleup_rank;
    ep.psum_expert = a->psum_num_recv_tokens_per_expert;
    ep.psum_start = a->do_expand ? s->psum_start : nullptr;
    ep.hist = s->hist, ep.ticket = s->ticket, ep.status = v.status;

    mcep::ElasticExpandParams xp = {};
    xp.layout_range = s->layout_range[par], xp.recv_topk_idx = a->recv_topk_idx;
    xp.flat_weights = a->recv_topk_weights ? s->flat_weights : nullptr;
    xp.flat_x = flat;
    xp.R = R, xp.K = K, xp.L = L, xp.row_bytes = 2 * H;
    xp.psum_start = s->psum_start, xp.psum_expert = a->psum_num_recv_tokens_per_expert;
    xp.recv_src_metadata = a->recv_src_metadata, xp.recv_x = a->recv_x;
    xp.recv_topk_weights = a->recv_topk_weights;

    const int num_sms = v.num_sms;
    const bool expand = a->do_expand != 0;
    const bool pdl = !v.defer;
    auto after = [=]() -> int {
        EL_CUDA(mcep::launch_elastic_epilogue(ep, num_sms, stream, pdl));
        if (expand) {
            EL_CUDA(mcep::launch_elastic_expand_scan(xp, stream));
            EL_CUDA(mcep::launch_elastic_expand_copy(xp, num_sms, stream));
        }
        return MCEP_OK;
    };
    if (v.defer) {
        EL_REQUIRE(!a->async_with_compute_stream);
        mcep::set_after_deferred(b, after);
        return MCEP_OK;
    }
    if (int rc = after()) return rc;
    if (a->async_with_compute_stream) return mcep_event_create(reinterpret_cast<uint64_t>(stream), out_event);
    return MCEP_OK;
}

int mcep_elastic_combine(mcep_buffer* b, const mcep_elastic_combine_args* a, mcep_event** out_event) {
    EL_REQUIRE(b != nullptr && a != nullptr && out_event != nullptr);
    *out_event = nullptr;
    const mcep::BufferView v = mcep::view_of(b);
    const int R = v.num_ranks, M = a->num_max_tokens_per_rank;
    const int T = a->num_combined_tokens, H = a->hidden, K = a->num_topk;
    // checks of mooncake_ep_elastic_buffer.cpp:371-376
    EL_REQUIRE((a->topk_idx != nullptr || T == 0) && a->recv_src_metadata != nullptr &&
               a->active_ranks != nullptr);
    EL_REQUIRE(a->combined_x != nullptr || T == 0);
    EL_REQUIRE(a->x != nullptr || a->num_input_tokens == 0);
    ElasticState* s = state_of(b);
    const ElasticState::Record* rec = nullptr;
    for (const auto& c : s->rec)
        if (c.key != nullptr && c.key == a->recv_src_metadata && (rec == nullptr || c.stamp > rec->stamp))
            rec = &c;
    if (rec == nullptr)
        return report_failure(MCEP_ERR_STATE,
                              "Failed: Assertion error 'elastic combine needs the handle of one of the last "
                              "two elastic dispatch calls of this buffer'");
    if (rec->T != T || rec->K != K || rec->M != M || rec->H != H || rec->E != a->num_experts ||
        rec->expand != (a->do_expand != 0))
        return report_failure(MCEP_ERR_INVALID,
                              "Failed: Assertion error 'elastic combine arguments match the dispatch call of "
                              "the handle'");
    const int par = rec->par;
    cudaStream_t stream = nullptr;
    if (int rc = pick_stream(s, v, a->async_with_compute_stream != 0, a->compute_stream, &stream)) return rc;

    const void* x = a->x;
    int zero_copy = 0;
    if (rec->expand) {
        void* y = s->flat_x;
        if (v.group) {
            size_t bytes = 0;
            if (int rc = mcep_buffer_next_combine_buffer(b, M, H, R, &y, &bytes)) return rc;
            EL_REQUIRE(y != nullptr);
            zero_copy = 1;
        }
        mcep::ElasticLocalReduceParams lp = {};
        lp.layout_range = s->layout_range[par], lp.recv_src_metadata = a->recv_src_metadata;
        lp.x = a->x, lp.R = R, lp.K = K, lp.H = H, lp.y = y;
        EL_CUDA(mcep::launch_elastic_local_reduce(lp, v.num_sms, stream));
        x = y;
    }
    mcep_combine_args ca = {};
    ca.x = x, ca.topk_idx = s->rank_topk[par], ca.topk_weights = s->ones;
    ca.src_info = s->src_info[par], ca.layout_range = s->layout_range[par];
    ca.active_ranks = a->active_ranks;
    ca.num_local_experts = 1, ca.num_combined_tokens = T, ca.hidden = H, ca.num_topk = K;
    ca.num_max_dispatch_tokens_per_rank = M, ca.num_experts = R, ca.timeout_us = a->timeout_us;
    ca.zero_copy = zero_copy, ca.combined_x = a->combined_x;
    ca.async_finish = 0, ca.return_recv_hook = 0;
    ca.compute_stream = reinterpret_cast<uint64_t>(stream);
    mcep_event* ev = nullptr;
    mcep_hook* hook = nullptr;
    if (int rc = mcep_combine(b, &ca, &ev, &hook)) return rc;
    if (a->async_with_compute_stream && !v.defer)
        return mcep_event_create(reinterpret_cast<uint64_t>(stream), out_event);
    return MCEP_OK;
}

}  // extern "C"
