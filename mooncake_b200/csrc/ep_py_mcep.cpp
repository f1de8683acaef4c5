// A pybind11 binding of the C ABI (include/mcep.h) with the surface of the
// reference's compiled module `mooncake._ep` (mooncake-ep/src/ep_py.cpp:14-87):
// `Buffer`, `ElasticBuffer`, `EventHandle`, `get_ep_buffer_size_hint`,
// `calculate_elastic_buffer_size`, `MAX_QP_COUNT`. It is what a maintainer who wants
// to keep `_ep` a compiled module would put in place of ep_py.cpp; the package
// itself uses the ctypes binding (mooncake_b200/ep.py) and does not need it.
//
//   g++ -O2 -shared -fPIC -std=c++17 $(python -m pybind11 --includes) \
//       -I include mooncake_b200/csrc/ep_py_mcep.cpp -o _ep$(python3-config --extension-suffix) \
//       -L mooncake_b200 -l:libmcep.so -Wl,-rpath,'$ORIGIN'
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <cstdint>
#include <functional>
#include <memory>
#include <optional>
#include <stdexcept>
#include <tuple>
#include <vector>

#include "mcep.h"

namespace py = pybind11;

namespace {

void check(int rc) {
    // EPException surfaces as RuntimeError in the reference
    // (mooncake-ep/include/mooncake_ep_exception.cuh:12-24)
    if (rc) throw std::runtime_error(mcep_last_error());
}

struct Event {  // mooncake-ep/include/mooncake_ep_event.h:9-44
    mcep_event* h = nullptr;
    explicit Event(uint64_t stream) { check(mcep_event_create(stream, &h)); }
    explicit Event(mcep_event* adopt) : h(adopt) {}
    Event(const Event&) = delete;
    ~Event() { mcep_event_free(h); }
    void current_stream_wait(uint64_t s) const { check(mcep_event_current_stream_wait(h, s)); }
    void synchronize() const { check(mcep_event_synchronize(h)); }
};

using CallResult = std::tuple<std::optional<std::shared_ptr<Event>>, std::optional<std::function<void()>>>;

CallResult wrap(mcep_event* ev, mcep_hook* hk) {
    CallResult r;
    if (ev) std::get<0>(r) = std::make_shared<Event>(ev);
    if (hk) {
        std::shared_ptr<mcep_hook> keep(hk, mcep_hook_free);
        std::get<1>(r) = [keep]() { check(mcep_hook_run(keep.get())); };
    }
    return r;
}

struct Buffer {  // mooncake-ep/include/mooncake_ep_buffer.h:65-195
    mcep_buffer* h = nullptr;
    int num_ranks;
    Buffer(int rank, int num_ranks_, int64_t bytes, bool disable_p2p) : num_ranks(num_ranks_) {
        check(mcep_buffer_create(rank, num_ranks_, bytes, disable_p2p ? 1 : 0, &h));
    }
    Buffer(const Buffer&) = delete;
    ~Buffer() { mcep_buffer_destroy(h); }

    // the RDMA surface: there is no RDMA route behind this library
    bool ibgda_disabled() const { return true; }
    bool is_roce() const { return false; }
    void update_local_qpns() {}
    void sync_ibgda_peers(py::args) {}
    std::pair<uint64_t, uint32_t> get_mr_info() const { return {0, 0}; }
    std::pair<uint64_t, uint64_t> get_gid() const { return {0, 0}; }
    std::vector<int32_t> get_local_qpns() const { return {}; }
    std::vector<int32_t> get_local_lids() const { return {}; }

    bool p2p_enabled() const { return mcep_buffer_p2p_enabled(h) != 0; }
    bool use_fast_path() const { return mcep_buffer_use_fast_path(h) != 0; }
    std::vector<int32_t> get_ipc_handle() {
        std::vector<int32_t> v(MCEP_FABRIC_HANDLE_INT32S);  // room for either kind of handle
        int n = 0;
        check(mcep_buffer_get_ipc_handle(h, v.data(), (int)v.size(), &n));
        v.resize(n);
        return v;
    }
    void sync_nvlink_ipc_handles(const std::vector<std::vector<int32_t>>& handles,
                                 const std::vector<int32_t>& active_ranks_mask) {
        size_t per = MCEP_IPC_HANDLE_INT32S;
        for (const auto& h : handles) per = std::max(per, h.size());
        std::vector<int32_t> flat((size_t)num_ranks * per, 0);
        std::vector<int32_t> mask(num_ranks, 1);
        for (int r = 0; r < num_ranks && r < (int)handles.size(); ++r)
            std::copy(handles[r].begin(), handles[r].end(), flat.begin() + (size_t)r * per);
        for (int r = 0; r < num_ranks && r < (int)active_ranks_mask.size(); ++r) mask[r] = active_ranks_mask[r];
        check(mcep_buffer_sync_nvlink_ipc_handles(h, flat.data(), (int)per, mask.data()));
    }

    // mooncake-ep/include/mooncake_ep_buffer.h:116-124
    CallResult dispatch(uint64_t x, uint64_t topk_idx, uint64_t active_ranks, int num_tokens, int hidden,
                        int num_topk, int num_max_dispatch_tokens_per_rank, int num_experts,
                        int64_t timeout_us, bool use_fp8, uint64_t packed_recv_x,
                        uint64_t packed_recv_x_scales, uint64_t packed_recv_count,
                        uint64_t packed_recv_src_info, uint64_t packed_recv_layout_range, bool async_finish,
                        bool return_recv_hook, uint64_t compute_stream) {
        mcep_dispatch_args a = {};
        a.x = reinterpret_cast<const void*>(x);
        a.topk_idx = reinterpret_cast<const int64_t*>(topk_idx);
        a.active_ranks = reinterpret_cast<int32_t*>(active_ranks);
        a.num_tokens = num_tokens, a.hidden = hidden, a.num_topk = num_topk;
        a.num_max_dispatch_tokens_per_rank = num_max_dispatch_tokens_per_rank;
        a.num_experts = num_experts, a.use_fp8 = use_fp8 ? 1 : 0, a.timeout_us = timeout_us;
        a.packed_recv_x = reinterpret_cast<void*>(packed_recv_x);
        a.packed_recv_x_scales = reinterpret_cast<float*>(packed_recv_x_scales);
        a.packed_recv_count = reinterpret_cast<int32_t*>(packed_recv_count);
        a.packed_recv_src_info = reinterpret_cast<int32_t*>(packed_recv_src_info);
        a.packed_recv_layout_range = reinterpret_cast<int64_t*>(packed_recv_layout_range);
        a.async_finish = async_finish ? 1 : 0, a.return_recv_hook = return_recv_hook ? 1 : 0;
        a.compute_stream = compute_stream;
        mcep_event* ev = nullptr;
        mcep_hook* hk = nullptr;
        check(mcep_dispatch(h, &a, &ev, &hk));
        return wrap(ev, hk);
    }

    // mooncake-ep/include/mooncake_ep_buffer.h:126-133
    CallResult combine(uint64_t x, uint64_t topk_idx, uint64_t topk_weights, uint64_t src_info,
                       uint64_t layout_range, uint64_t active_ranks, int num_local_experts,
                       int num_combined_tokens, int hidden, int num_topk,
                       int num_max_dispatch_tokens_per_rank, int num_experts, int64_t timeout_us,
                       bool zero_copy, uint64_t combined_x, bool async_finish, bool return_recv_hook,
                       uint64_t compute_stream) {
        mcep_combine_args a = {};
        a.x = reinterpret_cast<const void*>(x);
        a.topk_idx = reinterpret_cast<const int64_t*>(topk_idx);
        a.topk_weights = reinterpret_cast<const float*>(topk_weights);
        a.src_info = reinterpret_cast<const int32_t*>(src_info);
        a.layout_range = reinterpret_cast<const int64_t*>(layout_range);
        a.active_ranks = reinterpret_cast<int32_t*>(active_ranks);
        a.num_local_experts = num_local_experts, a.num_combined_tokens = num_combined_tokens;
        a.hidden = hidden, a.num_topk = num_topk;
        a.num_max_dispatch_tokens_per_rank = num_max_dispatch_tokens_per_rank;
        a.num_experts = num_experts, a.timeout_us = timeout_us, a.zero_copy = zero_copy ? 1 : 0;
        a.combined_x = reinterpret_cast<void*>(combined_x);
        a.async_finish = async_finish ? 1 : 0, a.return_recv_hook = return_recv_hook ? 1 : 0;
        a.compute_stream = compute_stream;
        mcep_event* ev = nullptr;
        mcep_hook* hk = nullptr;
        check(mcep_combine(h, &a, &ev, &hk));
        return wrap(ev, hk);
    }

    // additions of this library (include/mcep.h): where the next dispatch lands
    // its rows in place, and the tensor a zero-copy combine reads
    std::pair<uint64_t, size_t> next_recv_x(int M, int hidden, int num_experts, bool use_fp8) {
        void* p = nullptr;
        size_t n = 0;
        check(mcep_buffer_next_recv_x(h, M, hidden, num_experts, use_fp8 ? 1 : 0, &p, &n));
        return {reinterpret_cast<uint64_t>(p), n};
    }
    std::pair<uint64_t, size_t> next_combine_buffer(int M, int hidden, int num_experts) {
        void* p = nullptr;
        size_t n = 0;
        check(mcep_buffer_next_combine_buffer(h, M, hidden, num_experts, &p, &n));
        return {reinterpret_cast<uint64_t>(p), n};
    }
};

// mooncake-ep/include/elastic/mooncake_ep_elastic_buffer.h:38-110, for one NVLink domain
struct ElasticBuffer : Buffer {
    int rank;
    int64_t gpu_timeout_secs;
    ElasticBuffer(int rank_, int num_ranks_, int64_t num_buffer_bytes, int64_t /*num_max_tokens_per_rank*/,
                  int64_t /*hidden*/, int64_t /*num_topk*/, bool use_fp8_dispatch, bool /*deterministic*/,
                  bool /*allow_hybrid_mode*/, bool allow_multiple_reduction, bool /*prefer_overlap_with_compute*/,
                  int /*sl_idx*/, int /*num_allocated_qps*/, int /*num_cpu_timeout_secs*/, int num_gpu_timeout_secs)
        : Buffer(checked_rank(rank_, use_fp8_dispatch, allow_multiple_reduction), num_ranks_, num_buffer_bytes,
                 false),
          rank(rank_),
          gpu_timeout_secs(num_gpu_timeout_secs) {}
    // what is not built is refused before anything is allocated
    static int checked_rank(int rank, bool use_fp8_dispatch, bool allow_multiple_reduction) {
        if (use_fp8_dispatch) throw std::runtime_error("ElasticBuffer: pre-quantised dispatch is not built");
        if (!allow_multiple_reduction)
            throw std::runtime_error("ElasticBuffer supports only allow_multiple_reduction=True");
        return rank;
    }
    static int64_t calculate_buffer_size(int num_ranks, int64_t M, int64_t hidden, int64_t num_topk, bool, bool,
                                         bool) {
        return (int64_t)mcep_elastic_buffer_size_hint((int)M, (int)hidden, num_ranks, (int)std::max<int64_t>(num_topk, 1));
    }
    std::tuple<int, int> get_physical_domain_size() const { return {1, num_ranks}; }
    std::tuple<int, int> get_logical_domain_size() const { return {1, num_ranks}; }
    int get_theoretical_num_sms(int, int) const { return 0; }  // the kernels size their own grids
    int64_t timeout_us() const { return gpu_timeout_secs < 0 ? -1 : gpu_timeout_secs * 1000000; }

    // mooncake-ep/src/mooncake_ep_elastic_buffer.cpp:230-245 (the hybrid-mode tensors are accepted and unused)
    std::optional<std::shared_ptr<Event>> dispatch(
        uint64_t x, int x_element_size, uint64_t sf, int num_tokens, int hidden, int num_sf_packs,
        int sf_token_stride, int sf_hidden_stride, uint64_t topk_idx, int num_topk, uint64_t topk_weights,
        uint64_t active_ranks, int num_experts, int num_max_tokens_per_rank, int expert_alignment, int /*num_sms*/,
        bool do_expand, bool async_with_compute_stream, uint64_t compute_stream, bool cached_mode,
        uint64_t psum_rank, uint64_t psum_expert, uint64_t dst_buffer_slot_idx, uint64_t /*token_metadata*/,
        uint64_t /*channel_linked_list*/, uint64_t recv_x, uint64_t recv_x_scales, uint64_t recv_topk_idx,
        uint64_t recv_topk_weights, uint64_t recv_src_metadata) {
        mcep_elastic_dispatch_args a = {};
        a.x = reinterpret_cast<const void*>(x), a.x_element_size = x_element_size;
        a.sf = reinterpret_cast<const void*>(sf);
        a.num_tokens = num_tokens, a.hidden = hidden, a.num_sf_packs = num_sf_packs;
        a.sf_token_stride = sf_token_stride, a.sf_hidden_stride = sf_hidden_stride;
        a.topk_idx = reinterpret_cast<const int64_t*>(topk_idx), a.num_topk = num_topk;
        a.topk_weights = reinterpret_cast<const float*>(topk_weights);
        a.active_ranks = reinterpret_cast<int32_t*>(active_ranks);
        a.num_experts = num_experts, a.num_max_tokens_per_rank = num_max_tokens_per_rank;
        a.expert_alignment = expert_alignment, a.do_expand = do_expand ? 1 : 0;
        a.cached_mode = cached_mode ? 1 : 0, a.timeout_us = timeout_us();
        a.async_with_compute_stream = async_with_compute_stream ? 1 : 0, a.compute_stream = compute_stream;
        a.psum_num_recv_tokens_per_scaleup_rank = reinterpret_cast<int32_t*>(psum_rank);
        a.psum_num_recv_tokens_per_expert = reinterpret_cast<int32_t*>(psum_expert);
        a.dst_buffer_slot_idx = reinterpret_cast<int32_t*>(dst_buffer_slot_idx);
        a.recv_x = reinterpret_cast<void*>(recv_x), a.recv_x_scales = reinterpret_cast<void*>(recv_x_scales);
        a.recv_topk_idx = reinterpret_cast<int64_t*>(recv_topk_idx);
        a.recv_topk_weights = reinterpret_cast<float*>(recv_topk_weights);
        a.recv_src_metadata = reinterpret_cast<int32_t*>(recv_src_metadata);
        a.copied_topk_idx = nullptr;  // the reference's wrapper clones the routing itself
        mcep_event* ev = nullptr;
        check(mcep_elastic_dispatch(h, &a, &ev));
        if (ev) return std::make_shared<Event>(ev);
        return std::nullopt;
    }

    // mooncake-ep/src/mooncake_ep_elastic_buffer.cpp:362-370
    std::optional<std::shared_ptr<Event>> combine(
        uint64_t x, int num_input_tokens, int hidden, uint64_t topk_idx, int num_combined_tokens, int num_topk,
        uint64_t topk_weights, uint64_t psum_rank, uint64_t recv_src_metadata, uint64_t /*token_metadata*/,
        uint64_t /*channel_linked_list*/, uint64_t active_ranks, int num_experts, int num_max_tokens_per_rank,
        bool do_expand, int /*num_sms*/, bool async_with_compute_stream, uint64_t compute_stream,
        uint64_t combined_x) {
        mcep_elastic_combine_args a = {};
        a.x = reinterpret_cast<const void*>(x), a.num_input_tokens = num_input_tokens, a.hidden = hidden;
        a.topk_idx = reinterpret_cast<const int64_t*>(topk_idx);
        a.num_combined_tokens = num_combined_tokens, a.num_topk = num_topk;
        a.topk_weights = reinterpret_cast<const float*>(topk_weights);
        a.psum_num_recv_tokens_per_scaleup_rank = reinterpret_cast<const int32_t*>(psum_rank);
        a.recv_src_metadata = reinterpret_cast<const int32_t*>(recv_src_metadata);
        a.active_ranks = reinterpret_cast<int32_t*>(active_ranks);
        a.num_experts = num_experts, a.num_max_tokens_per_rank = num_max_tokens_per_rank;
        a.do_expand = do_expand ? 1 : 0, a.timeout_us = timeout_us();
        a.async_with_compute_stream = async_with_compute_stream ? 1 : 0, a.compute_stream = compute_stream;
        a.combined_x = reinterpret_cast<void*>(combined_x);
        mcep_event* ev = nullptr;
        check(mcep_elastic_combine(h, &a, &ev));
        if (ev) return std::make_shared<Event>(ev);
        return std::nullopt;
    }
};

}  // namespace

PYBIND11_MODULE(_ep, m) {
    m.def("get_ep_buffer_size_hint", &mcep_get_ep_buffer_size_hint);
    m.attr("MAX_QP_COUNT") = py::int_(MCEP_MAX_QP_COUNT);
    py::class_<Event, std::shared_ptr<Event>>(m, "EventHandle")
        .def(py::init<uint64_t>(), py::arg("stream_ptr") = 0)
        .def("current_stream_wait", &Event::current_stream_wait)
        .def("synchronize", &Event::synchronize);
    py::class_<Buffer>(m, "Buffer")
        .def(py::init<int, int, int64_t, bool>(), py::arg("rank"), py::arg("num_ranks"),
             py::arg("num_ep_buffer_bytes"), py::arg("disable_p2p") = false)
        .def("ibgda_disabled", &Buffer::ibgda_disabled)
        .def("is_roce", &Buffer::is_roce)
        .def("update_local_qpns", &Buffer::update_local_qpns)
        .def("sync_ibgda_peers", &Buffer::sync_ibgda_peers)
        .def("get_mr_info", &Buffer::get_mr_info)
        .def("get_gid", &Buffer::get_gid)
        .def("get_local_qpns", &Buffer::get_local_qpns)
        .def("get_local_lids", &Buffer::get_local_lids)
        .def("p2p_enabled", &Buffer::p2p_enabled)
        .def("use_fast_path", &Buffer::use_fast_path)
        .def("get_ipc_handle", &Buffer::get_ipc_handle)
        .def("sync_nvlink_ipc_handles", &Buffer::sync_nvlink_ipc_handles)
        .def("dispatch", &Buffer::dispatch)
        .def("combine", &Buffer::combine)
        .def("next_recv_x", &Buffer::next_recv_x)
        .def("next_combine_buffer", &Buffer::next_combine_buffer);
    m.def("calculate_elastic_buffer_size", &ElasticBuffer::calculate_buffer_size);
    py::class_<ElasticBuffer>(m, "ElasticBuffer")
        .def(py::init<int, int, int64_t, int64_t, int64_t, int64_t, bool, bool, bool, bool, bool, int, int, int,
                      int>(),
             py::arg("rank"), py::arg("num_ranks"), py::arg("num_buffer_bytes"),
             py::arg("num_max_tokens_per_rank"), py::arg("hidden"), py::arg("num_topk"),
             py::arg("use_fp8_dispatch"), py::arg("deterministic"), py::arg("allow_hybrid_mode"),
             py::arg("allow_multiple_reduction"), py::arg("prefer_overlap_with_compute"), py::arg("sl_idx"),
             py::arg("num_allocated_qps"), py::arg("num_cpu_timeout_secs"), py::arg("num_gpu_timeout_secs"))
        .def_static("calculate_buffer_size", &ElasticBuffer::calculate_buffer_size)
        .def("get_physical_domain_size", &ElasticBuffer::get_physical_domain_size)
        .def("get_logical_domain_size", &ElasticBuffer::get_logical_domain_size)
        .def("get_theoretical_num_sms", &ElasticBuffer::get_theoretical_num_sms)
        .def("ibgda_disabled", &ElasticBuffer::ibgda_disabled)
        .def("use_fast_path", &ElasticBuffer::use_fast_path)
        .def("update_local_qpns", &ElasticBuffer::update_local_qpns)
        .def("is_roce", &ElasticBuffer::is_roce)
        .def("sync_ibgda_peers", &ElasticBuffer::sync_ibgda_peers)
        .def("get_mr_info", &ElasticBuffer::get_mr_info)
        .def("get_gid", &ElasticBuffer::get_gid)
        .def("get_local_qpns", &ElasticBuffer::get_local_qpns)
        .def("get_local_lids", &ElasticBuffer::get_local_lids)
        .def("get_ipc_handle", &ElasticBuffer::get_ipc_handle)
        .def("sync_nvlink_ipc_handles", &ElasticBuffer::sync_nvlink_ipc_handles)
        .def("dispatch", &ElasticBuffer::dispatch)
        .def("combine", &ElasticBuffer::combine);
}
