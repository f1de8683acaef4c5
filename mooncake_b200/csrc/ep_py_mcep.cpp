// A pybind11 binding of the C ABI (include/mcep.h) with the surface of the
// reference's compiled module `mooncake._ep` for the legacy Buffer
// (mooncake-ep/src/ep_py.cpp:14-46): `Buffer`, `EventHandle`,
// `get_ep_buffer_size_hint`, `MAX_QP_COUNT`. It is what a maintainer who wants
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
}
