// Host harness around the reference's own dispatch / combine kernels.
//
// TEST INFRASTRUCTURE ONLY - never shipped, never on the product path. It is
// compiled by oracle/build.py together with the reference's translation unit
// mooncake-ep/src/mooncake_ep_kernel.cu (taken from a Mooncake checkout where
// it lies) into oracle/_ref/libmooncake_ep_ref.so, and lets the tests run the
// reference kernels on the same inputs as the kernels of this repository.
//
// It only does what the reference's host class does around the launch
// (mooncake-ep/src/mooncake_ep_buffer.cpp:212-218, 290-302, 426-437): carve the
// symmetric buffer into the two signal / data halves
// (mooncake-ep/include/mooncake_ep_buffer.h:42-61), pick the current half, pass
// the other half's receive signals as the area to clean, and call the launcher
// declared in mooncake-ep/include/mooncake_ep_api.cuh:7-45 with null RDMA tables.
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <exception>

#include <mooncake_ep_api.cuh>

namespace {

struct Half {
    int *send_signal, *recv_signal;
    void *send_data, *recv_data;
};

Half carve(void* base, int half, int M, int H, int E) {
    const size_t sig = (size_t)E * sizeof(int);
    const size_t data = (size_t)E * M * (2 * 16 + (size_t)H * 2);
    char* b = static_cast<char*>(base) + (size_t)half * (2 * sig + 2 * data);
    return Half{reinterpret_cast<int*>(b), reinterpret_cast<int*>(b + sig),
                reinterpret_cast<void*>(b + 2 * sig), reinterpret_cast<void*>(b + 2 * sig + data)};
}

char g_err[512];

}  // namespace

extern "C" const char* ref_last_error() { return g_err; }

extern "C" int ref_dispatch(void* base, const int32_t* available_dev, void* const* peer_ptrs_dev,
                            void* workspace, int half, const void* x, const int64_t* topk_idx,
                            int32_t* active_ranks, void* recv_x, float* recv_scales,
                            int* recv_src_info, int64_t* recv_layout_range, int* recv_count, int T,
                            int H, int M, int K, int E, int rank, int R, int use_fp8,
                            int64_t timeout_ticks, int phases, uint64_t stream) {
    try {
        Half cur = carve(base, half, M, H, E), nxt = carve(base, half ^ 1, M, H, E);
        mooncake::dispatch(recv_x, recv_scales, recv_src_info, recv_layout_range, recv_count,
                           active_ranks, base, cur.send_signal, cur.recv_signal, cur.send_data,
                           cur.recv_data, nullptr, nullptr, nullptr, nullptr, nullptr, available_dev,
                           peer_ptrs_dev, x, topk_idx, nxt.recv_signal, T, H, M, K, E, rank, R,
                           use_fp8 != 0, workspace, reinterpret_cast<cudaStream_t>(stream),
                           timeout_ticks, phases, 1);
    } catch (const std::exception& e) {
        snprintf(g_err, sizeof(g_err), "%s", e.what());
        return -1;
    }
    return 0;
}

extern "C" int ref_combine(void* base, const int32_t* available_dev, void* const* peer_ptrs_dev,
                           void* workspace, int half, const void* x, const int64_t* topk_idx,
                           const float* topk_weights, const int* src_info,
                           const int64_t* layout_range, int32_t* active_ranks, void* combined_x,
                           int T, int H, int M, int K, int E, int rank, int R,
                           int64_t timeout_ticks, int phases, uint64_t stream) {
    try {
        Half cur = carve(base, half, M, H, E), nxt = carve(base, half ^ 1, M, H, E);
        mooncake::combine(combined_x, active_ranks, base, cur.send_signal, cur.recv_signal,
                          cur.send_data, cur.recv_data, nullptr, nullptr, nullptr, nullptr, nullptr,
                          available_dev, peer_ptrs_dev, x, topk_idx, topk_weights, src_info,
                          layout_range, nxt.recv_signal, T, H, M, K, E, rank, R, workspace,
                          reinterpret_cast<cudaStream_t>(stream), timeout_ticks, phases, false, 1);
    } catch (const std::exception& e) {
        snprintf(g_err, sizeof(g_err), "%s", e.what());
        return -1;
    }
    return 0;
}
