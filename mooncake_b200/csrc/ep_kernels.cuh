// Parameter blocks and launchers of the EP kernels. Host code fills a block,
// the launcher picks the grid and starts the kernel on the given stream.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <string>

namespace mcep {

constexpr int kMaxTopk = 16;       // MCEP_MAX_TOPK
constexpr int kMaxRanks = 64;      // ranks of one group (one NVLink domain)
constexpr int kTileChannels = 512; // one warp pass: 32 lanes x 16 channels
constexpr int kHeaderBytes = 32;   // staged message header (token index + padding)

// Status bits the kernels may raise instead of trapping.
constexpr int kStatusSlotRange = 1;
constexpr int kStatusHardTimeout = 2;
constexpr int kStatusBadSource = 4;

struct LaunchCtx {
    cudaStream_t stream;
    int num_sms;
    bool pdl;  // launch with programmatic stream serialisation
};

// ---- routing layout ---------------------------------------------------------
struct LayoutParams {
    const int64_t* topk_idx;  // [T][K]
    int T, K, E, R;
    int32_t* count;           // [E]
    int32_t* slot;            // [T*K]
    int32_t* rank_count;      // [R] or null
    int32_t* expert_prefix;   // [E] or null
    int32_t* done;            // [E] zeroed here, or null
    unsigned* ticket;         // scratch word, required with rank_count/expert_prefix
    // single-rank groups: the layout already is the receive layout
    int32_t* recv_count;      // [E] or null
    int64_t* layout_range;    // [E] or null
};
cudaError_t launch_layout(const LayoutParams& p, const LaunchCtx& ctx);

// ---- dispatch ---------------------------------------------------------------
struct DispatchSendParams {
    const void* x;              // [T][H] bf16
    const int64_t* topk_idx;    // [T][K]
    const int32_t* slot;        // [T*K] from the layout kernel
    const int32_t* count;       // [E]
    int32_t* done;              // [E] completion counters (zero on entry)
    const int32_t* active_ranks;
    void* const* peer_base;     // [R] base of every rank's symmetric buffer
    int T, K, E, R, M, H, rank;
    int use_fp8;
    int fused;                  // count the slots here (slot/count unused) - small batches
    size_t stage_off;           // dispatch staging of this call's parity
    size_t flag_off;            // dispatch flags of this call's parity
    size_t msg_stride;
    uint32_t seq;
    int32_t* status;
    // direct mode (single rank): write the packed outputs, no staging, no flags
    int direct;
    void* recv_x;
    float* recv_scales;
    int32_t* recv_src_info;
    int32_t* recv_count;        // direct + fused: [E]
    int64_t* layout_range;      // direct + fused: [E]
};
// whether the send kernel may count the slots itself for this problem size
bool dispatch_send_can_fuse_layout(int T, int K, int H, int num_sms);
cudaError_t launch_dispatch_send(const DispatchSendParams& p, const LaunchCtx& ctx);

// How a receive kernel waits for flags (see resolve_flag in ep_kernels.cu).
struct WaitSpec {
    const uint64_t* flags;      // local flags of this call's parity and direction
    uint64_t* resolved;         // scratch, one word per flag: the verdict for this call
    int32_t* active_ranks;
    uint32_t seq;
    int64_t timeout_ns;         // < 0: only the hard bound applies
    int64_t hard_timeout_ns;
    int32_t* status;
};

struct DispatchRecvParams {
    WaitSpec w;                 // flags indexed expert * R + source
    const char* stage;          // local dispatch staging of this parity
    int L, R, M, H;
    int use_fp8;
    int expected_rows;          // host's estimate of the rows this rank receives (grid sizing)
    size_t msg_stride;
    void* recv_x;
    float* recv_scales;
    int32_t* recv_src_info;
    int32_t* recv_count;        // [L]
    int64_t* layout_range;      // [L][R]
};
cudaError_t launch_dispatch_recv(const DispatchRecvParams& p, const LaunchCtx& ctx);

// ---- combine ----------------------------------------------------------------
struct CombineSendParams {
    const void* x;              // [L][R*M][H] bf16
    const int32_t* src_info;    // [L][R*M]
    const int64_t* layout_range;// [L][R]
    const int32_t* active_ranks;
    void* const* peer_base;
    int32_t* done;              // [L*R] completion counters (zero on entry, zero on exit)
    int L, R, M, H, rank;
    size_t stage_off;           // combine staging of this parity
    size_t flag_off;            // combine flags of this parity
    uint32_t seq;
    int32_t* status;
};
cudaError_t launch_combine_send(const CombineSendParams& p, const LaunchCtx& ctx);

// Single rank: (token, k) -> packed row, inverted from the handle.
struct CombineInvertParams {
    const int32_t* src_info;    // [L][R*M]
    const int64_t* layout_range;// [L][R]
    const int64_t* topk_idx;    // [T][K]
    int L, R, M, T, K, rank;
    int32_t* rowmap;            // scratch [T*K]
    int32_t* status;
};
cudaError_t launch_combine_invert(const CombineInvertParams& p, const LaunchCtx& ctx);

struct CombineReduceParams {
    const int64_t* topk_idx;    // [T][K]
    const float* topk_weights;  // [T][K]
    const int32_t* active_ranks;
    int T, K, E, L, M, H;
    // staged: waits for each needed expert's flag (w.flags indexed by global
    // expert), then reads rows at stage + (expert * M + token) * 2H
    WaitSpec w;
    const char* stage;
    // direct: rows at x + (expert * R*M + rowmap[t*K+k]) * 2H (single rank)
    int direct;
    const void* x;
    const int32_t* rowmap;
    int RM;
    // direct + search: no rowmap; rows are looked up in the handle by the kernel
    int search;
    const int32_t* src_info;
    const int64_t* layout_range;
    void* combined_x;           // [T][H] bf16
};
cudaError_t launch_combine_reduce(const CombineReduceParams& p, const LaunchCtx& ctx);

// Both phases of a call in one launch (small batches in a group, no hook).
bool call_can_be_one_kernel(int T, int K, int H, int num_sms);
cudaError_t launch_dispatch_one_kernel(const DispatchSendParams& sp, const DispatchRecvParams& rp,
                                       const LaunchCtx& ctx);
cudaError_t launch_combine_one_kernel(const CombineSendParams& sp, const CombineReduceParams& rp,
                                      const LaunchCtx& ctx);

uint64_t kernel_launch_count();
// Per-kernel device times: switch on, run, then drain "name launches total_ms" lines.
void set_kernel_timing(bool on);
std::string drain_kernel_times();

}  // namespace mcep
