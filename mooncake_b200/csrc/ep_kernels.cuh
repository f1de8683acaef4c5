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
constexpr int kMaxExperts = 4096;  // MCEP_MAX_EXPERTS
constexpr int kTileChannels = 512; // one warp pass: 32 lanes x 16 channels
constexpr int kMetaHeaderBytes = 16;  // per-row side message: token index + padding, then scales

// Status bits the kernels may raise instead of trapping.
constexpr int kStatusSlotRange = 1;
constexpr int kStatusHardTimeout = 2;
constexpr int kStatusBadSource = 4;
constexpr int kStatusNoPeer = 8;  // a rank marked active has no mapped buffer

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
    unsigned* ticket;         // scratch word, required with rank_count/expert_prefix
    // single-rank groups: the layout already is the receive layout
    int32_t* recv_count;      // [E] or null
    int64_t* layout_range;    // [E] or null
    // optional scratch for the two-pass (chunked) variant: per-chunk histograms
    int32_t* chunk_hist;      // [chunk_hist_entries] or null
    size_t chunk_hist_entries;
};
cudaError_t launch_layout(const LayoutParams& p, const LaunchCtx& ctx);

// ---- single rank: packed outputs written directly ------------------------------
struct DirectDispatchParams {
    const void* x;              // [T][H] bf16
    const int64_t* topk_idx;    // [T][K]
    const int32_t* slot;        // [T*K] from the layout kernel (not fused)
    const int32_t* count;       // [E]   from the layout kernel (not fused)
    int T, K, E, M, H;
    int use_fp8;
    int fused;                  // count the slots here (slot/count unused) - small batches
    int32_t* status;
    void* recv_x;
    float* recv_scales;
    int32_t* recv_src_info;
    int32_t* recv_count;        // fused: [E]
    int64_t* layout_range;      // fused: [E]
    int32_t* rowmap;            // [T*K] row of (token, k) inside its expert, kept for combine
};
// whether a send kernel may count the slots itself for this problem size
bool can_fuse_layout(int T, int K, int E, int num_sms);
cudaError_t launch_direct_dispatch(const DirectDispatchParams& p, const LaunchCtx& ctx);

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

struct DirectCombineParams {
    const int64_t* topk_idx;    // [T][K]
    const float* topk_weights;  // [T][K]
    const int32_t* active_ranks;
    int T, K, E, M, H;
    const void* x;              // rows at x + (expert * M + rowmap[t*K+k]) * 2H
    const int32_t* rowmap;
    // search: no rowmap; rows are looked up in the handle by the kernel
    int search;
    const int32_t* src_info;
    const int64_t* layout_range;
    void* combined_x;           // [T][H] bf16
};
cudaError_t launch_direct_combine(const DirectCombineParams& p, const LaunchCtx& ctx);

// ---- groups: words exchanged through symmetric memory -----------------------------
// All words are 64-bit: (sequence number of the call << 32) | value, value >= 1.
// A word that does not carry the current sequence number has not arrived.
struct Words {
    // byte offsets inside every rank's symmetric allocation, for this call's parity
    size_t cnt_off;    // at the owner of an expert: [R src][L] tokens src sends to local expert
    size_t beg_off;    // at a sender: [E] first row of its segment in expert e, written by e's owner
    size_t dflag_off;  // at a receiver: [R src] all of src's dispatch rows have landed
    size_t cflag_off;  // at a token owner: [R owner] owner's expert outputs can be read
};

struct WaitCfg {
    int32_t* active_ranks;     // read and written (timeout -> 0)
    int64_t timeout_ns;        // < 0: only the hard bound applies
    int64_t hard_timeout_ns;
    int32_t* status;
};

// Dispatch in a group. Block 0 is the control block: it publishes this rank's
// per-expert counts to the experts' owners, collects the counts all sources
// announce for its own experts, fixes the receive layout and answers every
// source with the first row of its segment. The other blocks send token rows
// straight to their final place in the owners' packed receive area.
struct GroupDispatchParams {
    const void* x;              // [T][H] bf16
    const int64_t* topk_idx;    // [T][K]
    const int32_t* slot;        // [T*K] from the layout kernel (not fused)
    const int32_t* count;       // [E]   from the layout kernel (not fused)
    void* const* peer_base;     // [R] base of every rank's symmetric buffer
    char* local_base;           // this rank's
    int T, K, E, R, M, H, rank;
    int use_fp8;
    int fused;
    Words w;
    size_t rx_off;              // packed receive rows [L][R*M][row_bytes] of this parity
    size_t meta_off;            // side messages [L][R*M][meta_stride] of this parity
    int row_bytes, meta_stride;
    uint32_t seq;
    const uint32_t* seq_ptr;    // graph mode: the call's sequence number lives in device memory (else null)
    WaitCfg wait;
    // scratch in the local workspace (per parity)
    uint64_t* res_cnt;          // [L*R] the control block's verdict per (expert, source)
    uint64_t* res_dflag;        // [R] verdict words of the payload flags
    unsigned* ticket;           // sender blocks that have finished
    int32_t* rowmap;            // [T*K] row of (token, k) at its expert's owner, kept for combine
    // outputs (caller's tensors)
    void* recv_x;               // == local_base + rx_off when the caller took the in-place tensor
    float* recv_scales;
    int32_t* recv_src_info;
    int32_t* recv_count;        // [L]
    int64_t* layout_range;      // [L][R]
    int copy_rows;              // recv_x is a tensor of the caller's: copy the rows out
};
bool group_call_can_be_one_kernel(int T, int K, int E, int num_sms);
// one launch: control + send + receive duties
cudaError_t launch_group_dispatch(const GroupDispatchParams& p, const LaunchCtx& ctx);
// two launches (hook mode, large batches, caller-owned recv_x)
cudaError_t launch_group_dispatch_send(const GroupDispatchParams& p, const LaunchCtx& ctx);
cudaError_t launch_group_dispatch_recv(const GroupDispatchParams& p, const LaunchCtx& ctx);

// Combine in a group: expert outputs are made readable in symmetric memory
// (copied there, or written there by the caller: zero copy), every peer is told
// so with one word, and token owners read their rows straight from the experts'
// owners and reduce them.
struct GroupCombineParams {
    const void* x;              // [L][R*M][H] bf16 expert outputs (ignored with zero_copy)
    const int64_t* layout_range;// [L][R] from the handle
    const int64_t* topk_idx;    // [T][K]
    const float* topk_weights;  // [T][K]
    const int32_t* rowmap;      // [T*K] left by the dispatch call of this handle
    void* const* peer_base;
    char* local_base;
    int T, K, E, R, M, H, rank;
    int zero_copy;
    Words w;
    size_t cin_off;             // combine input [L][R*M][H] bf16 of this parity
    uint32_t seq;
    const uint32_t* seq_ptr;    // graph mode (see GroupDispatchParams)
    WaitCfg wait;
    uint64_t* res_cflag;        // [R]
    unsigned* ticket;
    void* combined_x;           // [T][H] bf16
};
cudaError_t launch_group_combine(const GroupCombineParams& p, const LaunchCtx& ctx);
cudaError_t launch_group_combine_publish(const GroupCombineParams& p, const LaunchCtx& ctx);
cudaError_t launch_group_combine_reduce(const GroupCombineParams& p, const LaunchCtx& ctx);

// In-process groups (several logical ranks on one GPU, tests): the send phase
// (phases = 1) or the whole call (phases = 3) of `n` ranks as ONE cooperative
// launch, because kernels that wait for one another must not be separate
// launches on one GPU. `dev_params` is device memory for `n` parameter blocks.
// All ranks must agree on payload type, hidden size and `fused`.
cudaError_t launch_group_dispatch_multi(const GroupDispatchParams* params, int n,
                                        GroupDispatchParams* dev_params, int phases,
                                        const LaunchCtx& ctx);
cudaError_t launch_group_combine_multi(const GroupCombineParams* params, int n,
                                       GroupCombineParams* dev_params, const LaunchCtx& ctx);

// A barrier of the group on the device: every rank writes one word to every
// active peer and waits for theirs; the ranks leave within about one NVLink
// latency of each other. `bar_off` = [R] u64 words in symmetric memory,
// `epoch` = the number of this barrier (all ranks count alike).
struct BarrierParams {
    void* const* peer_base;
    char* local_base;
    const int32_t* active_ranks;  // [R] or null (all active)
    size_t bar_off;
    int rank, R;
    uint32_t epoch;
    int64_t hard_timeout_ns;
    int32_t* status;
};
cudaError_t launch_barrier(const BarrierParams& p, const LaunchCtx& ctx);

// Graph mode: after the last kernel of a call, the word that holds the next
// sequence number of that call's parity moves on by two.
cudaError_t launch_advance_seq(uint32_t* word, const LaunchCtx& ctx);

uint64_t kernel_launch_count();
// Brackets a launch made outside ep_kernels.cu so that it is counted - and, when
// per-kernel timing is on, timed - like the launches made there.
class LaunchScope {
public:
    LaunchScope(const char* name, cudaStream_t stream);
    cudaError_t done(cudaError_t err);  // pass cudaGetLastError() of the launch

private:
    const char* name_;
    cudaStream_t stream_;
    cudaEvent_t a_ = nullptr, b_ = nullptr;
};
// Per-kernel device times: switch on, run, then drain "name launches total_ms" lines.
void set_kernel_timing(bool on);
std::string drain_kernel_times();

}  // namespace mcep
