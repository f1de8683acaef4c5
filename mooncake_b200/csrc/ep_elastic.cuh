// Kernels of the elastic-style calls (flat receive layout, one copy of a token
// per destination rank). The exchange itself is the group dispatch / combine of
// ep_kernels.cu with every rank standing for one "expert"; the kernels here
// prepare its routing input and turn its outputs into the tensors the elastic
// interface returns.
//
// Reference (paths inside the Mooncake tree): the interface is
// mooncake-wheel/mooncake/mooncake_elastic_buffer.py:437-774, the device code
// mooncake-ep/include/elastic/mooncake_ep_elastic_dispatch_official.cuh,
// ..._dispatch_copy_epilogue.cuh, ..._combine_official.cuh and
// ..._combine_reduce_epilogue.cuh.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace mcep {

// A record per row a rank is about to receive, stored by the source in the
// receiver's memory at [source rank][position among the source's rows]:
// [K] int32 expert choices, [K] fp32 weights, int32 token index at the source.
// `record_stride` bytes apart; one set per parity.
struct ElasticRouteParams {
    const int64_t* topk_idx;     // [T][K]
    const float* topk_weights;   // [T][K] or null
    int T, K, E, R, M, rank;
    int64_t* rank_topk;          // [T][K] destination rank at its last listing inside the token, else -1
    int32_t* dst_slot;           // [T][K] rank * M + position among this rank's tokens for that destination, else -1
    int64_t* copied_topk_idx;    // [T][K] copy of topk_idx kept with the handle, or null
    void* const* record_base;    // [R] every rank's record area of this call's parity (null: not mapped)
    int record_stride;
};
cudaError_t launch_elastic_route(const ElasticRouteParams& p, cudaStream_t stream);

struct ElasticEpilogueParams {
    const int64_t* layout_range;  // [R] (begin << 32) | count, as the exchange left it
    const char* records;          // this rank's record area of this call's parity
    int record_stride;
    int R, M, K, L, rank;
    int alignment;                // expert_alignment
    int expand;
    int64_t* recv_topk_idx;       // [n][K] local expert or -1
    float* recv_topk_weights;     // [n][K] or null (expand: scratch, scattered later)
    int32_t* recv_src_metadata;   // [n][K+2]
    int32_t* psum_rank;           // [R] inclusive
    int32_t* psum_expert;         // [L+1] exclusive, aligned counts
    int32_t* psum_start;          // expand: [L+1] copy kept while psum_expert becomes the segment ends
    int32_t* hist;                // [L] scratch, zero between calls
    unsigned* ticket;             // scratch word, zero between calls
    int32_t* status;
};
cudaError_t launch_elastic_epilogue(const ElasticEpilogueParams& p, int num_sms, cudaStream_t stream,
                                    bool pdl);

// Expanded layout: one row per (received token, local expert it chose), experts'
// segments starting at psum_start[e], rows of one expert in receive order.
struct ElasticExpandParams {
    const int64_t* layout_range;  // [R]
    const int64_t* recv_topk_idx; // [n][K]
    const float* flat_weights;    // [n][K] or null
    const void* flat_x;           // [n][row_bytes]
    int R, K, L, row_bytes;
    const int32_t* psum_start;    // [L+1]
    int32_t* psum_expert;         // [L+1]: entries < L become the ends of the segments
    int32_t* recv_src_metadata;   // [n][K+2], columns 2.. written here
    void* recv_x;                 // [rows][row_bytes]
    float* recv_topk_weights;     // [rows] or null
};
cudaError_t launch_elastic_expand_scan(const ElasticExpandParams& p, cudaStream_t stream);
cudaError_t launch_elastic_expand_copy(const ElasticExpandParams& p, int num_sms, cudaStream_t stream);

// Expanded layout, combine side: the rows of one received token are summed into
// one row before they travel (1 row: copied; more: fp32 accumulation in listing
// order, rounded to bf16 once).
struct ElasticLocalReduceParams {
    const int64_t* layout_range;      // [R]
    const int32_t* recv_src_metadata; // [n][K+2]
    const void* x;                    // [rows][H] bf16
    int R, K, H;
    void* y;                          // [n][H] bf16
};
cudaError_t launch_elastic_local_reduce(const ElasticLocalReduceParams& p, int num_sms,
                                        cudaStream_t stream);

// float ones of a given length (the weights of the exchange's reduction)
cudaError_t launch_elastic_fill_ones(float* w, size_t n, cudaStream_t stream);

}  // namespace mcep
