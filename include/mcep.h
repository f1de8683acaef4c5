/*
 * mcep - B200-native MoE expert-parallel dispatch / combine.
 *
 * C ABI of libmcep.so. Plain pointers and sizes only; every pointer that names
 * tensor data is a CUDA device pointer owned by the caller, every `stream`
 * argument is a `cudaStream_t` passed as an integer (0 = the default stream).
 *
 * The entry points are the ones a binding of Mooncake EP's `Buffer` needs; each
 * comment names the reference interface it replaces (paths inside the Mooncake
 * source tree).
 *
 * Errors: functions return MCEP_OK (0) or a negative code; `mcep_last_error()`
 * then holds a message for the calling thread. Device-side anomalies never
 * trap: they are recorded in a status word (`mcep_buffer_status`).
 */
#ifndef MCEP_H_
#define MCEP_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MCEP_OK 0
#define MCEP_ERR_INVALID (-1)   /* argument check failed (reference: EP_HOST_ASSERT) */
#define MCEP_ERR_CUDA (-2)      /* a CUDA runtime call failed (reference: CUDA_CHECK) */
#define MCEP_ERR_STATE (-3)     /* buffer not connected / peers not accessible */

/* mooncake-ep/include/mooncake_ep_configs.cuh:5 (MAX_QP_COUNT), re-exported by
 * the binding because the reference's Python bootstrap reads it. */
#define MCEP_MAX_QP_COUNT 256
/* Largest top-k per token. The reference allows 11
 * (mooncake-ep/src/mooncake_ep_kernel.cu:487,773). */
#define MCEP_MAX_TOPK 16
/* Largest number of experts (flag slots reserved per direction). */
#define MCEP_MAX_EXPERTS 4096
/* An exported memory handle is a 64-byte cudaIpcMemHandle_t carried as 16
 * int32, as in mooncake-transfer-engine/src/transport/device/
 * p2p_device_transport.cpp:483-488. */
#define MCEP_IPC_HANDLE_INT32S 16
/* With MC_USE_NVLINK_IPC=0 in the environment, and where every visible device
 * supports fabric handles, the buffer is a cuMemCreate allocation and the
 * exported handle is a CUmemFabricHandle followed by the allocation's size:
 * 72 bytes carried as 18 int32 (mooncake-transfer-engine/src/transport/device/
 * p2p_device_transport.cpp:40-75, 271-386). Elsewhere the request is ignored
 * and cudaMalloc + CUDA IPC is used, as the reference does. All ranks of a
 * group must run with the same setting. */
#define MCEP_FABRIC_HANDLE_INT32S 18

typedef struct mcep_buffer mcep_buffer;
typedef struct mcep_event mcep_event;
typedef struct mcep_hook mcep_hook;

/* Message of the last failure on this thread ("" when none). */
const char* mcep_last_error(void);

/* Number of kernels this library has launched in this process (all buffers). */
uint64_t mcep_kernel_launch_count(void);

/* Measurement aid: while on, every kernel launch is bracketed by CUDA events on
 * its own stream (kernels then run one after the other, never overlapped).
 * `mcep_drain_kernel_times` waits for the recorded launches and writes one line
 * per kernel, "name launches total_ms\n", NUL-terminated, then forgets them. */
int mcep_set_kernel_timing(int on);
int mcep_drain_kernel_times(char* out, size_t capacity);

/*
 * Bytes of symmetric memory a Buffer needs:
 *   4*E*4 + 4*E*M*(32 + 2*H)
 * Replaces mooncake::get_ep_buffer_size_hint / BufferPair
 * (mooncake-ep/include/mooncake_ep_buffer.h:29-63,197-203); same value.
 */
uint64_t mcep_get_ep_buffer_size_hint(int num_max_dispatch_tokens_per_rank,
                                      int hidden, int num_ranks,
                                      int num_experts);

/* ---- buffer life cycle ---------------------------------------------------
 * Replaces MooncakeEpBuffer::MooncakeEpBuffer / ~MooncakeEpBuffer
 * (mooncake-ep/src/mooncake_ep_buffer.cpp:74-191): allocates and zeroes the
 * symmetric buffer and a 32 MiB workspace on the current device and creates a
 * high-priority non-blocking communication stream. */
int mcep_buffer_create(int rank, int num_ranks, int64_t num_ep_buffer_bytes,
                       int disable_p2p, mcep_buffer** out);
int mcep_buffer_destroy(mcep_buffer* buf);

/* mooncake-ep/include/mooncake_ep_buffer.h:135-151. There is no RDMA route in
 * this library: ibgda_disabled() is always 1 and is_roce() always 0. */
int mcep_buffer_ibgda_disabled(const mcep_buffer* buf);
int mcep_buffer_p2p_enabled(const mcep_buffer* buf);
int mcep_buffer_is_roce(const mcep_buffer* buf);
/* 1 when every active rank's memory is mapped (single rank: always 1);
 * mooncake-ep/include/mooncake_ep_buffer.h:143, `use_fast_path`. */
int mcep_buffer_use_fast_path(const mcep_buffer* buf);
/* 1 when the buffer was allocated in the fabric-handle mode (MC_USE_NVLINK_IPC=0
 * and driver support, see MCEP_FABRIC_HANDLE_INT32S), 0 for cudaMalloc + CUDA IPC.
 * mooncake-transfer-engine/src/transport/device/p2p_device_transport.cpp:40-60. */
int mcep_buffer_uses_fabric_handles(const mcep_buffer* buf);

/* MooncakeEpBuffer::get_ipc_handle (mooncake-ep/src/mooncake_ep_buffer.cpp:518-521):
 * writes MCEP_IPC_HANDLE_INT32S int32 to `out` (capacity in int32; in fabric mode
 * MCEP_FABRIC_HANDLE_INT32S, so pass room for 18), `*n_written` = 0 when P2P is
 * disabled. */
int mcep_buffer_get_ipc_handle(mcep_buffer* buf, int32_t* out, int capacity,
                               int* n_written);

/* MooncakeEpBuffer::sync_nvlink_ipc_handles
 * (mooncake-ep/src/mooncake_ep_buffer.cpp:523-529) and
 * P2pDeviceTransportImpl::importPeerHandles
 * (mooncake-transfer-engine/src/transport/device/p2p_device_transport.cpp:491-715). `handles` is [num_ranks][n_per_handle]
 * int32, `active_ranks_mask` is [num_ranks] (0 = do not map that rank). A later
 * call replaces the earlier mapping (membership refresh). */
int mcep_buffer_sync_nvlink_ipc_handles(mcep_buffer* buf,
                                        const int32_t* handles,
                                        int n_per_handle,
                                        const int32_t* active_ranks_mask);

/* Membership refresh. The words ranks exchange carry the number of the call
 * they belong to, so all ranks of a group must have made the same number of
 * dispatch and of combine calls. get_ipc_handle leaves this rank's two call
 * counters in its symmetric memory; sync_nvlink_ipc_handles reads those of
 * every rank it maps and continues from the largest. A rank that sat out some
 * calls (masked out) or was re-created from scratch is therefore back in step
 * after every rank has run the two calls (Buffer.update_ep_member in the
 * reference's wrapper, mooncake-wheel/mooncake/mooncake_ep_buffer.py:306-307),
 * with nothing in flight. Handles of dispatch calls made before a counter
 * jumped can no longer be combined. */

/* In-process groups (several logical ranks in one process, e.g. tests that run
 * the ranks one after the other on one GPU): hand the peers' base pointers over
 * directly instead of through IPC handles (local_base plays the part of
 * get_ipc_handle, set_peer_bases that of sync_nvlink_ipc_handles). No
 * counterpart in the reference. */
int mcep_buffer_local_base(mcep_buffer* buf, void** base);
int mcep_buffer_set_peer_bases(mcep_buffer* buf, void* const* bases,
                               const int32_t* available);
/* In a group the kernels of different ranks wait for one another (an expert's
 * owner answers every source), which is fine on GPUs of their own but not as
 * separate launches on ONE GPU: nothing would make them run at the same time.
 * With option "defer_launch" = 1 a buffer's mcep_dispatch / mcep_combine call
 * prepares everything and launches nothing; mcep_launch_deferred then starts
 * what the listed buffers have prepared - all dispatch or all combine calls of
 * the same kind, same stream - as ONE cooperative launch that carries every
 * rank. (A combine call in hook mode needs no deferral: its first phase waits
 * for nobody.) Tests and single-GPU experiments only; no counterpart in the
 * reference. */
int mcep_launch_deferred(mcep_buffer* const* bufs, int n);

/* Options (no counterpart in the reference):
 *   "force_staged"    1 = a single rank also goes through symmetric memory and
 *                     the word exchange, as multi-rank groups do (default 0)
 *   "hard_timeout_ms" upper bound applied to every device-side wait, also when
 *                     timeout_us is -1 (default 10000)
 *   "pdl"             1 = kernels of one call are chained with programmatic
 *                     dependent launch (default 1)
 *   "fuse_layout"     1 = small batches count their routing layout inside the
 *                     send kernel instead of in a kernel of its own (default 1)
 *   "one_kernel"      1 = small batches in a group run the send and the receive
 *                     phase of a call in one launch (default 1)
 *   "defer_launch"    1 = in-process groups: prepare calls, launch them together
 *                     with mcep_launch_deferred (default 0)
 *   "graph_mode"      1 = calls of a group can be captured in a CUDA graph and
 *                     replayed (default 0). The words ranks exchange carry the
 *                     call's sequence number; by default it is a launch
 *                     argument, which a replay would repeat. In graph mode the
 *                     next number of each parity lives in device memory: the
 *                     kernels read it, and a one-thread kernel after the call's
 *                     last launch (in hook mode: launched by the hook) moves it
 *                     on. Costs one tiny launch per call. A captured graph must
 *                     hold an even number of dispatch calls and of combine calls
 *                     (whole layers of two micro-batches, or an even number of
 *                     layers), so that every replay starts on the parity it was
 *                     captured on; every rank of the group must replay alike.
 *                     Set it with nothing in flight, on every rank.
 * An unknown name is an error. */
int mcep_buffer_set_option(mcep_buffer* buf, const char* name, int64_t value);

/* Copies up to `n` int32 status words (0 = clean). Word 0: bit mask of
 * anomalies (1 row or slot out of range, 2 hard wait bound hit, 4 bad source
 * index, 8 a rank marked active has no mapped buffer and was left alone).
 * No counterpart in the reference, whose kernels trap instead. */
int mcep_buffer_status(mcep_buffer* buf, int32_t* out, int n);

/* A barrier of the group on the device, queued on `stream`: every rank writes
 * one word into every active peer's symmetric memory and waits for theirs, so
 * the ranks' streams leave it within about one NVLink latency of each other
 * (a collective of a library completes at different times on different ranks).
 * Every participating rank must call it the same number of times; ranks that
 * `active_ranks` (device, [num_ranks], may be NULL) marks 0 are not waited for
 * and must not call. The wait is bounded by "hard_timeout_ms" (status bit 2).
 * The legacy Buffer of the reference has no barrier; its elastic buffer has one
 * (mooncake-wheel/mooncake/mooncake_elastic_buffer.py:417-423). */
int mcep_buffer_barrier(mcep_buffer* buf, const int32_t* active_ranks, uint64_t stream);

/* Dispatch and combine calls this buffer has made (or adopted at a membership
 * refresh); in graph mode read from the device, after waiting for it to go
 * idle, so replayed graphs are counted. No counterpart in the reference. */
int mcep_buffer_call_counts(mcep_buffer* buf, uint32_t* dispatch_calls,
                            uint32_t* combine_calls);

/* Where the NEXT dispatch call of this buffer lands its rows: the packed
 * receive tensor [E/R][R*M][H] (e4m3 bytes or bf16) inside symmetric memory,
 * for the given shape. A binding that passes this pointer as
 * `packed_recv_x` gets the rows in place - peers store them there directly -
 * and the call moves no payload on the receiving side; the memory is reused by
 * the dispatch call after the next one. With any other pointer the rows are
 * copied out into it, as the reference does
 * (mooncake-ep/src/mooncake_ep_kernel.cu:442-466). `*out` is NULL for a single
 * rank (it writes the caller's tensor directly) or when the buffer is too small
 * for the shape (the dispatch call then reports it). */
int mcep_buffer_next_recv_x(mcep_buffer* buf, int num_max_dispatch_tokens_per_rank,
                            int hidden, int num_experts, int use_fp8, void** out,
                            size_t* bytes);

/* Zero-copy combine: the tensor [E/R][R*M][H] bf16 inside symmetric memory that
 * the NEXT combine call reads when it is given `zero_copy = 1`; the caller's
 * expert kernels write their outputs there instead of into a tensor of their
 * own (docs/source/design/mooncake-ep.md:165-167 in the Mooncake tree; the
 * reference's wrapper rejects it today, mooncake-wheel/mooncake/
 * mooncake_ep_buffer.py:551,680). `*out` is NULL for a single rank, whose
 * combine reads the caller's tensor directly either way. */
int mcep_buffer_next_combine_buffer(mcep_buffer* buf, int num_max_dispatch_tokens_per_rank,
                                    int hidden, int num_experts, void** out,
                                    size_t* bytes);

/* ---- dispatch --------------------------------------------------------------
 * Replaces MooncakeEpBuffer::dispatch
 * (mooncake-ep/include/mooncake_ep_buffer.h:116-124,
 *  mooncake-ep/src/mooncake_ep_buffer.cpp:193-339); argument meaning and
 * checks as there. Outputs (caller-allocated):
 *   packed_recv_x            [E/R][R*M][H]   e4m3 bytes (use_fp8) or bf16
 *   packed_recv_x_scales     [E/R][H/128][R*M] fp32 storage (use_fp8 only)
 *   packed_recv_count        [E/R] int32
 *   packed_recv_src_info     [E/R][R*M] int32  token index at its source rank
 *   packed_recv_layout_range [E/R][R] int64    (begin << 32) | count, 0 if empty
 * Rows are ordered by source rank, then by token index. `active_ranks` [R]
 * int32 is read AND written (a source that misses `timeout_us` is set to 0).
 * In a group the owner of an expert fixes the layout from the counts all sources
 * announce and tells each source where its rows go; if a source goes silent
 * after announcing its counts, its rows stay in the layout with unspecified
 * contents and the source is marked inactive.
 */
typedef struct mcep_dispatch_args {
    const void* x;              /* [num_tokens][hidden] bf16 */
    const int64_t* topk_idx;    /* [num_tokens][num_topk], -1 = no expert */
    int32_t* active_ranks;      /* [num_ranks] */
    int32_t num_tokens;
    int32_t hidden;
    int32_t num_topk;
    int32_t num_max_dispatch_tokens_per_rank;
    int32_t num_experts;
    int32_t use_fp8;
    int64_t timeout_us;         /* -1: bounded only by "hard_timeout_ms" */
    void* packed_recv_x;
    float* packed_recv_x_scales;
    int32_t* packed_recv_count;
    int32_t* packed_recv_src_info;
    int64_t* packed_recv_layout_range;
    int32_t async_finish;       /* run on the communication stream, return an event */
    int32_t return_recv_hook;   /* send now on `compute_stream`, receive in the hook */
    uint64_t compute_stream;
} mcep_dispatch_args;

/* `*out_event` / `*out_hook` are set to NULL when the mode returns none
 * (the reference returns std::nullopt there). */
int mcep_dispatch(mcep_buffer* buf, const mcep_dispatch_args* args,
                  mcep_event** out_event, mcep_hook** out_hook);

/* ---- combine ---------------------------------------------------------------
 * Replaces MooncakeEpBuffer::combine
 * (mooncake-ep/include/mooncake_ep_buffer.h:126-133,
 *  mooncake-ep/src/mooncake_ep_buffer.cpp:341-474).
 *   x            [E/R][R*M][H] bf16 expert outputs in the packed layout
 *   combined_x   [num_combined_tokens][H] bf16
 * combined[t] = bf16( sum over k in order, fp32 FMA, of w[t][k] * x_row ),
 * skipping topk_idx < 0 and experts whose owner rank is inactive.
 * In a group, `src_info` must be the tensor a dispatch call of this buffer
 * filled, and that call must be one of the buffer's last two dispatch calls
 * (the rows' positions at the experts' owners are kept from then); the same
 * handle may be combined more than once. With `zero_copy` the expert outputs
 * are read from mcep_buffer_next_combine_buffer's tensor and `x` is ignored.
 */
typedef struct mcep_combine_args {
    const void* x;
    const int64_t* topk_idx;
    const float* topk_weights;
    const int32_t* src_info;
    const int64_t* layout_range;
    int32_t* active_ranks;
    int32_t num_local_experts;
    int32_t num_combined_tokens;
    int32_t hidden;
    int32_t num_topk;
    int32_t num_max_dispatch_tokens_per_rank;
    int32_t num_experts;
    int64_t timeout_us;
    int32_t zero_copy;          /* read mcep_buffer_next_combine_buffer's tensor instead of x */
    void* combined_x;
    int32_t async_finish;
    int32_t return_recv_hook;
    uint64_t compute_stream;
} mcep_combine_args;

int mcep_combine(mcep_buffer* buf, const mcep_combine_args* args,
                 mcep_event** out_event, mcep_hook** out_hook);

/* ---- elastic-style calls -----------------------------------------------------
 * The interface of the reference's ElasticBuffer for one NVLink domain
 * (mooncake-wheel/mooncake/mooncake_elastic_buffer.py:437-774; host side
 * mooncake-ep/src/mooncake_ep_elastic_buffer.cpp:230-426; device side
 * mooncake-ep/include/elastic/mooncake_ep_elastic_dispatch_official.cuh,
 * ..._dispatch_copy_epilogue.cuh, ..._combine_official.cuh,
 * ..._combine_reduce_epilogue.cuh), on the exchange of mcep_dispatch /
 * mcep_combine with every rank standing for one "expert":
 *   - a token travels ONCE to every rank that owns at least one of its experts
 *     (the reference deduplicates the same way, dispatch_official.cuh:113-117);
 *   - the receiver gets the rows flat, ordered by source rank, then by token
 *     index (the order of the reference's `deterministic` mode);
 *   - combine sends ONE row per received token back and the token's owner adds
 *     the rows of the ranks it reached, in the order of each rank's last listing
 *     in the token's top-k list, unweighted.
 * Outputs of dispatch (caller-allocated, capacities as the reference allocates
 * them: n_cap = num_ranks * num_max_tokens_per_rank rows, times num_topk for
 * recv_x / recv_topk_weights when do_expand):
 *   psum_num_recv_tokens_per_scaleup_rank [R] int32  inclusive sum of the rows each source sent
 *   psum_num_recv_tokens_per_expert [L+1] int32  exclusive sum of the per-expert
 *       (token, expert) hits, each rounded up to expert_alignment; with
 *       do_expand entries < L end up as the END of each expert's segment, as the
 *       reference's epilogue leaves them (dispatch_copy_epilogue.cuh:138-141)
 *   dst_buffer_slot_idx [T][K] int32  rank * M + position of the token among this
 *       rank's tokens for that destination, at the lane that sends; else -1
 *   recv_x [n][H] bf16; with do_expand one row per (received token, local expert
 *       it chose), experts' segments in order, rows of an expert in receive order
 *   recv_topk_idx [n][K] int64  local expert index or -1
 *   recv_topk_weights [n][K] fp32 (do_expand: [rows], the weight of that choice); optional
 *   recv_src_metadata [n][K+2] int32: source rank * M + token, source rank * K +
 *       last lane that names a local expert, and with do_expand the row of each lane
 * Rows beyond the received count are left untouched. Only bf16 payloads
 * (x_element_size 2, no scale packs); the reference's pre-quantised (x, sf)
 * input is not built. `cached_mode` (dispatch again with the routing of an
 * earlier handle) recomputes the same layout from `topk_idx` - pass the
 * handle's copy of it. */
typedef struct mcep_elastic_dispatch_args {
    const void* x;               /* [num_tokens][hidden] */
    int32_t x_element_size;      /* 2 */
    const void* sf;              /* must be NULL */
    int32_t num_tokens, hidden, num_sf_packs, sf_token_stride, sf_hidden_stride;
    const int64_t* topk_idx;     /* [num_tokens][num_topk] */
    int32_t num_topk;
    const float* topk_weights;   /* [num_tokens][num_topk] or NULL */
    int32_t* active_ranks;       /* [num_ranks], as in mcep_dispatch */
    int32_t num_experts, num_max_tokens_per_rank, expert_alignment;
    int32_t do_expand, cached_mode;
    int64_t timeout_us;          /* the reference's num_gpu_timeout_secs, in microseconds; -1: hard bound only */
    int32_t async_with_compute_stream;  /* run on the communication stream, return an event */
    uint64_t compute_stream;
    int32_t* psum_num_recv_tokens_per_scaleup_rank;
    int32_t* psum_num_recv_tokens_per_expert;
    int32_t* dst_buffer_slot_idx;
    void* recv_x;
    void* recv_x_scales;         /* must be NULL */
    int64_t* recv_topk_idx;
    float* recv_topk_weights;    /* or NULL */
    int32_t* recv_src_metadata;
    int64_t* copied_topk_idx;    /* [num_tokens][num_topk] or NULL: receives a copy of topk_idx for the handle
                                  * (the reference's kernel has the same output, dispatch_official.cuh:397-399) */
} mcep_elastic_dispatch_args;
int mcep_elastic_dispatch(mcep_buffer* buf, const mcep_elastic_dispatch_args* args,
                          mcep_event** out_event);

/* Replaces MooncakeElasticBuffer::combine
 * (mooncake-ep/src/mooncake_ep_elastic_buffer.cpp:362-426).
 * x: [n][H] bf16, one row per received token (do_expand: the expanded rows,
 * summed per received token before they travel - one row copied, two added as
 * one bf16 addition, more accumulated in fp32 and rounded once:
 * mooncake-ep/include/elastic/mooncake_ep_elastic_combine_official.cuh:146-216
 * with multiple reduction). `recv_src_metadata`
 * must be the tensor a dispatch call of this buffer filled, one of its last
 * two; `topk_idx` the [T][K] tensor of that call. `topk_weights` is accepted
 * and not used by the reduction, as in the reference's forward pass. */
typedef struct mcep_elastic_combine_args {
    const void* x;
    int32_t num_input_tokens, hidden;
    const int64_t* topk_idx;
    int32_t num_combined_tokens, num_topk;
    const float* topk_weights;
    const int32_t* psum_num_recv_tokens_per_scaleup_rank;
    const int32_t* recv_src_metadata;
    int32_t* active_ranks;
    int32_t num_experts, num_max_tokens_per_rank, do_expand;
    int64_t timeout_us;
    int32_t async_with_compute_stream;
    uint64_t compute_stream;
    void* combined_x;            /* [num_combined_tokens][hidden] bf16 */
} mcep_elastic_combine_args;
int mcep_elastic_combine(mcep_buffer* buf, const mcep_elastic_combine_args* args,
                         mcep_event** out_event);

/* Bytes an mcep_buffer needs for the elastic calls of this shape (the counterpart
 * of ElasticBuffer.get_buffer_size_hint,
 * mooncake-wheel/mooncake/mooncake_elastic_buffer.py:315-358). */
uint64_t mcep_elastic_buffer_size_hint(int num_max_tokens_per_rank, int hidden,
                                       int num_ranks, int num_topk);

/* ---- events and hooks --------------------------------------------------------
 * mooncake-ep/include/mooncake_ep_event.h:9-44 (EventHandle) and the
 * std::function returned by dispatch/combine. */
int mcep_event_create(uint64_t stream, mcep_event** out); /* records on `stream` */
int mcep_event_current_stream_wait(mcep_event* ev, uint64_t stream);
int mcep_event_synchronize(mcep_event* ev);
int mcep_event_free(mcep_event* ev);
int mcep_hook_run(mcep_hook* hook);
int mcep_hook_free(mcep_hook* hook);

/* ---- routing layout ----------------------------------------------------------
 * Per-expert and per-rank token counts, prefix offsets and the per-entry slot
 * (position of a (token, expert) message among this rank's messages for that
 * expert, token-ascending) from the top-k indices. The reference computes these
 * inside its dispatch kernel with atomics in arrival order
 * (mooncake-ep/src/mooncake_ep_kernel.cu:274,335-355); its deterministic
 * counterpart is mooncake-ep/include/elastic/
 * mooncake_ep_elastic_dispatch_deterministic_prologue.cuh:16-169.
 *   count[E], rank_count[R], expert_prefix[E] (exclusive, inside the owner
 *   rank's block), slot[T*K] (-1 for masked or repeated entries), all int32.
 * `scratch` is at least mcep_routing_layout_scratch_bytes() of device memory,
 * zeroed once before its first use; calls that share it must not overlap.
 */
size_t mcep_routing_layout_scratch_bytes(void);
int mcep_routing_layout(const int64_t* topk_idx, int num_tokens, int num_topk,
                        int num_experts, int num_ranks, int32_t* count,
                        int32_t* rank_count, int32_t* expert_prefix,
                        int32_t* slot, void* scratch, uint64_t stream);

/* ---- combine without any allocation -------------------------------------------
 * No counterpart in the reference. For callers that are not allowed to allocate
 * device memory (code that runs under a fixed device-memory budget, a serving
 * loop that bans allocator calls once warm, a region owned by a memory pool):
 * they cannot create an mcep_buffer, because creating one calls cudaMalloc.
 * This is the single-rank combine (every expert local, num_ranks == 1) with
 * its scratch - the (token, k) -> packed-row map - in a static device array
 * that is part of the library image (about 256 KiB on every GPU that loads the
 * library, held until the process exits). It calls no cudaMalloc, cudaFree or
 * allocating library routine; the caller passes inputs and the output.
 *   x            [E][M][H] bf16 expert outputs in the packed layout
 *   src_info     [E][M], layout_range [E][1]: the handle of the dispatch
 *   combined_x   [T][H] bf16
 * Same result, bit for bit, as mcep_combine on a single-rank buffer.
 * Limit: num_combined_tokens * num_topk <= MCEP_STATIC_MAX_ENTRIES, otherwise
 * MCEP_ERR_INVALID with a message naming the limit.
 * The first call on a device looks the array's device address up
 * (cudaGetSymbolAddress) and writes two constants with cudaMemcpy; make that
 * first call before any stream capture begins. All calls share the one array:
 * two calls whose kernels overlap on the GPU (different streams, no ordering
 * between them) race on it - order them. Errors of this entry point are read
 * with mcep_static_last_error(). */
#define MCEP_STATIC_MAX_ENTRIES 65536
int mcep_combine_single_rank_static(const void* x, const int64_t* topk_idx,
                                    const float* topk_weights, const int32_t* src_info,
                                    const int64_t* layout_range, int num_experts,
                                    int num_combined_tokens, int hidden, int num_topk,
                                    int num_max_dispatch_tokens_per_rank,
                                    void* combined_x, uint64_t stream);
const char* mcep_static_last_error(void);
/* No counterpart in the reference. Anomalies the kernels of
 * mcep_combine_single_rank_static met in the handle they were given (bit mask
 * as in mcep_buffer_status: 1 row out of range, 4 bad token index) since the
 * last call of this function on the current device; reading clears the word.
 * Waits for the device to go idle first; allocates nothing. */
int mcep_static_status(int32_t* out);

#ifdef __cplusplus
}
#endif
#endif /* MCEP_H_ */
