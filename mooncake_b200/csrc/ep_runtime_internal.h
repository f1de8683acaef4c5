// What the elastic-style entry points (ep_elastic.cu) need to know about a
// buffer, without the whole of its definition.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <functional>

struct mcep_buffer;

namespace mcep {

struct BufferView {
    char* base;               // symmetric allocation (null for a single rank without one)
    size_t data_off;          // where the caller-sized data area starts inside it
    int64_t num_bytes;        // size of the data area
    void* const* peer_host;   // [num_ranks] bases of all ranks' allocations (host copy)
    int rank, num_ranks, num_sms;
    int32_t* status;          // device status words
    cudaStream_t comm_stream;
    bool group;               // the calls go through symmetric memory
    bool defer;               // calls are prepared and launched later (in-process groups)
};
BufferView view_of(mcep_buffer* b);

// Bytes of the data area both parities of an exchange with these sizes occupy.
size_t exchange_bytes(int num_ranks, int num_experts, int M, int hidden);

// Deferred launches: work to start right after the buffer's prepared dispatch
// has been launched (run once, then forgotten).
void set_after_deferred(mcep_buffer* b, std::function<int()> fn);

// The first kernel of the buffer's NEXT dispatch call may be launched with
// programmatic stream serialisation: the caller has just queued, on the same
// stream, a kernel that lets its dependents start early and whose outputs that
// first kernel reads only after waiting for it (all first kernels wait at their top).
void allow_chained_first_launch(mcep_buffer* b);

// Records the message mcep_last_error() returns and hands `code` back.
int report_failure(int code, const char* message);

// Called by mcep_buffer_destroy: frees what the elastic entry points keep for `b`.
void elastic_release(mcep_buffer* b);

}  // namespace mcep
