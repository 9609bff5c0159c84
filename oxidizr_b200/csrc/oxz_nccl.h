// Function table of the NCCL entry points the library uses, resolved with dlopen/dlsym at first use.
#pragma once

#include <nccl.h>
#include <stdint.h>

namespace oxz {

struct NcclApi {
    bool loaded = false;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
};

// nullptr when the NCCL library could not be loaded.
const NcclApi* nccl_api();
int32_t nccl_fail(const char* what, int rc);

}  // namespace oxz

struct oxz_comm;
namespace oxz {
int32_t comm_check(oxz_comm* c, const char* who);

// Collectives the step enqueues, for either kind of communicator. With NCCL they are asynchronous on `s`; a local
// group drains `s`, meets the other rank threads on the host and resumes.
// Barrier: every rank's work enqueued before it on its own stream has finished when it ends.
int32_t comm_stream_barrier(oxz_comm* c, int32_t* d_flag, cudaStream_t s);
// Union over ranks of n per-tensor flags: on the host for a local group (h_inout, in place; *host_known = true), on the
// device for NCCL (d_in -> d_out on `s`, which also serves as a barrier; *host_known = false).
int32_t comm_present_union(oxz_comm* c, uint8_t* h_inout, const uint8_t* d_in, uint8_t* d_out, uint64_t n, cudaStream_t s,
                           bool* host_known);
// Sum of n device doubles over ranks, in place. h_tmp: n pinned doubles of staging for the local kind.
int32_t comm_stream_allreduce_f64(oxz_comm* c, double* d_buf, uint32_t n, double* h_tmp, cudaStream_t s);
// Sum of n device 32-bit words over ranks, in place (merging disjoint slices bit for bit). Blocking for a local group.
int32_t comm_stream_allreduce_u32(oxz_comm* c, uint32_t* d_buf, uint64_t n, cudaStream_t s);
// All-gather of `bytes` host bytes per rank into out_all (world * bytes), blocking.
int32_t comm_allgather_host(oxz_comm* c, const void* in, void* out_all, size_t bytes, cudaStream_t s);
}
