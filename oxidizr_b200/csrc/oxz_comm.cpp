// The communicator: NCCL, loaded at run time (the library carries no link-time dependency on it, as the
// reference's cudarc loads NCCL dynamically), plus the small blocking collectives the trainer calls directly.
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>

#include "oxz_internal.h"
#include "oxz_nccl.h"

namespace oxz {

static NcclApi g_api;
static std::once_flag g_once;
static std::string g_load_error;

static void load_nccl() {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        // RTLD_NOLOAD first: a process that already holds NCCL (through torch, say) must share that copy.
        h = dlopen(n, RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
        if (h) break;
    }
    for (const char* n : names) {
        if (h) break;
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    }
    if (!h) {
        g_load_error = std::string("NCCL library not found: ") + (dlerror() ? dlerror() : "dlopen failed");
        return;
    }
#define OXZ_SYM(field, name)                                              \
    g_api.field = reinterpret_cast<decltype(g_api.field)>(dlsym(h, name)); \
    if (!g_api.field) {                                                   \
        g_load_error = std::string("NCCL symbol missing: ") + name;       \
        return;                                                           \
    }
    OXZ_SYM(GetUniqueId, "ncclGetUniqueId")
    OXZ_SYM(CommInitRank, "ncclCommInitRank")
    OXZ_SYM(CommInitAll, "ncclCommInitAll")
    OXZ_SYM(CommDestroy, "ncclCommDestroy")
    OXZ_SYM(CommAbort, "ncclCommAbort")
    OXZ_SYM(GetErrorString, "ncclGetErrorString")
    OXZ_SYM(AllReduce, "ncclAllReduce")
    OXZ_SYM(ReduceScatter, "ncclReduceScatter")
    OXZ_SYM(AllGather, "ncclAllGather")
    OXZ_SYM(Broadcast, "ncclBroadcast")
    OXZ_SYM(GroupStart, "ncclGroupStart")
    OXZ_SYM(GroupEnd, "ncclGroupEnd")
#undef OXZ_SYM
    g_api.loaded = true;
}

const NcclApi* nccl_api() {
    std::call_once(g_once, load_nccl);
    return g_api.loaded ? &g_api : nullptr;
}

int32_t nccl_fail(const char* what, int rc) {
    const NcclApi* api = nccl_api();
    return fail(OXZ_ERR_NCCL, "%s failed: %s", what, api ? api->GetErrorString((ncclResult_t)rc) : "NCCL not loaded");
}

static int32_t need_api(const NcclApi** api) {
    *api = nccl_api();
    if (!*api) return fail(OXZ_ERR_UNSUPPORTED, "%s", g_load_error.c_str());
    return OXZ_OK;
}

static int32_t finish_comm(oxz_comm* c) {
    OXZ_CUDA(cudaSetDevice(c->device));
    OXZ_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    OXZ_CUDA(cudaMalloc(&c->d_small, 512));
    OXZ_CUDA(cudaMemset(c->d_small, 0, 512));
    return OXZ_OK;
}

int32_t comm_check(oxz_comm* c, const char* who) {
    if (!c) return fail(OXZ_ERR_INVALID, "%s: null communicator", who);
    if (c->aborted.load()) return fail(OXZ_ERR_ABORTED, "%s: the communicator was aborted", who);
    return OXZ_OK;
}

}  // namespace oxz

using namespace oxz;

extern "C" {

int32_t oxz_comm_unique_id(uint8_t id[128]) {
    const NcclApi* api;
    OXZ_TRY(need_api(&api));
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    ncclUniqueId u;
    ncclResult_t rc = api->GetUniqueId(&u);
    if (rc != ncclSuccess) return nccl_fail("ncclGetUniqueId", rc);
    memcpy(id, &u, 128);
    return OXZ_OK;
}

int32_t oxz_comm_init_rank(int32_t device, int32_t rank, int32_t world, const uint8_t id[128], oxz_comm** out) {
    if (!out || !id) return fail(OXZ_ERR_INVALID, "oxz_comm_init_rank: null argument");
    *out = nullptr;
    if (world < 1) return fail(OXZ_ERR_INVALID, "world size is 0: a run needs at least one rank.");
    if (rank < 0 || rank >= world)
        return fail(OXZ_ERR_INVALID, "rank %d is not below world size %d. Pass a rank in [0, %d).", rank, world, world);
    const NcclApi* api;
    OXZ_TRY(need_api(&api));
    OXZ_CUDA(cudaSetDevice(device));
    ncclUniqueId u;
    memcpy(&u, id, 128);
    ncclComm_t comm;
    ncclResult_t rc = api->CommInitRank(&comm, world, u, rank);
    if (rc != ncclSuccess) return nccl_fail("ncclCommInitRank", rc);
    oxz_comm* c = new oxz_comm();
    c->nccl = comm;
    c->rank = rank;
    c->world = world;
    c->device = device;
    int32_t s = finish_comm(c);
    if (s != OXZ_OK) {
        api->CommAbort(comm);
        delete c;
        return s;
    }
    *out = c;
    return OXZ_OK;
}

int32_t oxz_comm_init_all(int32_t n, const int32_t* devices, oxz_comm** out) {
    if (!out || !devices) return fail(OXZ_ERR_INVALID, "oxz_comm_init_all: null argument");
    if (n < 1 || n > (int32_t)MAX_PEERS) return fail(OXZ_ERR_INVALID, "oxz_comm_init_all: %d ranks is outside [1, %u]", n, MAX_PEERS);
    const NcclApi* api;
    OXZ_TRY(need_api(&api));
    std::vector<ncclComm_t> comms(n);
    ncclResult_t rc = api->CommInitAll(comms.data(), n, devices);
    if (rc != ncclSuccess) return nccl_fail("ncclCommInitAll", rc);
    for (int i = 0; i < n; i++) {
        oxz_comm* c = new oxz_comm();
        c->nccl = comms[i];
        c->rank = i;
        c->world = n;
        c->device = devices[i];
        int32_t s = finish_comm(c);
        if (s != OXZ_OK) return s;
        out[i] = c;
    }
    return OXZ_OK;
}

int32_t oxz_comm_world_size(const oxz_comm* c, int32_t* world) {
    if (!c || !world) return fail(OXZ_ERR_INVALID, "oxz_comm_world_size: null argument");
    *world = c->world;
    return OXZ_OK;
}

int32_t oxz_comm_rank(const oxz_comm* c, int32_t* rank) {
    if (!c || !rank) return fail(OXZ_ERR_INVALID, "oxz_comm_rank: null argument");
    *rank = c->rank;
    return OXZ_OK;
}

int32_t oxz_comm_abort(oxz_comm* c) {
    if (!c) return fail(OXZ_ERR_INVALID, "oxz_comm_abort: null communicator");
    int expected = 0;
    if (!c->aborted.compare_exchange_strong(expected, 1)) return OXZ_OK;  // the first abort wins
    const NcclApi* api = nccl_api();
    if (api && c->nccl) {
        ncclResult_t rc = api->CommAbort((ncclComm_t)c->nccl);
        c->nccl = nullptr;
        if (rc != ncclSuccess) return nccl_fail("ncclCommAbort", rc);
    }
    return OXZ_OK;
}

int32_t oxz_comm_destroy(oxz_comm* c) {
    if (!c) return OXZ_OK;
    const NcclApi* api = nccl_api();
    cudaSetDevice(c->device);
    if (api && c->nccl && !c->aborted.load()) api->CommDestroy((ncclComm_t)c->nccl);
    if (c->d_small) cudaFree(c->d_small);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
    return OXZ_OK;
}

int32_t oxz_allreduce_i64x2(oxz_comm* c, int64_t inout[2]) {
    OXZ_TRY(comm_check(c, "oxz_allreduce_i64x2"));
    if (!inout) return fail(OXZ_ERR_INVALID, "oxz_allreduce_i64x2: null argument");
    if (c->world <= 1) return OXZ_OK;
    for (int i = 0; i < 2; i++)
        if (inout[i] < 0) return fail(OXZ_ERR_INVALID, "step count %lld is negative. Every rank must pass counts of 0 or more", (long long)inout[i]);
    const NcclApi* api = nccl_api();
    OXZ_CUDA(cudaSetDevice(c->device));
    OXZ_CUDA(cudaMemcpyAsync(c->d_small, inout, 16, cudaMemcpyHostToDevice, c->stream));
    ncclResult_t rc = api->AllReduce(c->d_small, c->d_small, 2, ncclInt64, ncclSum, (ncclComm_t)c->nccl, c->stream);
    if (rc != ncclSuccess) return nccl_fail("the step-count sum", rc);
    OXZ_CUDA(cudaMemcpyAsync(inout, c->d_small, 16, cudaMemcpyDeviceToHost, c->stream));
    OXZ_CUDA(cudaStreamSynchronize(c->stream));
    if (c->aborted.load()) return fail(OXZ_ERR_ABORTED, "oxz_allreduce_i64x2: the communicator was aborted");
    return OXZ_OK;
}

int32_t oxz_allreduce_f64(oxz_comm* c, double* inout, uint32_t n) {
    OXZ_TRY(comm_check(c, "oxz_allreduce_f64"));
    if (!inout && n) return fail(OXZ_ERR_INVALID, "oxz_allreduce_f64: null argument");
    if (n > 16) return fail(OXZ_ERR_INVALID, "oxz_allreduce_f64: %u values, at most 16", n);
    if (c->world <= 1 || n == 0) return OXZ_OK;
    const NcclApi* api = nccl_api();
    OXZ_CUDA(cudaSetDevice(c->device));
    OXZ_CUDA(cudaMemcpyAsync(c->d_small, inout, n * 8, cudaMemcpyHostToDevice, c->stream));
    ncclResult_t rc = api->AllReduce(c->d_small, c->d_small, n, ncclFloat64, ncclSum, (ncclComm_t)c->nccl, c->stream);
    if (rc != ncclSuccess) return nccl_fail("the loss sum", rc);
    OXZ_CUDA(cudaMemcpyAsync(inout, c->d_small, n * 8, cudaMemcpyDeviceToHost, c->stream));
    OXZ_CUDA(cudaStreamSynchronize(c->stream));
    if (c->aborted.load()) return fail(OXZ_ERR_ABORTED, "oxz_allreduce_f64: the communicator was aborted");
    return OXZ_OK;
}

int32_t oxz_broadcast(oxz_comm* c, void* device_ptr, uint64_t bytes, int32_t root) {
    OXZ_TRY(comm_check(c, "oxz_broadcast"));
    if (root < 0 || root >= c->world) return fail(OXZ_ERR_INVALID, "oxz_broadcast: root %d of world %d", root, c->world);
    if (c->world <= 1 || bytes == 0) return OXZ_OK;
    if (!device_ptr) return fail(OXZ_ERR_INVALID, "oxz_broadcast: null buffer");
    const NcclApi* api = nccl_api();
    OXZ_CUDA(cudaSetDevice(c->device));
    ncclResult_t rc = api->Broadcast(device_ptr, device_ptr, bytes, ncclInt8, root, (ncclComm_t)c->nccl, c->stream);
    if (rc != ncclSuccess) return nccl_fail("ncclBroadcast", rc);
    OXZ_CUDA(cudaStreamSynchronize(c->stream));
    return OXZ_OK;
}

int32_t oxz_barrier(oxz_comm* c) {
    OXZ_TRY(comm_check(c, "oxz_barrier"));
    if (c->world <= 1) return OXZ_OK;
    const NcclApi* api = nccl_api();
    OXZ_CUDA(cudaSetDevice(c->device));
    int32_t* flag = reinterpret_cast<int32_t*>(static_cast<char*>(c->d_small) + 256);
    ncclResult_t rc = api->AllReduce(flag, flag, 1, ncclInt32, ncclSum, (ncclComm_t)c->nccl, c->stream);
    if (rc != ncclSuccess) return nccl_fail("barrier", rc);
    OXZ_CUDA(cudaStreamSynchronize(c->stream));
    return OXZ_OK;
}

}  // extern "C"
