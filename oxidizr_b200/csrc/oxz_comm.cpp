// The communicator: NCCL, loaded at run time (the library carries no link-time dependency on it, as the
// reference's cudarc loads NCCL dynamically), plus the small blocking collectives the trainer calls directly.
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <condition_variable>
#include <cstring>
#include <functional>
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
    // kernels that wait on other ranks poll this word in host memory: an abort from any thread ends their wait
    OXZ_CUDA(cudaHostAlloc((void**)&c->h_abort_flag, sizeof(int32_t), cudaHostAllocMapped | cudaHostAllocPortable));
    *c->h_abort_flag = 0;
    return OXZ_OK;
}

// ---- local group: rank threads of one process meet on the host ----
struct LocalGroup {
    std::mutex mu;
    std::condition_variable cv;
    int world = 1;
    double timeout_s = 30.0;
    uint64_t generation = 0;
    int arrived = 0;
    bool aborted = false;
    std::vector<std::vector<uint8_t>> slots;
    std::vector<uint8_t> result;
};

// Every rank hands in `bytes` bytes; the last to arrive runs `combine(slots, result)`; every rank leaves with a
// copy of the result. A rank that waits longer than the group's timeout, or an abort from any thread, ends the
// collective with an error on every rank and leaves the group unusable, as the reference's LocalCommunicator does.
static int32_t local_exchange(oxz_comm* c, const void* in, size_t bytes, void* out, size_t out_bytes,
                              const std::function<void(const std::vector<std::vector<uint8_t>>&, std::vector<uint8_t>&)>& combine,
                              const char* what) {
    LocalGroup& g = *c->local;
    std::unique_lock<std::mutex> lock(g.mu);
    if (g.aborted) return fail(OXZ_ERR_ABORTED, "%s: the communicator was aborted", what);
    g.slots[c->rank].assign(static_cast<const uint8_t*>(in), static_cast<const uint8_t*>(in) + bytes);
    const uint64_t gen = g.generation;
    if (++g.arrived == g.world) {
        g.result.clear();
        combine(g.slots, g.result);
        g.arrived = 0;
        g.generation++;
        g.cv.notify_all();
    } else {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(g.timeout_s);
        while (g.generation == gen && !g.aborted) {
            if (g.cv.wait_until(lock, deadline) == std::cv_status::timeout && g.generation == gen && !g.aborted) {
                g.aborted = true;
                g.cv.notify_all();
                return fail(OXZ_ERR_TIMEOUT, "%s: rank %d waited %.3g s for %d of %d ranks that never joined", what,
                            c->rank, g.timeout_s, g.world - g.arrived, g.world);
            }
        }
        if (g.generation == gen) return fail(OXZ_ERR_ABORTED, "%s: the communicator was aborted", what);
    }
    if (out && out_bytes) memcpy(out, g.result.data(), out_bytes < g.result.size() ? out_bytes : g.result.size());
    return OXZ_OK;
}

template <class T>
static int32_t local_sum(oxz_comm* c, T* inout, size_t n, const char* what) {
    return local_exchange(c, inout, n * sizeof(T), inout, n * sizeof(T),
                          [n](const std::vector<std::vector<uint8_t>>& slots, std::vector<uint8_t>& result) {
                              result.assign(n * sizeof(T), 0);
                              T* r = reinterpret_cast<T*>(result.data());
                              for (const auto& sl : slots) {  // rank order: the sum is reproducible
                                  const T* v = reinterpret_cast<const T*>(sl.data());
                                  for (size_t i = 0; i < n; i++) r[i] = r[i] + v[i];
                              }
                          }, what);
}

static int32_t local_gather(oxz_comm* c, const void* in, void* out_all, size_t bytes, const char* what) {
    return local_exchange(c, in, bytes, out_all, bytes * c->world,
                          [](const std::vector<std::vector<uint8_t>>& slots, std::vector<uint8_t>& result) {
                              for (const auto& sl : slots) result.insert(result.end(), sl.begin(), sl.end());
                          }, what);
}

int32_t comm_stream_barrier(oxz_comm* c, int32_t* d_flag, cudaStream_t s) {
    if (c->kind == 1) {
        OXZ_CUDA(cudaStreamSynchronize(s));
        uint8_t z = 0;
        return local_exchange(c, &z, 0, nullptr, 0, [](const auto&, auto&) {}, "step barrier");
    }
    ncclResult_t rc = nccl_api()->AllReduce(d_flag, d_flag, 1, ncclInt32, ncclSum, (ncclComm_t)c->nccl, s);
    if (rc != ncclSuccess) return nccl_fail("step barrier", rc);
    return OXZ_OK;
}

// The union over ranks of per-tensor flags (1 = this rank has a gradient): a local group forms it on the host, in
// place in h_inout, and *host_known says so; NCCL forms it on the device (maximum of bytes), d_in -> d_out, which also
// serves as a barrier on `s`.
int32_t comm_present_union(oxz_comm* c, uint8_t* h_inout, const uint8_t* d_in, uint8_t* d_out, uint64_t n, cudaStream_t s,
                           bool* host_known) {
    if (c->kind == 1) {
        *host_known = true;
        return local_exchange(c, h_inout, n, h_inout, n,
                              [n](const std::vector<std::vector<uint8_t>>& slots, std::vector<uint8_t>& result) {
                                  result.assign(n, 0);
                                  for (const auto& sl : slots)
                                      for (size_t i = 0; i < n && i < sl.size(); i++) result[i] |= sl[i] ? 1 : 0;
                              }, "the union of the ranks' gradient flags");
    }
    *host_known = false;
    if (n == 0) return OXZ_OK;
    ncclResult_t rc = nccl_api()->AllReduce(d_in, d_out, n, ncclUint8, ncclMax, (ncclComm_t)c->nccl, s);
    if (rc != ncclSuccess) return nccl_fail("the union of the ranks' gradient flags", rc);
    return OXZ_OK;
}

int32_t comm_stream_allreduce_f64(oxz_comm* c, double* d_buf, uint32_t n, double* h_tmp, cudaStream_t s) {
    if (c->kind == 1) {
        OXZ_CUDA(cudaMemcpyAsync(h_tmp, d_buf, n * 8, cudaMemcpyDeviceToHost, s));
        OXZ_CUDA(cudaStreamSynchronize(s));
        OXZ_TRY(local_sum<double>(c, h_tmp, n, "the norm all-reduce"));
        OXZ_CUDA(cudaMemcpyAsync(d_buf, h_tmp, n * 8, cudaMemcpyHostToDevice, s));
        // h_tmp is reused by the caller right after: the copy must have read it
        OXZ_CUDA(cudaStreamSynchronize(s));
        return OXZ_OK;
    }
    ncclResult_t rc = nccl_api()->AllReduce(d_buf, d_buf, n, ncclFloat64, ncclSum, (ncclComm_t)c->nccl, s);
    if (rc != ncclSuccess) return nccl_fail("the norm all-reduce", rc);
    return OXZ_OK;
}

int32_t comm_stream_allreduce_u32(oxz_comm* c, uint32_t* d_buf, uint64_t n, cudaStream_t s) {
    if (c->kind == 1) {
        std::vector<uint32_t> host(n);
        OXZ_CUDA(cudaMemcpyAsync(host.data(), d_buf, n * 4, cudaMemcpyDeviceToHost, s));
        OXZ_CUDA(cudaStreamSynchronize(s));
        OXZ_TRY(local_sum<uint32_t>(c, host.data(), n, "the state merge"));
        OXZ_CUDA(cudaMemcpyAsync(d_buf, host.data(), n * 4, cudaMemcpyHostToDevice, s));
        OXZ_CUDA(cudaStreamSynchronize(s));
        return OXZ_OK;
    }
    ncclResult_t rc = nccl_api()->AllReduce(d_buf, d_buf, n, ncclUint32, ncclSum, (ncclComm_t)c->nccl, s);
    if (rc != ncclSuccess) return nccl_fail("the state merge", rc);
    return OXZ_OK;
}

int32_t comm_allgather_host(oxz_comm* c, const void* in, void* out_all, size_t bytes, cudaStream_t s) {
    if (c->kind == 1) return local_gather(c, in, out_all, bytes, "peer rendezvous");
    char* d_all = nullptr;
    OXZ_CUDA(cudaMalloc(&d_all, bytes * c->world));
    OXZ_CUDA(cudaMemcpyAsync(d_all + bytes * c->rank, in, bytes, cudaMemcpyHostToDevice, s));
    ncclResult_t rc = nccl_api()->AllGather(d_all + bytes * c->rank, d_all, bytes, ncclInt8, (ncclComm_t)c->nccl, s);
    if (rc != ncclSuccess) {
        cudaFree(d_all);
        return nccl_fail("peer rendezvous", rc);
    }
    OXZ_CUDA(cudaMemcpyAsync(out_all, d_all, bytes * c->world, cudaMemcpyDeviceToHost, s));
    OXZ_CUDA(cudaStreamSynchronize(s));
    OXZ_CUDA(cudaFree(d_all));
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
    return oxz::guarded("oxz_comm_unique_id", [&]() -> int32_t {
        const NcclApi* api;
        OXZ_TRY(need_api(&api));
        static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
        ncclUniqueId u;
        ncclResult_t rc = api->GetUniqueId(&u);
        if (rc != ncclSuccess) return nccl_fail("ncclGetUniqueId", rc);
        memcpy(id, &u, 128);
        return OXZ_OK;
    });
}

int32_t oxz_comm_init_rank(int32_t device, int32_t rank, int32_t world, const uint8_t id[128], oxz_comm** out) {
    return oxz::guarded("oxz_comm_init_rank", [&]() -> int32_t {
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
    });
}

int32_t oxz_comm_init_all(int32_t n, const int32_t* devices, oxz_comm** out) {
    return oxz::guarded("oxz_comm_init_all", [&]() -> int32_t {
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
            out[i] = c;
            int32_t s = finish_comm(c);
            if (s != OXZ_OK) {
                for (int j = 0; j <= i; j++) { oxz_comm_destroy(out[j]); out[j] = nullptr; }
                for (int j = i + 1; j < n; j++) api->CommAbort(comms[j]);
                return s;
            }
        }
        return OXZ_OK;
    });
}

int32_t oxz_comm_init_local(int32_t n, const int32_t* devices, double timeout_seconds, oxz_comm** out) {
    return oxz::guarded("oxz_comm_init_local", [&]() -> int32_t {
        if (!out) return fail(OXZ_ERR_INVALID, "oxz_comm_init_local: null argument");
        if (n < 1 || n > (int32_t)MAX_PEERS) return fail(OXZ_ERR_INVALID, "oxz_comm_init_local: %d ranks is outside [1, %u]", n, MAX_PEERS);
        if (!(timeout_seconds > 0.0)) return fail(OXZ_ERR_INVALID, "oxz_comm_init_local: the timeout %g s must be positive", timeout_seconds);
        auto group = std::make_shared<LocalGroup>();
        group->world = n;
        group->timeout_s = timeout_seconds;
        group->slots.resize(n);
        for (int i = 0; i < n; i++) {
            oxz_comm* c = new oxz_comm();
            c->kind = 1;
            c->local = group;
            c->rank = i;
            c->world = n;
            c->device = devices ? devices[i] : -1;
            if (c->device >= 0) {
                int32_t s = finish_comm(c);
                if (s != OXZ_OK) return s;
            }
            out[i] = c;
        }
        return OXZ_OK;
    });
}

int32_t oxz_comm_world_size(const oxz_comm* c, int32_t* world) {
    return oxz::guarded("oxz_comm_world_size", [&]() -> int32_t {
        if (!c || !world) return fail(OXZ_ERR_INVALID, "oxz_comm_world_size: null argument");
        *world = c->world;
        return OXZ_OK;
    });
}

int32_t oxz_comm_rank(const oxz_comm* c, int32_t* rank) {
    return oxz::guarded("oxz_comm_rank", [&]() -> int32_t {
        if (!c || !rank) return fail(OXZ_ERR_INVALID, "oxz_comm_rank: null argument");
        *rank = c->rank;
        return OXZ_OK;
    });
}

int32_t oxz_comm_abort(oxz_comm* c) {
    return oxz::guarded("oxz_comm_abort", [&]() -> int32_t {
        if (!c) return fail(OXZ_ERR_INVALID, "oxz_comm_abort: null communicator");
        int expected = 0;
        if (!c->aborted.compare_exchange_strong(expected, 1)) return OXZ_OK;  // the first abort wins
        if (c->h_abort_flag) *reinterpret_cast<volatile int32_t*>(c->h_abort_flag) = 1;  // ends the kernels' own waits
        if (c->kind == 1) {
            std::lock_guard<std::mutex> lock(c->local->mu);
            c->local->aborted = true;
            c->local->cv.notify_all();
            return OXZ_OK;
        }
        const NcclApi* api = nccl_api();
        if (api && c->nccl) {
            ncclResult_t rc = api->CommAbort((ncclComm_t)c->nccl);
            c->nccl = nullptr;
            if (rc != ncclSuccess) return nccl_fail("ncclCommAbort", rc);
        }
        return OXZ_OK;
    });
}

int32_t oxz_comm_destroy(oxz_comm* c) {
    return oxz::guarded("oxz_comm_destroy", [&]() -> int32_t {
        if (!c) return OXZ_OK;
        const NcclApi* api = c->kind == 0 ? nccl_api() : nullptr;
        if (c->device >= 0) cudaSetDevice(c->device);
        if (api && c->nccl && !c->aborted.load()) api->CommDestroy((ncclComm_t)c->nccl);
        if (c->d_small) cudaFree(c->d_small);
        if (c->h_abort_flag) cudaFreeHost(c->h_abort_flag);
        if (c->stream) cudaStreamDestroy(c->stream);
        delete c;
        return OXZ_OK;
    });
}

int32_t oxz_allreduce_i64x2(oxz_comm* c, int64_t inout[2]) {
    return oxz::guarded("oxz_allreduce_i64x2", [&]() -> int32_t {
        OXZ_TRY(comm_check(c, "oxz_allreduce_i64x2"));
        if (!inout) return fail(OXZ_ERR_INVALID, "oxz_allreduce_i64x2: null argument");
        if (c->world <= 1) return OXZ_OK;
        for (int i = 0; i < 2; i++)
            if (inout[i] < 0) return fail(OXZ_ERR_INVALID, "step count %lld is negative. Every rank must pass counts of 0 or more", (long long)inout[i]);
        if (c->kind == 1) return local_sum<int64_t>(c, inout, 2, "the step-count sum");
        const NcclApi* api = nccl_api();
        OXZ_CUDA(cudaSetDevice(c->device));
        OXZ_CUDA(cudaMemcpyAsync(c->d_small, inout, 16, cudaMemcpyHostToDevice, c->stream));
        ncclResult_t rc = api->AllReduce(c->d_small, c->d_small, 2, ncclInt64, ncclSum, (ncclComm_t)c->nccl, c->stream);
        if (rc != ncclSuccess) return nccl_fail("the step-count sum", rc);
        OXZ_CUDA(cudaMemcpyAsync(inout, c->d_small, 16, cudaMemcpyDeviceToHost, c->stream));
        OXZ_CUDA(cudaStreamSynchronize(c->stream));
        if (c->aborted.load()) return fail(OXZ_ERR_ABORTED, "oxz_allreduce_i64x2: the communicator was aborted");
        return OXZ_OK;
    });
}

int32_t oxz_allreduce_f64(oxz_comm* c, double* inout, uint32_t n) {
    return oxz::guarded("oxz_allreduce_f64", [&]() -> int32_t {
        OXZ_TRY(comm_check(c, "oxz_allreduce_f64"));
        if (!inout && n) return fail(OXZ_ERR_INVALID, "oxz_allreduce_f64: null argument");
        if (n > 16) return fail(OXZ_ERR_INVALID, "oxz_allreduce_f64: %u values, at most 16", n);
        if (c->world <= 1 || n == 0) return OXZ_OK;
        if (c->kind == 1) return local_sum<double>(c, inout, n, "the loss sum");
        const NcclApi* api = nccl_api();
        OXZ_CUDA(cudaSetDevice(c->device));
        OXZ_CUDA(cudaMemcpyAsync(c->d_small, inout, n * 8, cudaMemcpyHostToDevice, c->stream));
        ncclResult_t rc = api->AllReduce(c->d_small, c->d_small, n, ncclFloat64, ncclSum, (ncclComm_t)c->nccl, c->stream);
        if (rc != ncclSuccess) return nccl_fail("the loss sum", rc);
        OXZ_CUDA(cudaMemcpyAsync(inout, c->d_small, n * 8, cudaMemcpyDeviceToHost, c->stream));
        OXZ_CUDA(cudaStreamSynchronize(c->stream));
        if (c->aborted.load()) return fail(OXZ_ERR_ABORTED, "oxz_allreduce_f64: the communicator was aborted");
        return OXZ_OK;
    });
}

int32_t oxz_broadcast(oxz_comm* c, void* device_ptr, uint64_t bytes, int32_t root) {
    return oxz::guarded("oxz_broadcast", [&]() -> int32_t {
        OXZ_TRY(comm_check(c, "oxz_broadcast"));
        if (root < 0 || root >= c->world) return fail(OXZ_ERR_INVALID, "oxz_broadcast: root %d of world %d", root, c->world);
        if (c->world <= 1 || bytes == 0) return OXZ_OK;
        if (!device_ptr) return fail(OXZ_ERR_INVALID, "oxz_broadcast: null buffer");
        if (c->kind == 1) {
            // through host memory: the root's bytes are what every rank leaves with
            OXZ_CUDA(cudaSetDevice(c->device));
            std::vector<uint8_t> host(c->rank == root ? bytes : 0);
            if (c->rank == root) OXZ_CUDA(cudaMemcpy(host.data(), device_ptr, bytes, cudaMemcpyDeviceToHost));
            std::vector<uint8_t> got(bytes);
            OXZ_TRY(local_exchange(c, host.data(), host.size(), got.data(), bytes,
                                   [root](const auto& slots, auto& result) { result = slots[root]; }, "oxz_broadcast"));
            if (c->rank != root) OXZ_CUDA(cudaMemcpy(device_ptr, got.data(), bytes, cudaMemcpyHostToDevice));
            return OXZ_OK;
        }
        const NcclApi* api = nccl_api();
        OXZ_CUDA(cudaSetDevice(c->device));
        ncclResult_t rc = api->Broadcast(device_ptr, device_ptr, bytes, ncclInt8, root, (ncclComm_t)c->nccl, c->stream);
        if (rc != ncclSuccess) return nccl_fail("ncclBroadcast", rc);
        OXZ_CUDA(cudaStreamSynchronize(c->stream));
        return OXZ_OK;
    });
}

int32_t oxz_barrier(oxz_comm* c) {
    return oxz::guarded("oxz_barrier", [&]() -> int32_t {
        OXZ_TRY(comm_check(c, "oxz_barrier"));
        if (c->world <= 1) return OXZ_OK;
        if (c->kind == 1) {
            uint8_t z = 0;
            return local_exchange(c, &z, 0, nullptr, 0, [](const auto&, auto&) {}, "oxz_barrier");
        }
        const NcclApi* api = nccl_api();
        OXZ_CUDA(cudaSetDevice(c->device));
        int32_t* flag = reinterpret_cast<int32_t*>(static_cast<char*>(c->d_small) + 256);
        ncclResult_t rc = api->AllReduce(flag, flag, 1, ncclInt32, ncclSum, (ncclComm_t)c->nccl, c->stream);
        if (rc != ncclSuccess) return nccl_fail("barrier", rc);
        OXZ_CUDA(cudaStreamSynchronize(c->stream));
        return OXZ_OK;
    });
}

}  // extern "C"
