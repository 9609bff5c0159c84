// Device state of a plan and the optimizer step itself: the order of src/trainer.rs:515-695 as one stream of
// kernel launches with the skip decision taken on the device.
#include <unistd.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <utility>
#include <mutex>

#include "oxz_internal.h"
#include "oxz_nccl.h"

using namespace oxz;

namespace {

TileMap tile_map(const oxz_plan* p) {
    TileMap m;
    m.tiles_per_shard = (uint32_t)(p->bucket_tiles / (uint64_t)p->world);
    m.tiles_per_bucket = (uint32_t)p->bucket_tiles;
    m.n_buckets = (uint32_t)p->n_buckets;
    m.last_shard_tiles = (uint32_t)(p->last_bucket_tiles / (uint64_t)p->world);
    m.rank = (uint32_t)p->rank;
    m.n_local_tiles = (uint32_t)p->local_tiles;
    m.first_tile = 0;
    return m;
}

ncclDataType_t nccl_dtype(int32_t dt) { return dt == OXZ_F32 ? ncclFloat32 : dt == OXZ_BF16 ? ncclBfloat16 : ncclFloat16; }

struct PeerBlob {
    uint64_t pid;
    uint64_t grads_ptr, work_ptr, mail_ptr;
    int32_t device, has_mail;
    cudaIpcMemHandle_t grads_handle, work_handle, mail_handle;
};

// Exchanges the gradient and weight buffers of every rank and maps the peers' copies into this process.
// Ranks of one process (one thread per rank) use each other's pointers directly after enabling peer access;
// ranks of other processes are opened through CUDA IPC handles.
int32_t exchange_peers(oxz_plan* p, oxz_comm* c) {
    if (c->kind == 0 && !nccl_api()) return fail(OXZ_ERR_UNSUPPORTED, "the NCCL communicator's library is not loaded");
    PeerBlob mine{};
    mine.pid = (uint64_t)getpid();
    mine.grads_ptr = (uint64_t)p->grads;
    mine.work_ptr = (uint64_t)p->work;
    mine.device = p->device;
    OXZ_CUDA(cudaIpcGetMemHandle(&mine.grads_handle, p->grads));
    OXZ_CUDA(cudaIpcGetMemHandle(&mine.work_handle, p->work));
    mine.has_mail = p->mail ? 1 : 0;
    mine.mail_ptr = (uint64_t)p->mail;
    if (p->mail) OXZ_CUDA(cudaIpcGetMemHandle(&mine.mail_handle, p->mail));
    const int W = p->cw;
    std::vector<PeerBlob> all(W);
    OXZ_TRY(comm_allgather_host(c, &mine, all.data(), sizeof(PeerBlob), p->stream));
    // the mailbox serves only when every rank made one (the same environment and tensor count everywhere)
    bool all_mail = p->mail != nullptr;
    for (int r = 0; r < W; r++) all_mail = all_mail && all[r].has_mail != 0;
    p->use_mail = all_mail;
    for (int r = 0; r < W; r++) {
        if (r == p->cr) {
            p->peers.grads[r] = p->grads;
            p->peers.work[r] = p->work;
            p->mail_peers.box[r] = p->mail;
            continue;
        }
        const PeerBlob& b = all[r];
        if (b.pid == mine.pid) {
            if (b.device != p->device) {
                int can = 0;
                OXZ_CUDA(cudaDeviceCanAccessPeer(&can, p->device, b.device));
                if (!can) return fail(OXZ_ERR_UNSUPPORTED, "device %d cannot access device %d as a peer", p->device, b.device);
                cudaError_t e = cudaDeviceEnablePeerAccess(b.device, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else if (e != cudaSuccess) return fail(OXZ_ERR_CUDA, "cudaDeviceEnablePeerAccess(%d): %s", b.device, cudaGetErrorString(e));
            }
            p->peers.grads[r] = (const void*)b.grads_ptr;
            p->peers.work[r] = (void*)b.work_ptr;
            if (all_mail) p->mail_peers.box[r] = (MailBox*)b.mail_ptr;
        } else {
            void *g = nullptr, *w = nullptr;
            OXZ_CUDA(cudaIpcOpenMemHandle(&g, b.grads_handle, cudaIpcMemLazyEnablePeerAccess));
            OXZ_CUDA(cudaIpcOpenMemHandle(&w, b.work_handle, cudaIpcMemLazyEnablePeerAccess));
            p->ipc_opened.push_back(g);
            p->ipc_opened.push_back(w);
            p->peers.grads[r] = g;
            p->peers.work[r] = w;
            if (all_mail) {
                void* mb = nullptr;
                OXZ_CUDA(cudaIpcOpenMemHandle(&mb, b.mail_handle, cudaIpcMemLazyEnablePeerAccess));
                p->ipc_opened.push_back(mb);
                p->mail_peers.box[r] = (MailBox*)mb;
            }
        }
    }
    return OXZ_OK;
}

// The same rendezvous for the second gradient buffer alone.
int32_t exchange_alt_grads(oxz_plan* p, oxz_comm* c) {
    struct Blob {
        uint64_t pid, ptr;
        int32_t device, pad;
        cudaIpcMemHandle_t handle;
    };
    Blob mine{};
    mine.pid = (uint64_t)getpid();
    mine.ptr = (uint64_t)p->grads_alt;
    mine.device = p->device;
    OXZ_CUDA(cudaIpcGetMemHandle(&mine.handle, p->grads_alt));
    std::vector<Blob> all(p->cw);
    OXZ_TRY(comm_allgather_host(c, &mine, all.data(), sizeof(Blob), p->stream));
    for (int r = 0; r < p->cw; r++) {
        if (r == p->cr) {
            p->peer_grads_alt[r] = p->grads_alt;
        } else if (all[r].pid == mine.pid) {
            p->peer_grads_alt[r] = (const void*)all[r].ptr;  // peer access was enabled for the first buffer
        } else {
            void* g = nullptr;
            OXZ_CUDA(cudaIpcOpenMemHandle(&g, all[r].handle, cudaIpcMemLazyEnablePeerAccess));
            p->ipc_opened.push_back(g);
            p->peer_grads_alt[r] = g;
        }
    }
    return OXZ_OK;
}

// Runs of one tensor's flat span that a rank owns: calls fn(flat_start, local_start, len) per run.
template <class F>
void for_owned_runs(const oxz_plan* p, uint64_t tensor, F fn) {
    const uint64_t lo = p->offset[tensor], hi = lo + p->numel[tensor];
    if (hi == lo) return;
    const uint64_t bucket_elems = p->bucket_tiles * TILE;
    const uint64_t full_shard = bucket_elems / (uint64_t)p->world;
    for (uint64_t b = lo / bucket_elems; b < p->n_buckets && b * bucket_elems < hi; b++) {
        const uint64_t tiles = (b == p->n_buckets - 1) ? p->last_bucket_tiles : p->bucket_tiles;
        const uint64_t shard = tiles * TILE / (uint64_t)p->world;
        const uint64_t s0 = b * bucket_elems + (uint64_t)p->rank * shard, s1 = s0 + shard;
        const uint64_t a = lo > s0 ? lo : s0, z = hi < s1 ? hi : s1;
        if (a < z) fn(a, b * full_shard + (a - s0), z - a);
    }
}

// Buckets [b0, b1) of pipeline group g: the buckets are split into pipe_groups nearly equal runs.
void group_buckets(const oxz_plan* p, uint32_t g, uint64_t* b0, uint64_t* b1) {
    const uint64_t nb = p->n_buckets, G = p->pipe_groups;
    *b0 = nb * g / G;
    *b1 = nb * (g + 1) / G;
}

// The local tile range of buckets [b0, b1).
void group_tiles(const oxz_plan* p, uint64_t b0, uint64_t b1, uint32_t* first, uint32_t* end) {
    const uint64_t tps = p->bucket_tiles / (uint64_t)p->world;
    *first = (uint32_t)(b0 * tps);
    *end = (uint32_t)(b1 == p->n_buckets ? p->local_tiles : b1 * tps);
}

// Copies this rank's shard of buckets [b0, b1) between two buffers with the copy engine. A buffer is either flat
// (the shard of bucket b sits at b * bucket + rank * shard) or packed (at b * shard, the layout of the local state).
// The full buckets form one strided 2-D copy; a shorter last bucket is one more 1-D copy.
int32_t copy_shard_rows(const oxz_plan* p, char* dst, bool dst_packed, const char* src, bool src_packed, size_t es,
                        uint64_t b0, uint64_t b1, cudaStream_t st) {
    const uint64_t W = (uint64_t)p->world, bucket = p->bucket_tiles * TILE, shard = bucket / W;
    const uint64_t last = p->n_buckets - 1;
    const bool has_last = b1 == p->n_buckets && p->last_bucket_tiles != p->bucket_tiles;
    const uint64_t full_end = has_last ? last : b1;
    auto at = [&](bool packed, uint64_t b, uint64_t shard_elems) -> uint64_t {
        return packed ? b * shard : b * bucket + (uint64_t)p->rank * shard_elems;
    };
    if (full_end > b0) {
        OXZ_CUDA(cudaMemcpy2DAsync(dst + at(dst_packed, b0, shard) * es, (dst_packed ? shard : bucket) * es,
                                   src + at(src_packed, b0, shard) * es, (src_packed ? shard : bucket) * es, shard * es,
                                   full_end - b0, cudaMemcpyDeviceToDevice, st));
    }
    if (has_last && b1 > b0) {
        const uint64_t lshard = p->last_bucket_tiles * TILE / W;
        OXZ_CUDA(cudaMemcpyAsync(dst + at(dst_packed, last, lshard) * es, src + at(src_packed, last, lshard) * es, lshard * es,
                                 cudaMemcpyDeviceToDevice, st));
    }
    return OXZ_OK;
}

float* state_array(oxz_plan* p, int32_t kind) {
    switch (kind) {
        case OXZ_STATE_MASTER: return p->master;
        case OXZ_STATE_EXP_AVG: return p->exp_avg;
        case OXZ_STATE_EXP_AVG_SQ: return p->exp_avg_sq;
        default: return nullptr;
    }
}

int32_t check_state_call(oxz_plan* p, int32_t kind, uint64_t tensor, const void* host, const char* who) {
    if (!p || !host) return fail(OXZ_ERR_INVALID, "%s: null argument", who);
    if (!p->allocated) return fail(OXZ_ERR_STATE, "%s: the plan has no device state. Call oxz_state_alloc first", who);
    if (p->inflight) return fail(OXZ_ERR_STATE, "%s: a step is in flight. Call oxz_step_wait first", who);
    if (tensor >= p->T) return fail(OXZ_ERR_INVALID, "%s: tensor %llu of %llu", who, (unsigned long long)tensor, (unsigned long long)p->T);
    if (kind < OXZ_STATE_MASTER || kind > OXZ_STATE_GRADS) return fail(OXZ_ERR_INVALID, "%s: unknown state kind %d", who, kind);
    return OXZ_OK;
}

}  // namespace

extern "C" {

int32_t oxz_plan_destroy(oxz_plan* p) {
    return oxz::guarded("oxz_plan_destroy", [&]() -> int32_t {
        if (!p) return OXZ_OK;
        if (p->allocated || p->own_stream) {  // also after an allocation that failed midway
            cudaSetDevice(p->device);
            if (p->stream) cudaStreamSynchronize(p->stream);
            for (void* q : p->ipc_opened) cudaIpcCloseMemHandle(q);
            if (p->work && p->work != (void*)p->master) cudaFree(p->work);
            for (void* q : {(void*)p->grads, (void*)p->master, (void*)p->exp_avg, (void*)p->exp_avg_sq, p->reduced,
                            (void*)p->d_tile_meta, (void*)p->d_present, (void*)p->d_offsets, (void*)p->d_numel,
                            (void*)p->d_src, (void*)p->d_partials, (void*)p->d_acc, (void*)p->d_scalars, (void*)p->d_present_in,
                            (void*)p->mail})
                if (q) cudaFree(q);
            for (void* q : {(void*)p->h_scalars, (void*)p->h_acc, (void*)p->h_extras, (void*)p->h_present, (void*)p->h_union, (void*)p->h_src})
                if (q) cudaFreeHost(q);
            if (p->grads_alt) cudaFree(p->grads_alt);
            if (p->upload_stream) cudaStreamDestroy(p->upload_stream);
            if (p->ev_uploaded) cudaEventDestroy(p->ev_uploaded);
            for (auto e : p->ev_last_read) if (e) cudaEventDestroy(e);
            if (p->early_stream) cudaStreamDestroy(p->early_stream);
            if (p->ev_produced) cudaEventDestroy(p->ev_produced);
            if (p->ev_early) cudaEventDestroy(p->ev_early);
            if (p->stage) cudaFree(p->stage);
            for (auto st : p->copy_stream) if (st) cudaStreamDestroy(st);
            if (p->ev_go) cudaEventDestroy(p->ev_go);
            for (auto& row : p->ev_copied) for (auto e : row) if (e) cudaEventDestroy(e);
            for (auto e : p->ev_updated) if (e) cudaEventDestroy(e);
            for (auto e : p->ev_pushed) if (e) cudaEventDestroy(e);
            if (p->done) cudaEventDestroy(p->done);
            for (auto e : p->ev) if (e) cudaEventDestroy(e);
            if (p->own_stream) cudaStreamDestroy(p->own_stream);
        }
        delete p;
        return OXZ_OK;
    });
}

int32_t oxz_plan_set_stream(oxz_plan* p, void* stream) {
    return oxz::guarded("oxz_plan_set_stream", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_plan_set_stream: null plan");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_plan_set_stream: call oxz_state_alloc first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_plan_set_stream: a step is in flight");
        p->stream = stream ? (cudaStream_t)stream : p->own_stream;
        return OXZ_OK;
    });
}

int32_t oxz_state_alloc(oxz_plan* p, oxz_comm* comm) {
    return oxz::guarded("oxz_state_alloc", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_state_alloc: null plan");
        if (p->allocated) return fail(OXZ_ERR_STATE, "oxz_state_alloc: the plan already has device state");
        if (p->own_stream) return fail(OXZ_ERR_STATE, "oxz_state_alloc: an earlier allocation of this plan failed midway. Destroy the plan and create it again");
        if (p->cw > 1) {
            OXZ_TRY(comm_check(comm, "oxz_state_alloc"));
            if (comm->world != p->cw || comm->rank != p->cr)
                return fail(OXZ_ERR_INVALID, "oxz_state_alloc: the plan is rank %d of %d but the communicator is rank %d of %d",
                            p->cr, p->cw, comm->rank, comm->world);
        }
        OXZ_CUDA(cudaSetDevice(p->device));
        OXZ_TRY(query_geom(p->device, &p->geom));
        OXZ_CUDA(cudaStreamCreateWithFlags(&p->own_stream, cudaStreamNonBlocking));
        p->stream = p->own_stream;
        p->comm = comm;
        const uint64_t padded = p->total_tiles * TILE, local = p->local_tiles * TILE;
        const size_t gs = dtype_size(p->gdt), ps = dtype_size(p->pdt);
        auto zalloc = [](void** q, size_t bytes) -> cudaError_t {
            cudaError_t e = cudaMalloc(q, bytes ? bytes : 16);
            if (e != cudaSuccess) return e;
            return cudaMemset(*q, 0, bytes ? bytes : 16);
        };
        OXZ_CUDA(zalloc(&p->grads, padded * gs));
        OXZ_CUDA(zalloc((void**)&p->master, local * 4));
        OXZ_CUDA(zalloc((void**)&p->exp_avg, local * 4));
        OXZ_CUDA(zalloc((void**)&p->exp_avg_sq, local * 4));
        const bool separate_work = !(p->pdt == OXZ_F32 && p->world == 1);
        if (separate_work) OXZ_CUDA(zalloc(&p->work, padded * ps));
        else p->work = p->master;
        const bool peer_mode = p->mode == OXZ_SYNC_P2P || p->mode == OXZ_SYNC_COPY || p->mode == OXZ_SYNC_REPLICATED;
        if (p->cw > 1) OXZ_CUDA(zalloc(&p->reduced, local * (peer_mode ? 4 : gs)));
        OXZ_CUDA(zalloc((void**)&p->d_tile_meta, p->total_tiles * 4));
        OXZ_CUDA(cudaMemcpy(p->d_tile_meta, p->tile_meta.data(), p->total_tiles * 4, cudaMemcpyHostToDevice));
        OXZ_CUDA(zalloc((void**)&p->d_present, p->T));
        if (p->T) OXZ_CUDA(cudaMemset(p->d_present, 1, p->T));
        if (p->cw > 1) {
            OXZ_CUDA(zalloc((void**)&p->d_present_in, p->T));
            if (p->T) OXZ_CUDA(cudaMemset(p->d_present_in, 1, p->T));
        }
        OXZ_CUDA(zalloc((void**)&p->d_offsets, p->T * 8));
        OXZ_CUDA(zalloc((void**)&p->d_numel, p->T * 8));
        if (p->T) {
            OXZ_CUDA(cudaMemcpy(p->d_offsets, p->offset.data(), p->T * 8, cudaMemcpyHostToDevice));
            OXZ_CUDA(cudaMemcpy(p->d_numel, p->numel.data(), p->T * 8, cudaMemcpyHostToDevice));
        }
        OXZ_CUDA(zalloc((void**)&p->d_src, p->T * 8));
        OXZ_CUDA(zalloc((void**)&p->d_partials, (size_t)norm_partial_slots(p->geom) * 3 * 8 * MAX_PIPE));
        OXZ_CUDA(zalloc((void**)&p->d_acc, ACC_DOUBLES * 8));
        OXZ_CUDA(zalloc((void**)&p->d_scalars, sizeof(DevScalars)));
        OXZ_CUDA(cudaMallocHost((void**)&p->h_scalars, sizeof(DevScalars)));
        OXZ_CUDA(cudaMallocHost((void**)&p->h_acc, ACC_DOUBLES * 8));
        OXZ_CUDA(cudaMallocHost((void**)&p->h_extras, MAX_EXTRAS * 8));
        OXZ_CUDA(cudaMallocHost((void**)&p->h_present, p->T ? p->T : 1));
        OXZ_CUDA(cudaMallocHost((void**)&p->h_union, p->T ? p->T : 1));
        memset(p->h_union, 1, p->T ? p->T : 1);
        OXZ_CUDA(cudaMallocHost((void**)&p->h_src, (p->T ? p->T : 1) * 8));
        memset(p->h_present, 1, p->T ? p->T : 1);
        OXZ_CUDA(cudaEventCreateWithFlags(&p->done, cudaEventDisableTiming));
        // Exchanges between ranks through peer memory instead of small NCCL collectives: for the modes whose kernels
        // already address peer memory, behind an NCCL communicator (its ranks sit on distinct GPUs, so the waiting
        // kernels of different ranks never share one), when the flags of all tensors fit a slot. OXZ_MAIL=0 keeps NCCL.
        // By default up to four ranks, where the mailboxes were verified on real GPUs; OXZ_MAIL=1 asks for them at any
        // rank count (the kernels do not depend on it), OXZ_MAIL=0 never.
        const char* mail_env = getenv("OXZ_MAIL");
        const bool mail_on = mail_env ? atoi(mail_env) != 0 : p->cw <= 4;
        const bool want_mail = (p->mode == OXZ_SYNC_P2P || p->mode == OXZ_SYNC_REPLICATED) && p->cw > 1 && comm->kind == 0 &&
                               p->T <= MAIL_PAYLOAD && mail_on;
        if (want_mail) {
            static_assert(sizeof(MailBox) <= (2u << 20), "a mailbox fits its allocation");
            OXZ_CUDA(zalloc((void**)&p->mail, 2u << 20));  // an allocation of its own page size, shared with the peers
            const char* lim = getenv("OXZ_MAIL_TIMEOUT_MS");
            const double ms = lim ? atof(lim) : 30000.0;
            p->mail_limit_ns = (uint64_t)((ms > 0.0 ? ms : 30000.0) * 1e6);
        }
        OXZ_CUDA(cudaDeviceSynchronize());
        p->peers.grads[0] = p->grads;
        p->peers.work[0] = p->work;
        if (peer_mode) OXZ_TRY(exchange_peers(p, comm));
        p->own_work.work[0] = p->work;
        if (p->mode == OXZ_SYNC_COPY) {
            // one staging slot per peer, laid out like this rank's local state; the own slot is the gradient buffer itself
            OXZ_CUDA(zalloc(&p->stage, (size_t)(p->world - 1) * local * gs));
            int slot = 0;
            for (int r = 0; r < p->world; r++) {
                if (r == p->rank) {
                    p->staged_src.grads[r] = p->grads;
                } else {
                    p->staged_src.grads[r] = static_cast<char*>(p->stage) + (size_t)slot * local * gs;
                    slot++;
                }
                OXZ_CUDA(cudaStreamCreateWithFlags(&p->copy_stream[r], cudaStreamNonBlocking));
                OXZ_CUDA(cudaEventCreateWithFlags(&p->ev_pushed[r], cudaEventDisableTiming));
                for (uint32_t g = 0; g < MAX_PIPE; g++) OXZ_CUDA(cudaEventCreateWithFlags(&p->ev_copied[r][g], cudaEventDisableTiming));
            }
            OXZ_CUDA(cudaEventCreateWithFlags(&p->ev_go, cudaEventDisableTiming));
            for (uint32_t g = 0; g < MAX_PIPE; g++) OXZ_CUDA(cudaEventCreateWithFlags(&p->ev_updated[g], cudaEventDisableTiming));
            const char* e = getenv("OXZ_PIPE_GROUPS");
            uint32_t want = e ? (uint32_t)atoi(e) : 4;
            if (want < 1) want = 1;
            if (want > MAX_PIPE) want = MAX_PIPE;
            if (want > p->n_buckets) want = (uint32_t)p->n_buckets;
            p->pipe_groups = want;
        }
        p->allocated = true;
        return OXZ_OK;
    });
}

int32_t oxz_state_pointers(const oxz_plan* p, void** grads, void** work, void** master, void** exp_avg,
                           void** exp_avg_sq) {
    return oxz::guarded("oxz_state_pointers", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_state_pointers: null plan");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_state_pointers: call oxz_state_alloc first");
        if (grads) *grads = p->grads;
        if (work) *work = p->work;
        if (master) *master = p->master;
        if (exp_avg) *exp_avg = p->exp_avg;
        if (exp_avg_sq) *exp_avg_sq = p->exp_avg_sq;
        return OXZ_OK;
    });
}

int32_t oxz_state_import(oxz_plan* p, int32_t kind, uint64_t tensor, const void* host) {
    return oxz::guarded("oxz_state_import", [&]() -> int32_t {
        OXZ_TRY(check_state_call(p, kind, tensor, host, "oxz_state_import"));
        OXZ_CUDA(cudaSetDevice(p->device));
        OXZ_CUDA(cudaStreamSynchronize(p->stream));
        const uint64_t n = p->numel[tensor];
        if (kind == OXZ_STATE_GRADS || kind == OXZ_STATE_WORK) {
            const size_t es = dtype_size(kind == OXZ_STATE_GRADS ? p->gdt : p->pdt);
            char* base = static_cast<char*>(kind == OXZ_STATE_GRADS ? p->grads : p->work);
            if (kind == OXZ_STATE_WORK && p->work == (void*)p->master) kind = OXZ_STATE_MASTER;
            else {
                OXZ_CUDA(cudaMemcpy(base + p->offset[tensor] * es, host, n * es, cudaMemcpyHostToDevice));
                return OXZ_OK;
            }
        }
        float* arr = state_array(p, kind);
        cudaError_t err = cudaSuccess;
        for_owned_runs(p, tensor, [&](uint64_t flat, uint64_t local, uint64_t len) {
            if (err != cudaSuccess) return;
            err = cudaMemcpy(arr + local, static_cast<const float*>(host) + (flat - p->offset[tensor]), len * 4, cudaMemcpyHostToDevice);
        });
        if (err != cudaSuccess) return fail(OXZ_ERR_CUDA, "oxz_state_import: %s", cudaGetErrorString(err));
        return OXZ_OK;
    });
}

int32_t oxz_state_export(oxz_plan* p, int32_t kind, uint64_t tensor, void* host) {
    return oxz::guarded("oxz_state_export", [&]() -> int32_t {
        OXZ_TRY(check_state_call(p, kind, tensor, host, "oxz_state_export"));
        OXZ_CUDA(cudaSetDevice(p->device));
        OXZ_CUDA(cudaStreamSynchronize(p->stream));
        const uint64_t n = p->numel[tensor];
        if (kind == OXZ_STATE_GRADS || kind == OXZ_STATE_WORK) {
            const size_t es = dtype_size(kind == OXZ_STATE_GRADS ? p->gdt : p->pdt);
            const char* base = static_cast<const char*>(kind == OXZ_STATE_GRADS ? p->grads : p->work);
            if (kind == OXZ_STATE_WORK && p->work == (void*)p->master) kind = OXZ_STATE_MASTER;
            else {
                OXZ_CUDA(cudaMemcpy(host, base + p->offset[tensor] * es, n * es, cudaMemcpyDeviceToHost));
                return OXZ_OK;
            }
        }
        const float* arr = state_array(p, kind);
        cudaError_t err = cudaSuccess;
        for_owned_runs(p, tensor, [&](uint64_t flat, uint64_t local, uint64_t len) {
            if (err != cudaSuccess) return;
            err = cudaMemcpy(static_cast<float*>(host) + (flat - p->offset[tensor]), arr + local, len * 4, cudaMemcpyDeviceToHost);
        });
        if (err != cudaSuccess) return fail(OXZ_ERR_CUDA, "oxz_state_export: %s", cudaGetErrorString(err));
        return OXZ_OK;
    });
}

int32_t oxz_state_set_timestep(oxz_plan* p, uint64_t t) {
    return oxz::guarded("oxz_state_set_timestep", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_state_set_timestep: null plan");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_state_set_timestep: a step is in flight");
        p->timestep = t;
        return OXZ_OK;
    });
}

int32_t oxz_state_timestep(const oxz_plan* p, uint64_t* t) {
    return oxz::guarded("oxz_state_timestep", [&]() -> int32_t {
        if (!p || !t) return fail(OXZ_ERR_INVALID, "oxz_state_timestep: null argument");
        *t = p->timestep;
        return OXZ_OK;
    });
}

int32_t oxz_grads_flatten_async(oxz_plan* p, const void* const* grad_ptrs, int32_t accumulate) {
    return oxz::guarded("oxz_grads_flatten_async", [&]() -> int32_t {
        if (!p || !grad_ptrs) return fail(OXZ_ERR_INVALID, "oxz_grads_flatten_async: null argument");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_grads_flatten_async: call oxz_state_alloc first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_grads_flatten_async: a step is in flight. Call oxz_step_wait first");
        OXZ_CUDA(cudaSetDevice(p->device));
        for (uint64_t i = 0; i < p->T; i++) {
            if (grad_ptrs[i] && ((uintptr_t)grad_ptrs[i] & 15))
                return fail(OXZ_ERR_INVALID, "oxz_grads_flatten_async: the gradient of tensor %llu is not 16-byte aligned", (unsigned long long)i);
        }
        // The pointer table is staged in pinned memory; the previous use must have left the stream.
        OXZ_CUDA(cudaStreamSynchronize(p->stream));
        for (uint64_t i = 0; i < p->T; i++) p->h_src[i] = grad_ptrs[i];
        if (p->T) OXZ_CUDA(cudaMemcpyAsync(p->d_src, p->h_src, p->T * 8, cudaMemcpyHostToDevice, p->stream));
        return launch_flatten(p->stream, p->geom, p->grads, p->gdt, (uint32_t)p->total_tiles, p->d_tile_meta, p->d_offsets,
                              p->d_numel, p->d_src, accumulate);
    });
}

int32_t oxz_grads_upload_async(oxz_plan* p, uint64_t tensor, const void* host) {
    return oxz::guarded("oxz_grads_upload_async", [&]() -> int32_t {
        if (!p || !host) return fail(OXZ_ERR_INVALID, "oxz_grads_upload_async: null argument");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_grads_upload_async: call oxz_state_alloc first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_grads_upload_async: a step is in flight. Call oxz_step_wait first");
        if (tensor >= p->T) return fail(OXZ_ERR_INVALID, "oxz_grads_upload_async: tensor %llu of %llu", (unsigned long long)tensor, (unsigned long long)p->T);
        OXZ_CUDA(cudaSetDevice(p->device));
        const size_t es = dtype_size(p->gdt);
        OXZ_CUDA(cudaMemcpyAsync(static_cast<char*>(p->grads) + p->offset[tensor] * es, host, p->numel[tensor] * es,
                                 cudaMemcpyHostToDevice, p->stream));
        return OXZ_OK;
    });
}

int32_t oxz_grads_double_buffer(oxz_plan* p, oxz_comm* comm) {
    return oxz::guarded("oxz_grads_double_buffer", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_grads_double_buffer: null plan");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_grads_double_buffer: call oxz_state_alloc first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_grads_double_buffer: a step is in flight. Call oxz_step_wait first");
        if (p->double_buffered) return OXZ_OK;
        if (p->grads_alt) return fail(OXZ_ERR_STATE, "oxz_grads_double_buffer: an earlier call failed midway. Destroy the plan and create it again");
        if (p->mode == OXZ_SYNC_COPY) return fail(OXZ_ERR_UNSUPPORTED, "oxz_grads_double_buffer does not serve OXZ_SYNC_COPY plans");
        const bool peer_mode = p->mode == OXZ_SYNC_P2P || p->mode == OXZ_SYNC_REPLICATED;
        if (peer_mode) {
            OXZ_TRY(comm_check(comm, "oxz_grads_double_buffer"));
            if (comm != p->comm) return fail(OXZ_ERR_INVALID, "oxz_grads_double_buffer: this is not the communicator the state was allocated with");
        }
        OXZ_CUDA(cudaSetDevice(p->device));
        const size_t bytes = p->total_tiles * TILE * dtype_size(p->gdt);
        OXZ_CUDA(cudaMalloc(&p->grads_alt, bytes ? bytes : 16));
        OXZ_CUDA(cudaMemset(p->grads_alt, 0, bytes ? bytes : 16));
        OXZ_CUDA(cudaStreamCreateWithFlags(&p->upload_stream, cudaStreamNonBlocking));
        OXZ_CUDA(cudaEventCreateWithFlags(&p->ev_uploaded, cudaEventDisableTiming));
        for (auto& e : p->ev_last_read) OXZ_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        OXZ_CUDA(cudaDeviceSynchronize());
        if (peer_mode) OXZ_TRY(exchange_alt_grads(p, comm));
        p->double_buffered = true;
        return OXZ_OK;
    });
}

int32_t oxz_grads_upload_next_async(oxz_plan* p, uint64_t tensor, const void* host) {
    return oxz::guarded("oxz_grads_upload_next_async", [&]() -> int32_t {
        if (!p || !host) return fail(OXZ_ERR_INVALID, "oxz_grads_upload_next_async: null argument");
        if (!p->double_buffered) return fail(OXZ_ERR_STATE, "oxz_grads_upload_next_async: call oxz_grads_double_buffer first");
        if (tensor >= p->T) return fail(OXZ_ERR_INVALID, "oxz_grads_upload_next_async: tensor %llu of %llu", (unsigned long long)tensor, (unsigned long long)p->T);
        OXZ_CUDA(cudaSetDevice(p->device));
        // the step that last read the other buffer (and, with peers, whose end says that every rank has read it) must be over
        OXZ_CUDA(cudaStreamWaitEvent(p->upload_stream, p->ev_last_read[1 - p->cur_grads], 0));
        const size_t es = dtype_size(p->gdt);
        OXZ_CUDA(cudaMemcpyAsync(static_cast<char*>(p->grads_alt) + p->offset[tensor] * es, host, p->numel[tensor] * es,
                                 cudaMemcpyHostToDevice, p->upload_stream));
        return OXZ_OK;
    });
}

int32_t oxz_grads_swap(oxz_plan* p) {
    return oxz::guarded("oxz_grads_swap", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_grads_swap: null plan");
        if (!p->double_buffered) return fail(OXZ_ERR_STATE, "oxz_grads_swap: call oxz_grads_double_buffer first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_grads_swap: a step is in flight. Call oxz_step_wait first");
        if (p->early_groups) return fail(OXZ_ERR_STATE, "oxz_grads_swap: buckets of the current buffer were already handed in for this step");
        OXZ_CUDA(cudaSetDevice(p->device));
        OXZ_CUDA(cudaEventRecord(p->ev_uploaded, p->upload_stream));
        std::swap(p->grads, p->grads_alt);
        for (int r = 0; r < p->cw; r++) std::swap(p->peers.grads[r], p->peer_grads_alt[r]);
        p->cur_grads ^= 1;
        p->upload_pending = true;
        return OXZ_OK;
    });
}

namespace {

bool same_or_both_nan(double a, double b) { return a == b || (std::isnan(a) && std::isnan(b)); }

// Records which tensors have a gradient this step. With several ranks the flags the kernels read are the UNION over
// ranks: a tensor is left alone only when no rank produced a gradient for it (src/dp/reduce.rs:20); a rank without one
// contributes the zeros its gradient buffer holds there. A local group forms the union on the host; an NCCL group on
// the device, either here (a byte-wise maximum, which is also a barrier on `s`) or, when `by_gate`, in the opening
// gate kernel the caller launches next. *some_absent: whether the kernels must look the flags up. Where the host
// does not see the union it answers for this rank's own flags, which can only err towards looking them up.
int32_t sync_present(oxz_plan* p, oxz_comm* comm, const uint8_t* present, cudaStream_t s, bool by_gate, bool* some_absent) {
    bool changed = false, own_absent = false;
    for (uint64_t i = 0; i < p->T; i++) {
        const uint8_t v = present ? (present[i] ? 1 : 0) : 1;
        if (p->h_present[i] != v) {
            p->h_present[i] = v;
            changed = true;
        }
        own_absent |= v == 0;
    }
    *some_absent = own_absent;
    if (p->cw == 1) {
        if (changed) OXZ_CUDA(cudaMemcpyAsync(p->d_present, p->h_present, p->T, cudaMemcpyHostToDevice, s));
        return OXZ_OK;
    }
    if (changed) OXZ_CUDA(cudaMemcpyAsync(p->d_present_in, p->h_present, p->T, cudaMemcpyHostToDevice, s));
    if (comm->kind != 1 && by_gate) return OXZ_OK;
    memcpy(p->h_union, p->h_present, p->T);
    bool host_known = false;
    OXZ_TRY(comm_present_union(comm, p->h_union, p->d_present_in, p->d_present, p->T, s, &host_known));
    if (host_known) {
        if (p->T) OXZ_CUDA(cudaMemcpyAsync(p->d_present, p->h_union, p->T, cudaMemcpyHostToDevice, s));
        *some_absent = false;
        for (uint64_t i = 0; i < p->T; i++) *some_absent |= p->h_union[i] == 0;
    }
    return OXZ_OK;
}

// An exchange through the mailboxes used as a barrier; with `carry_present` it also forms the union of the flags.
int32_t mail_gate(oxz_plan* p, oxz_comm* comm, cudaStream_t s, bool carry_present) {
    return launch_gate(s, p->mail_peers, p->cw, p->cr, ++p->mail_seq, p->d_present_in, p->d_present,
                       carry_present ? (uint32_t)p->T : 0u, p->d_scalars, p->mail_limit_ns, comm->h_abort_flag);
}

// The norm pass (fused with the pull over ranks in P2P mode) over buckets [b0, b1) into partial-sum group `group`.
int32_t reduce_buckets(oxz_plan* p, cudaStream_t s, const LaunchGeom& geom, uint64_t b0, uint64_t b1, uint32_t group,
                       uint32_t slots, bool some_absent, float inv_scale, float clamp_hi, int32_t clamp_on) {
    TileMap gm = tile_map(p);
    group_tiles(p, b0, b1, &gm.first_tile, &gm.n_local_tiles);
    double* partials = p->d_partials + (size_t)group * slots * 3;
    if (p->mode == OXZ_SYNC_SINGLE)
        return launch_sumsq(s, geom, p->grads, p->gdt, gm, p->d_tile_meta, p->d_present, some_absent, inv_scale, clamp_hi,
                            clamp_on, partials);
    // The bulk-copy form of the pull where the shape allows it (measured on two B200: 1.85 ms against 1.96 ms for
    // 1.24 G bf16 gradients); OXZ_PULL_BULK=0 keeps the per-lane loads.
    const char* bulk_env = getenv("OXZ_PULL_BULK");
    const bool want_bulk = !bulk_env || atoi(bulk_env) != 0;
    if (want_bulk && pull_bulk_fits(gm, p->cw, p->gdt)) {
        // its grid is smaller than the group's slot count: the slots it does not write must read as zero
        OXZ_CUDA(cudaMemsetAsync(partials, 0, (size_t)slots * 3 * 8, s));
        p->last_pull_kernel = OXZ_PULL_KERNEL_BULK;
        return launch_pull_bulk(s, geom, p->peers, p->cw, p->gdt, gm, p->d_tile_meta, p->d_present, some_absent, inv_scale,
                                clamp_hi, clamp_on, static_cast<float*>(p->reduced), partials, slots, p->d_scalars);
    }
    p->last_pull_kernel = OXZ_PULL_KERNEL_LOADS;
    return launch_pull_sumsq(s, geom, p->peers, p->cw, 0, p->gdt, gm, p->d_tile_meta, p->d_present, some_absent,
                             inv_scale, clamp_hi, clamp_on, static_cast<float*>(p->reduced), partials);
}

}  // namespace

static int32_t check_hyper(const oxz_hyper* h) {
    auto pos = [](double x) { return std::isfinite(x) && x > 0.0; };
    if (!std::isfinite(h->lr) || h->lr < 0.0) return fail(OXZ_ERR_INVALID, "learning rate %g must be finite and not negative", h->lr);
    if (!(h->beta1 >= 0.0 && h->beta1 < 1.0) || !(h->beta2 >= 0.0 && h->beta2 < 1.0))
        return fail(OXZ_ERR_INVALID, "adamw betas (%g, %g) must lie in [0, 1)", h->beta1, h->beta2);
    if (!std::isfinite(h->eps) || h->eps < 0.0) return fail(OXZ_ERR_INVALID, "adamw_eps %g must be finite and not negative", h->eps);
    if (!std::isfinite(h->weight_decay)) return fail(OXZ_ERR_INVALID, "weight_decay %g must be finite", h->weight_decay);
    if (std::isnan(h->max_grad_norm) || h->max_grad_norm <= 0.0) return fail(OXZ_ERR_INVALID, "max_grad_norm %g must be positive", h->max_grad_norm);
    // check_max_grad_value, src/grad_clip.rs:18-26
    if (!std::isnan(h->max_grad_value) && !pos(h->max_grad_value))
        return fail(OXZ_ERR_INVALID, "trainer.max_grad_value is %g: it must be a finite positive number. Set a positive value, or remove the key to disable per-element clipping.", h->max_grad_value);
    if (!std::isnan(h->target_grad_norm) && !pos(h->target_grad_norm))
        return fail(OXZ_ERR_INVALID, "target_grad_norm %g must be finite and positive", h->target_grad_norm);
    if (!std::isnan(h->loss_scale) && h->loss_scale != 0.0 && !pos(h->loss_scale))
        return fail(OXZ_ERR_INVALID, "loss scale %g must be finite and positive", h->loss_scale);
    if (!std::isfinite(h->clip_eps) || h->clip_eps < 0.0) return fail(OXZ_ERR_INVALID, "clip_eps %g must be finite and not negative", h->clip_eps);
    return OXZ_OK;
}

int32_t oxz_step_async(oxz_plan* p, oxz_comm* comm, const oxz_hyper* h, const uint8_t* present, double* extras,
                       uint32_t n_extras) {
    return oxz::guarded("oxz_step_async", [&]() -> int32_t {
        if (!p || !h) return fail(OXZ_ERR_INVALID, "oxz_step_async: null argument");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_step_async: the plan has no device state. Call oxz_state_alloc first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_step_async: the previous step is still in flight. Call oxz_step_wait first");
        if (n_extras > MAX_EXTRAS || (n_extras && !extras)) return fail(OXZ_ERR_INVALID, "oxz_step_async: at most %u extras", MAX_EXTRAS);
        OXZ_TRY(check_hyper(h));
        if (p->cw > 1) {
            OXZ_TRY(comm_check(comm, "oxz_step_async"));
            if (comm != p->comm) return fail(OXZ_ERR_INVALID, "oxz_step_async: this is not the communicator the state was allocated with");
        }
        OXZ_CUDA(cudaSetDevice(p->device));
        cudaStream_t s = p->stream;
        const bool nccl_mode = p->mode == OXZ_SYNC_NCCL;
        if (nccl_mode && comm->kind != 0)
            return fail(OXZ_ERR_UNSUPPORTED, "OXZ_SYNC_NCCL needs an NCCL communicator; a local group serves OXZ_SYNC_P2P");
        const NcclApi* api = nccl_mode ? nccl_api() : nullptr;
        ncclComm_t nc = nccl_mode ? (ncclComm_t)comm->nccl : nullptr;

        // which tensors have a gradient this step
        bool some_absent = false;
        // the opening gate of the pulling modes carries the flags itself when the ranks meet through the mailboxes
        const bool gate_carries = p->use_mail;
        // with NCCL the union of the flags, formed on `s` just below, is a barrier over the ranks' streams already
        const bool flags_were_barrier = p->cw > 1 && comm->kind == 0 && !gate_carries && p->early_groups == 0 && p->T > 0;
        if (p->early_groups == 0) {
            OXZ_TRY(sync_present(p, comm, present, s, gate_carries, &some_absent));
        } else {
            for (uint64_t i = 0; i < p->T; i++) {
                const uint8_t v = present ? (present[i] ? 1 : 0) : 1;
                if (p->h_present[i] != v) return fail(OXZ_ERR_INVALID, "oxz_step_async: `present` differs from the one oxz_grads_ready_async was given for this step");
                some_absent |= (p->cw > 1 && comm->kind == 1 ? p->h_union[i] : v) == 0;
            }
            if (!same_or_both_nan(h->loss_scale, p->early_scale) || !same_or_both_nan(h->max_grad_value, p->early_clamp))
                return fail(OXZ_ERR_INVALID, "oxz_step_async: loss_scale or max_grad_value differs from the one oxz_grads_ready_async was given for this step");
        }

        // per-step scalars, f64 on the host, rounded to f32 once
        const uint64_t t = p->timestep + 1;
        const bool scaled = !std::isnan(h->loss_scale) && h->loss_scale != 0.0;
        AdamParams ap{};
        const double bc1 = 1.0 - std::pow(h->beta1, (double)t), bc2 = 1.0 - std::pow(h->beta2, (double)t);
        ap.beta1 = (float)h->beta1;
        ap.one_minus_beta1 = (float)(1.0 - h->beta1);
        ap.beta2 = (float)h->beta2;
        ap.one_minus_beta2 = (float)(1.0 - h->beta2);
        ap.eps = (float)h->eps;
        ap.bias2_sqrt = (float)std::sqrt(bc2);
        ap.inv_scale = scaled ? (float)(1.0 / h->loss_scale) : 1.0f;
        ap.clamp_on = std::isnan(h->max_grad_value) ? 0 : 1;
        ap.clamp_hi = ap.clamp_on ? (float)h->max_grad_value : 0.f;
        ap.decay_after = h->decay_after ? 1 : 0;
        ap.eps_mode = h->eps_mode ? 1 : 0;
        if (const char* e = getenv("OXZ_PUSH_HINT")) ap.push_hint = atoi(e);  // tuning aid
        for (size_t g = 0; g < p->group_lr_scale.size(); g++) {
            const double lr_t = h->lr * (double)p->group_lr_scale[g];
            const double wd = p->group_no_decay[g] ? 0.0 : h->weight_decay;
            ap.step_size[g] = ap.eps_mode == 0 ? (float)(lr_t / bc1) : (float)(lr_t * std::sqrt(bc2) / bc1);
            ap.decay_mul[g] = (float)(1.0 - lr_t * wd);
        }
        FinalizeParams fp{};
        fp.max_grad_norm = h->max_grad_norm;
        fp.has_target = std::isnan(h->target_grad_norm) ? 0 : 1;
        fp.target_grad_norm = fp.has_target ? h->target_grad_norm : 0.0;
        fp.clip_eps = h->clip_eps;
        fp.spike_skip = h->spike_skip ? 1 : 0;

        const TileMap map = tile_map(p);
        const bool replicated = p->mode == OXZ_SYNC_REPLICATED;
        const bool pulls = p->mode == OXZ_SYNC_P2P || replicated;  // the gradient sum is the fused pull kernel
        const bool peer_mode = pulls || p->mode == OXZ_SYNC_COPY;
        uint32_t slots = peer_mode ? pull_partial_slots(p->geom, p->gdt) : norm_partial_slots(p->geom);
        const void* gsrc = p->grads;
        int32_t gsrc_dt = p->gdt;
        int32_t* bar = p->cw > 1 ? reinterpret_cast<int32_t*>(static_cast<char*>(comm->d_small) + 384) : nullptr;

        auto mark = [&](int i) -> cudaError_t { return p->profile ? cudaEventRecord(p->ev[i], s) : cudaSuccess; };
        if (p->upload_pending) {
            // gradients copied into this buffer while the step before was still running
            OXZ_CUDA(cudaStreamWaitEvent(s, p->ev_uploaded, 0));
            p->upload_pending = false;
        }
        OXZ_CUDA(mark(0));
        if (p->mode == OXZ_SYNC_SINGLE || pulls) {
            // buckets already reduced during backward are skipped; the rest goes now, one launch per run of buckets
            uint32_t groups = p->early_groups;
            if (groups) OXZ_CUDA(cudaStreamWaitEvent(s, p->ev_early, 0));
            bool any_left = false;
            for (uint64_t b = 0; b < p->n_buckets; b++) any_left |= !(groups && p->early_done[b]);
            // every rank's remaining gradients must be complete before anyone pulls them
            if (pulls && any_left) {
                if (p->use_mail) OXZ_TRY(mail_gate(p, comm, s, true));
                else if (!flags_were_barrier) OXZ_TRY(comm_stream_barrier(comm, bar, s));
            }
            OXZ_CUDA(mark(1));
            for (uint64_t b = 0; b < p->n_buckets;) {
                if (groups && p->early_done[b]) { b++; continue; }
                uint64_t e = b;
                while (e < p->n_buckets && !(p->early_groups && p->early_done[e])) e++;
                if (groups >= MAX_PIPE) return fail(OXZ_ERR_STATE, "oxz_step_async: the buckets left after oxz_grads_ready_async form too many separate runs");
                OXZ_TRY(reduce_buckets(p, s, p->geom, b, e, groups, slots, some_absent, ap.inv_scale, ap.clamp_hi, ap.clamp_on));
                groups++;
                b = e;
            }
            slots *= groups;
            p->early_groups = 0;
            if (pulls) {
                gsrc = p->reduced;
                gsrc_dt = OXZ_F32;
            }
        } else if (p->mode == OXZ_SYNC_COPY) {
            // every rank's gradients must be complete before anyone copies them
            if (!flags_were_barrier) OXZ_TRY(comm_stream_barrier(comm, bar, s));
            OXZ_CUDA(mark(1));
            OXZ_CUDA(cudaEventRecord(p->ev_go, s));
            const size_t gs = dtype_size(p->gdt);
            const uint32_t G = p->pipe_groups;
            for (int r = 0; r < p->world; r++)
                if (r != p->rank) OXZ_CUDA(cudaStreamWaitEvent(p->copy_stream[r], p->ev_go, 0));
            for (uint32_t g = 0; g < G; g++) {
                uint64_t b0, b1;
                group_buckets(p, g, &b0, &b1);
                for (int r = 0; r < p->world; r++) {
                    if (r == p->rank) continue;
                    // the peer's slices of this rank's shard, buckets [b0, b1): a strided read, packed into the slot
                    OXZ_TRY(copy_shard_rows(p, static_cast<char*>(const_cast<void*>(p->staged_src.grads[r])), true,
                                            static_cast<const char*>(p->peers.grads[r]), false, gs, b0, b1, p->copy_stream[r]));
                    OXZ_CUDA(cudaEventRecord(p->ev_copied[r][g], p->copy_stream[r]));
                }
                for (int r = 0; r < p->world; r++)
                    if (r != p->rank) OXZ_CUDA(cudaStreamWaitEvent(s, p->ev_copied[r][g], 0));
                TileMap gm = map;
                group_tiles(p, b0, b1, &gm.first_tile, &gm.n_local_tiles);
                OXZ_TRY(launch_pull_sumsq(s, p->geom, p->staged_src, p->world, 1, p->gdt, gm, p->d_tile_meta, p->d_present, some_absent,
                                          ap.inv_scale, ap.clamp_hi, ap.clamp_on, static_cast<float*>(p->reduced),
                                          p->d_partials + (size_t)g * slots * 3));
            }
            slots *= G;
            gsrc = p->reduced;
            gsrc_dt = OXZ_F32;
        } else {
            const size_t gs = dtype_size(p->gdt);
            ncclResult_t rc = api->GroupStart();
            if (rc != ncclSuccess) return nccl_fail("ncclGroupStart", rc);
            for (uint64_t b = 0; b < p->n_buckets; b++) {
                uint64_t start, len, ss, sl;
                oxz_plan_bucket(p, b, p->rank, &start, &len, &ss, &sl);
                const uint64_t local = b * (p->bucket_tiles / (uint64_t)p->world) * TILE;
                rc = api->ReduceScatter(static_cast<const char*>(p->grads) + start * gs, static_cast<char*>(p->reduced) + local * gs,
                                        sl, nccl_dtype(p->gdt), ncclSum, nc, s);
                if (rc != ncclSuccess) return nccl_fail("the gradient reduce-scatter", rc);
            }
            rc = api->GroupEnd();
            if (rc != ncclSuccess) return nccl_fail("the gradient reduce-scatter", rc);
            OXZ_CUDA(mark(1));
            OXZ_TRY(launch_sumsq(s, p->geom, p->reduced, p->gdt, map, p->d_tile_meta, p->d_present, some_absent, ap.inv_scale,
                                 ap.clamp_hi, ap.clamp_on, p->d_partials));
            gsrc = p->reduced;
        }
        OXZ_CUDA(mark(2));
        if (p->cw > 1) {
            for (uint32_t i = 0; i < n_extras; i++) p->h_extras[i] = extras[i];
            if (n_extras) OXZ_CUDA(cudaMemcpyAsync(p->d_acc + ACC_EXTRAS, p->h_extras, n_extras * 8, cudaMemcpyHostToDevice, s));
        }
        // The one data exchange of the step: {sum of squares, inf count, NaN count, a wait ran out, extras...}. In P2P
        // mode its end also tells every rank that all peers have finished reading its gradient buffer. A full replica
        // has measured every element itself: only the run-out flag and the extras are summed.
        if (p->cw > 1 && p->use_mail) {
            OXZ_TRY(launch_decide(s, p->mail_peers, p->cw, p->cr, ++p->mail_seq, p->d_partials, slots, p->d_acc, n_extras,
                                  replicated ? 0 : 1, fp, p->d_scalars, p->mail_limit_ns, comm->h_abort_flag));
        } else {
            OXZ_TRY(launch_reduce_partials(s, p->d_partials, slots, p->d_acc, p->d_scalars));
            if (p->cw > 1) {
                if (!replicated) OXZ_TRY(comm_stream_allreduce_f64(comm, p->d_acc, ACC_EXTRAS + n_extras, p->h_acc, s));
                else OXZ_TRY(comm_stream_allreduce_f64(comm, p->d_acc + ACC_EXPIRED, 1 + n_extras, p->h_acc + ACC_EXPIRED, s));
            }
            OXZ_TRY(launch_finalize(s, p->d_acc, fp, p->d_scalars));
        }
        OXZ_CUDA(cudaMemcpyAsync(p->h_scalars, p->d_scalars, sizeof(DevScalars), cudaMemcpyDeviceToHost, s));
        // the pull kernels (also those of buckets reduced ahead of the next step) raise this flag; it was just copied out
        // with the rest and starts the next step cleared
        OXZ_CUDA(cudaMemsetAsync(&p->d_scalars->wait_expired, 0, sizeof(int32_t), s));
        if (p->cw > 1 && n_extras)
            OXZ_CUDA(cudaMemcpyAsync(p->h_acc, p->d_acc, (ACC_EXTRAS + n_extras) * 8, cudaMemcpyDeviceToHost, s));

        OXZ_CUDA(mark(3));
        const bool separate_work = p->work != (void*)p->master;
        const int32_t n_work = !separate_work ? 0 : (p->mode == OXZ_SYNC_P2P ? p->world : 1);
        if (p->mode == OXZ_SYNC_COPY) {
            // the update runs group by group; as soon as a group's weights are written the copy engines push them to
            // every peer while the next group updates
            const size_t ps = dtype_size(p->pdt);
            PeerTable own{};
            own.work[0] = p->work;
            for (uint32_t g = 0; g < p->pipe_groups; g++) {
                uint64_t b0, b1;
                group_buckets(p, g, &b0, &b1);
                TileMap gm = map;
                group_tiles(p, b0, b1, &gm.first_tile, &gm.n_local_tiles);
                OXZ_TRY(launch_adamw(s, p->geom, gsrc, gsrc_dt, p->master, p->exp_avg, p->exp_avg_sq, own, 1, p->pdt, gm,
                                     p->d_tile_meta, p->d_present, some_absent, p->d_scalars, ap));
                OXZ_CUDA(cudaEventRecord(p->ev_updated[g], s));
                for (int r = 0; r < p->world; r++) {
                    if (r == p->rank) continue;
                    OXZ_CUDA(cudaStreamWaitEvent(p->copy_stream[r], p->ev_updated[g], 0));
                    OXZ_TRY(copy_shard_rows(p, static_cast<char*>(p->peers.work[r]), false, static_cast<const char*>(p->work), false,
                                            ps, b0, b1, p->copy_stream[r]));
                }
            }
            OXZ_CUDA(mark(4));
            for (int r = 0; r < p->world; r++) {
                if (r == p->rank) continue;
                OXZ_CUDA(cudaEventRecord(p->ev_pushed[r], p->copy_stream[r]));
                OXZ_CUDA(cudaStreamWaitEvent(s, p->ev_pushed[r], 0));
            }
            // every rank's copies into this rank's weight buffer must have landed before the step is reported done
            OXZ_TRY(comm_stream_barrier(comm, bar, s));
        } else {
            // p->peers lists the communicator's ranks; a full replica writes only its own weights
            OXZ_TRY(launch_adamw(s, p->geom, gsrc, gsrc_dt, p->master, p->exp_avg, p->exp_avg_sq, replicated ? p->own_work : p->peers,
                                 n_work, p->pdt, map, p->d_tile_meta, p->d_present, some_absent, p->d_scalars, ap));
            OXZ_CUDA(mark(4));
        }
        p->last_update_kernel = last_update_kernel();
        if (p->mode == OXZ_SYNC_NCCL) {
            const size_t ps = dtype_size(p->pdt);
            ncclResult_t rc = api->GroupStart();
            if (rc != ncclSuccess) return nccl_fail("ncclGroupStart", rc);
            for (uint64_t b = 0; b < p->n_buckets; b++) {
                uint64_t start, len, ss, sl;
                oxz_plan_bucket(p, b, p->rank, &start, &len, &ss, &sl);
                rc = api->AllGather(static_cast<const char*>(p->work) + ss * ps, static_cast<char*>(p->work) + start * ps, sl * ps,
                                    ncclInt8, nc, s);
                if (rc != ncclSuccess) return nccl_fail("the weight all-gather", rc);
            }
            rc = api->GroupEnd();
            if (rc != ncclSuccess) return nccl_fail("the weight all-gather", rc);
        } else if (p->mode == OXZ_SYNC_P2P) {
            // every rank's stores into this rank's weight buffer must have landed before the step is reported done
            if (p->use_mail) OXZ_TRY(mail_gate(p, comm, s, false));
            else OXZ_TRY(comm_stream_barrier(comm, bar, s));
        }
        OXZ_CUDA(mark(5));
        if (p->double_buffered) OXZ_CUDA(cudaEventRecord(p->ev_last_read[p->cur_grads], s));
        OXZ_CUDA(cudaEventRecord(p->done, s));
        p->inflight = true;
        p->inflight_hyper = *h;
        p->inflight_extras = extras;
        p->inflight_n_extras = n_extras;
        return OXZ_OK;
    });
}

int32_t oxz_grads_ready_async(oxz_plan* p, oxz_comm* comm, const oxz_hyper* h, const uint8_t* present, uint64_t first_bucket,
                              uint64_t n_buckets, void* producer_stream) {
    return oxz::guarded("oxz_grads_ready_async", [&]() -> int32_t {
        if (!p || !h) return fail(OXZ_ERR_INVALID, "oxz_grads_ready_async: null argument");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_grads_ready_async: the plan has no device state. Call oxz_state_alloc first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_grads_ready_async: the previous step is still in flight. Call oxz_step_wait first");
        if (p->mode != OXZ_SYNC_SINGLE && p->mode != OXZ_SYNC_P2P)
            return fail(OXZ_ERR_UNSUPPORTED, "oxz_grads_ready_async serves OXZ_SYNC_SINGLE and OXZ_SYNC_P2P plans");
        OXZ_TRY(check_hyper(h));
        if (n_buckets == 0 || first_bucket + n_buckets > p->n_buckets)
            return fail(OXZ_ERR_INVALID, "oxz_grads_ready_async: buckets [%llu, %llu) of %llu", (unsigned long long)first_bucket,
                        (unsigned long long)(first_bucket + n_buckets), (unsigned long long)p->n_buckets);
        if (p->early_groups >= MAX_PIPE - 2) return fail(OXZ_ERR_STATE, "oxz_grads_ready_async: at most %u calls per step", MAX_PIPE - 2);
        if (p->cw > 1) {
            OXZ_TRY(comm_check(comm, "oxz_grads_ready_async"));
            if (comm != p->comm) return fail(OXZ_ERR_INVALID, "oxz_grads_ready_async: this is not the communicator the state was allocated with");
        }
        OXZ_CUDA(cudaSetDevice(p->device));
        if (!p->early_stream) {
            OXZ_CUDA(cudaStreamCreateWithFlags(&p->early_stream, cudaStreamNonBlocking));
            OXZ_CUDA(cudaEventCreateWithFlags(&p->ev_produced, cudaEventDisableTiming));
            OXZ_CUDA(cudaEventCreateWithFlags(&p->ev_early, cudaEventDisableTiming));
        }
        cudaStream_t es = p->early_stream;
        if (p->upload_pending) OXZ_CUDA(cudaStreamWaitEvent(es, p->ev_uploaded, 0));  // the buckets may have come from the host
        bool some_absent = false;
        if (p->early_groups == 0) {
            p->early_done.assign(p->n_buckets, 0);
            p->early_scale = h->loss_scale;
            p->early_clamp = h->max_grad_value;
            // the side stream must not run ahead of the previous step's update, which read the same buffers
            OXZ_CUDA(cudaEventRecord(p->ev_early, p->stream));
            OXZ_CUDA(cudaStreamWaitEvent(es, p->ev_early, 0));
            OXZ_TRY(sync_present(p, comm, present, es, false, &some_absent));
        } else {
            if (!same_or_both_nan(h->loss_scale, p->early_scale) || !same_or_both_nan(h->max_grad_value, p->early_clamp))
                return fail(OXZ_ERR_INVALID, "oxz_grads_ready_async: loss_scale or max_grad_value changed within one step");
            for (uint64_t i = 0; i < p->T; i++) {
                const uint8_t v = present ? (present[i] ? 1 : 0) : 1;
                if (p->h_present[i] != v) return fail(OXZ_ERR_INVALID, "oxz_grads_ready_async: `present` changed within one step");
                some_absent |= (p->cw > 1 && comm->kind == 1 ? p->h_union[i] : v) == 0;
            }
        }
        for (uint64_t b = first_bucket; b < first_bucket + n_buckets; b++)
            if (p->early_done[b]) return fail(OXZ_ERR_INVALID, "oxz_grads_ready_async: bucket %llu was already handed in this step", (unsigned long long)b);
        // the producer's work so far must have finished before the buckets are read
        OXZ_CUDA(cudaEventRecord(p->ev_produced, (cudaStream_t)producer_stream));
        OXZ_CUDA(cudaStreamWaitEvent(es, p->ev_produced, 0));
        if (p->mode == OXZ_SYNC_P2P) {
            int32_t* bar = reinterpret_cast<int32_t*>(static_cast<char*>(comm->d_small) + 448);
            OXZ_TRY(comm_stream_barrier(comm, bar, es));
        }
        const bool scaled = !std::isnan(h->loss_scale) && h->loss_scale != 0.0;
        const int32_t clamp_on = std::isnan(h->max_grad_value) ? 0 : 1;
        // a quarter of the usual grid: the pull is NVLink-bound and backward still needs the SMs
        LaunchGeom geom = p->geom;
        const int cap = (geom.sm_count / 4) * 4;
        geom.norm_blocks = geom.norm_blocks < cap ? geom.norm_blocks : cap;
        for (int& b : geom.pull_blocks) b = b < cap ? b : cap;
        for (int& b : geom.bulk_blocks) b = b < cap ? b : cap;
        const uint32_t slots = p->mode == OXZ_SYNC_P2P ? pull_partial_slots(p->geom, p->gdt) : norm_partial_slots(p->geom);
        // the smaller grid fills only the first slots of its group; the rest must read as zero
        OXZ_CUDA(cudaMemsetAsync(p->d_partials + (size_t)p->early_groups * slots * 3, 0, (size_t)slots * 3 * 8, es));
        OXZ_TRY(reduce_buckets(p, es, geom, first_bucket, first_bucket + n_buckets, p->early_groups, slots, some_absent,
                               scaled ? (float)(1.0 / h->loss_scale) : 1.0f, clamp_on ? (float)h->max_grad_value : 0.f, clamp_on));
        OXZ_CUDA(cudaEventRecord(p->ev_early, es));
        for (uint64_t b = first_bucket; b < first_bucket + n_buckets; b++) p->early_done[b] = 1;
        p->early_groups++;
        return OXZ_OK;
    });
}

int32_t oxz_step_wait(oxz_plan* p, oxz_step_result* res) {
    return oxz::guarded("oxz_step_wait", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_step_wait: null plan");
        if (!p->inflight) return fail(OXZ_ERR_STATE, "oxz_step_wait: no step is in flight");
        OXZ_CUDA(cudaSetDevice(p->device));
        cudaError_t e = cudaEventSynchronize(p->done);
        p->inflight = false;
        if (p->comm && p->comm->aborted.load()) return fail(OXZ_ERR_ABORTED, "oxz_step_wait: the communicator was aborted during the step");
        if (e != cudaSuccess) return fail(OXZ_ERR_CUDA, "oxz_step_wait: %s", cudaGetErrorString(e));
        const DevScalars& d = *p->h_scalars;
        if (d.wait_expired == 2)
            return fail(OXZ_ERR_ABORTED, "oxz_step_wait: the communicator was aborted while a kernel of the step waited for the other ranks; nothing was updated");
        if (d.wait_expired)
            return fail(OXZ_ERR_TIMEOUT, "oxz_step_wait: a bounded wait inside a kernel of the step ran out, on this rank or another, before a peer's "
                                         "data or arrival was seen; nothing was updated on any rank that reports this. Abort the group");
        const oxz_hyper& h = p->inflight_hyper;
        const bool applied = !d.skip;
        if (applied) p->timestep += 1;
        if (p->cw > 1)
            for (uint32_t i = 0; i < p->inflight_n_extras; i++) p->inflight_extras[i] = p->h_acc[ACC_EXTRAS + i];
        if (res) {
            res->grad_norm = d.norm;
            res->overflow = d.overflow;
            res->applied = applied ? 1 : 0;
            res->timestep = p->timestep;
            res->clip_coef = (double)d.c1 * (double)d.c2;
            double rep = d.norm;
            if (applied) {
                rep = d.norm < h.max_grad_norm ? d.norm : h.max_grad_norm;
                if (!std::isnan(h.target_grad_norm) && h.target_grad_norm < rep) rep = h.target_grad_norm;
            }
            res->reported_norm = rep;
        }
        return OXZ_OK;
    });
}

int32_t oxz_plan_launch_geometry(const oxz_plan* p, int32_t* sm_count, int32_t* norm_blocks, int32_t* update_blocks) {
    return oxz::guarded("oxz_plan_launch_geometry", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_plan_launch_geometry: null plan");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_plan_launch_geometry: call oxz_state_alloc first");
        if (sm_count) *sm_count = p->geom.sm_count;
        if (norm_blocks) *norm_blocks = p->geom.norm_blocks;
        if (update_blocks) *update_blocks = p->geom.adam_blocks;
        return OXZ_OK;
    });
}

int32_t oxz_plan_last_pull_kernel(const oxz_plan* p, int32_t* kind) {
    return oxz::guarded("oxz_plan_last_pull_kernel", [&]() -> int32_t {
        if (!p || !kind) return fail(OXZ_ERR_INVALID, "oxz_plan_last_pull_kernel: null argument");
        *kind = p->last_pull_kernel;
        return OXZ_OK;
    });
}

int32_t oxz_plan_last_update_kernel(const oxz_plan* p, int32_t* kind) {
    return oxz::guarded("oxz_plan_last_update_kernel", [&]() -> int32_t {
        if (!p || !kind) return fail(OXZ_ERR_INVALID, "oxz_plan_last_update_kernel: null argument");
        *kind = p->last_update_kernel;
        return OXZ_OK;
    });
}

int32_t oxz_plan_exchange_kind(const oxz_plan* p, int32_t* kind) {
    return oxz::guarded("oxz_plan_exchange_kind", [&]() -> int32_t {
        if (!p || !kind) return fail(OXZ_ERR_INVALID, "oxz_plan_exchange_kind: null argument");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_plan_exchange_kind: call oxz_state_alloc first");
        *kind = p->cw <= 1 ? OXZ_EXCHANGE_NONE : p->use_mail ? OXZ_EXCHANGE_MAILBOX : OXZ_EXCHANGE_COMM;
        return OXZ_OK;
    });
}

int32_t oxz_selftest_bounded_wait(int32_t device, uint32_t limit_ms, int32_t* outcome) {
    return oxz::guarded("oxz_selftest_bounded_wait", [&]() -> int32_t {
        if (!outcome) return fail(OXZ_ERR_INVALID, "oxz_selftest_bounded_wait: null argument");
        if (limit_ms == 0 || limit_ms > 2000) return fail(OXZ_ERR_INVALID, "oxz_selftest_bounded_wait: limit_ms %u is outside [1, 2000]", limit_ms);
        OXZ_CUDA(cudaSetDevice(device));
        // two mailboxes in this device's memory: "mine", and one standing for a second rank that never runs, so nothing
        // ever posts that rank's arrival in mine and the wait for it runs into its limit
        MailBox* boxes = nullptr;
        DevScalars* d_sc = nullptr;
        DevScalars h_sc{};
        OXZ_CUDA(cudaMalloc((void**)&boxes, 2 * sizeof(MailBox)));
        cudaError_t e = cudaMalloc((void**)&d_sc, sizeof(DevScalars));
        if (e != cudaSuccess) {
            cudaFree(boxes);
            return fail(OXZ_ERR_CUDA, "oxz_selftest_bounded_wait: %s", cudaGetErrorString(e));
        }
        auto finish = [&](int32_t status) {
            cudaFree(boxes);
            cudaFree(d_sc);
            return status;
        };
        if (cudaMemset(boxes, 0, 2 * sizeof(MailBox)) != cudaSuccess || cudaMemset(d_sc, 0, sizeof(DevScalars)) != cudaSuccess)
            return finish(fail(OXZ_ERR_CUDA, "oxz_selftest_bounded_wait: cudaMemset failed"));
        MailPeers two{};
        two.box[0] = boxes;
        two.box[1] = boxes + 1;
        int32_t st = launch_gate(nullptr, two, 2, 0, 1, nullptr, nullptr, 0, d_sc, (uint64_t)limit_ms * 1000000ull, nullptr);
        if (st != OXZ_OK) return finish(st);
        if (cudaMemcpy(&h_sc, d_sc, sizeof(DevScalars), cudaMemcpyDeviceToHost) != cudaSuccess)
            return finish(fail(OXZ_ERR_CUDA, "oxz_selftest_bounded_wait: the context did not survive the wait that ran out"));
        *outcome = h_sc.wait_expired;
        if (h_sc.wait_expired != 1) return finish(fail(OXZ_ERR_STATE, "oxz_selftest_bounded_wait: the wait recorded %d, not a run-out", h_sc.wait_expired));
        // the same kernel alone: its own arrival is all it waits for
        if (cudaMemset(d_sc, 0, sizeof(DevScalars)) != cudaSuccess) return finish(fail(OXZ_ERR_CUDA, "oxz_selftest_bounded_wait: cudaMemset failed"));
        MailPeers one{};
        one.box[0] = boxes;
        st = launch_gate(nullptr, one, 1, 0, 2, nullptr, nullptr, 0, d_sc, (uint64_t)limit_ms * 1000000ull, nullptr);
        if (st != OXZ_OK) return finish(st);
        if (cudaMemcpy(&h_sc, d_sc, sizeof(DevScalars), cudaMemcpyDeviceToHost) != cudaSuccess)
            return finish(fail(OXZ_ERR_CUDA, "oxz_selftest_bounded_wait: the second launch failed"));
        if (h_sc.wait_expired != 0) return finish(fail(OXZ_ERR_STATE, "oxz_selftest_bounded_wait: a rank alone did not pass its own gate"));
        return finish(OXZ_OK);
    });
}

int32_t oxz_grad_norms_per_tensor(oxz_plan* p, oxz_comm* comm, double loss_scale, double max_grad_value, double* norms) {
    return oxz::guarded("oxz_grad_norms_per_tensor", [&]() -> int32_t {
        if (!p || !norms) return fail(OXZ_ERR_INVALID, "oxz_grad_norms_per_tensor: null argument");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_grad_norms_per_tensor: the plan has no device state. Call oxz_state_alloc first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_grad_norms_per_tensor: a step is in flight. Call oxz_step_wait first");
        if (p->early_groups) return fail(OXZ_ERR_STATE, "oxz_grad_norms_per_tensor: buckets of the next step were already handed in");
        if (!std::isnan(max_grad_value) && !(std::isfinite(max_grad_value) && max_grad_value > 0.0))
            return fail(OXZ_ERR_INVALID, "trainer.max_grad_value is %g: it must be a finite positive number. Set a positive value, or remove the key to disable per-element clipping.", max_grad_value);
        if (p->cw > 1) {
            OXZ_TRY(comm_check(comm, "oxz_grad_norms_per_tensor"));
            if (comm != p->comm) return fail(OXZ_ERR_INVALID, "oxz_grad_norms_per_tensor: this is not the communicator the state was allocated with");
        }
        if (p->T == 0) return OXZ_OK;
        OXZ_CUDA(cudaSetDevice(p->device));
        cudaStream_t s = p->stream;
        const size_t n = 3 * (size_t)p->T;
        double* d_out = nullptr;
        double* h_out = nullptr;
        OXZ_CUDA(cudaMalloc((void**)&d_out, n * 8));
        cudaError_t e = cudaMallocHost((void**)&h_out, n * 8);
        if (e != cudaSuccess) {
            cudaFree(d_out);
            return fail(OXZ_ERR_CUDA, "oxz_grad_norms_per_tensor: %s", cudaGetErrorString(e));
        }
        auto run = [&]() -> int32_t {
            OXZ_CUDA(cudaMemsetAsync(d_out, 0, n * 8, s));
            const bool scaled = !std::isnan(loss_scale) && loss_scale != 0.0;
            const int32_t clamp_on = std::isnan(max_grad_value) ? 0 : 1;
            // with several ranks the summed gradients of the tiles this rank owns are what the step's reduction left
            // (f32 for the pulling and copying modes, the gradients' own type after an NCCL reduce-scatter)
            const bool summed = p->cw > 1;
            const void* src = summed ? p->reduced : p->grads;
            const int32_t dt = !summed ? p->gdt : (p->mode == OXZ_SYNC_NCCL ? p->gdt : OXZ_F32);
            OXZ_TRY(launch_sumsq_tensors(s, p->geom, src, dt, tile_map(p), p->d_tile_meta, p->d_present,
                                         scaled ? (float)(1.0 / loss_scale) : 1.0f, clamp_on ? (float)max_grad_value : 0.f,
                                         clamp_on, d_out));
            // ranks own disjoint tiles: the sum over ranks completes every tensor (a full replica already holds all)
            if (p->cw > 1 && p->mode != OXZ_SYNC_REPLICATED) OXZ_TRY(comm_stream_allreduce_f64(comm, d_out, (uint32_t)n, h_out, s));
            OXZ_CUDA(cudaMemcpyAsync(h_out, d_out, n * 8, cudaMemcpyDeviceToHost, s));
            OXZ_CUDA(cudaStreamSynchronize(s));
            // which tensors some rank had a gradient for: the flags the last step's kernels read
            std::vector<uint8_t> flags(p->T);
            OXZ_CUDA(cudaMemcpy(flags.data(), p->d_present, p->T, cudaMemcpyDeviceToHost));
            for (uint64_t i = 0; i < p->T; i++) {
                if (!flags[i]) norms[i] = -1.0;
                else if (h_out[3 * i + 2] > 0.0) norms[i] = std::nan("");
                else if (h_out[3 * i + 1] > 0.0) norms[i] = INFINITY;
                else norms[i] = std::sqrt(h_out[3 * i]);
            }
            return OXZ_OK;
        };
        const int32_t st = run();
        cudaFreeHost(h_out);
        cudaFree(d_out);
        return st;
    });
}

int32_t oxz_plan_set_profile(oxz_plan* p, int32_t on) {
    return oxz::guarded("oxz_plan_set_profile", [&]() -> int32_t {
        if (!p) return fail(OXZ_ERR_INVALID, "oxz_plan_set_profile: null plan");
        if (!p->allocated) return fail(OXZ_ERR_STATE, "oxz_plan_set_profile: call oxz_state_alloc first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_plan_set_profile: a step is in flight");
        OXZ_CUDA(cudaSetDevice(p->device));
        if (on && !p->ev[0])
            for (auto& e : p->ev) OXZ_CUDA(cudaEventCreate(&e));
        p->profile = on != 0;
        return OXZ_OK;
    });
}

int32_t oxz_step_profile_read(oxz_plan* p, oxz_step_profile* out) {
    return oxz::guarded("oxz_step_profile_read", [&]() -> int32_t {
        if (!p || !out) return fail(OXZ_ERR_INVALID, "oxz_step_profile_read: null argument");
        if (!p->profile) return fail(OXZ_ERR_STATE, "oxz_step_profile_read: profiling is off. Call oxz_plan_set_profile first");
        if (p->inflight) return fail(OXZ_ERR_STATE, "oxz_step_profile_read: a step is in flight. Call oxz_step_wait first");
        OXZ_CUDA(cudaSetDevice(p->device));
        float d[5];
        for (int i = 0; i < 5; i++) OXZ_CUDA(cudaEventElapsedTime(&d[i], p->ev[i], p->ev[i + 1]));
        out->collect_ms = d[0];
        out->norm_ms = d[1];
        out->decide_ms = d[2];
        out->update_ms = d[3];
        out->publish_ms = d[4];
        OXZ_CUDA(cudaEventElapsedTime(&out->total_ms, p->ev[0], p->ev[5]));
        return OXZ_OK;
    });
}

int32_t oxz_step(oxz_plan* p, oxz_comm* comm, const oxz_hyper* h, const uint8_t* present, double* extras,
                 uint32_t n_extras, oxz_step_result* res) {
    return oxz::guarded("oxz_step", [&]() -> int32_t {
        OXZ_TRY(oxz_step_async(p, comm, h, present, extras, n_extras));
        return oxz_step_wait(p, res);
    });
}

// ---- standalone norm ----
namespace {
struct NormScratch {
    int blocks = 0;
    uint32_t slots = 0;
    double* d_partials = nullptr;
    double* d_acc = nullptr;
    DevScalars* d_scalars = nullptr;
    DevScalars* h_scalars = nullptr;
};
std::mutex g_norm_mu;
std::map<int, NormScratch> g_norm_scratch;
}  // namespace

int32_t oxz_grad_norm(const void* device_grads, int32_t dtype, uint64_t n, double loss_scale, double max_grad_value,
                      void* stream, double* norm) {
    return oxz::guarded("oxz_grad_norm", [&]() -> int32_t {
        if (!norm || (!device_grads && n)) return fail(OXZ_ERR_INVALID, "oxz_grad_norm: null argument");
        if (dtype != OXZ_F32 && dtype != OXZ_BF16 && dtype != OXZ_F16) return fail(OXZ_ERR_INVALID, "oxz_grad_norm: dtype %d is none of f32, bf16, f16", dtype);
        if ((uintptr_t)device_grads & 15) return fail(OXZ_ERR_INVALID, "oxz_grad_norm: the gradients are not 16-byte aligned");
        if (!std::isnan(max_grad_value) && !(std::isfinite(max_grad_value) && max_grad_value > 0.0))
            return fail(OXZ_ERR_INVALID, "trainer.max_grad_value is %g: it must be a finite positive number. Set a positive value, or remove the key to disable per-element clipping.", max_grad_value);
        int dev = 0;
        OXZ_CUDA(cudaGetDevice(&dev));
        std::lock_guard<std::mutex> lock(g_norm_mu);
        NormScratch& sc = g_norm_scratch[dev];
        if (!sc.d_partials) {
            LaunchGeom g;
            OXZ_TRY(query_geom(dev, &g));
            sc.blocks = g.norm_blocks;
            sc.slots = norm_partial_slots(g);
            OXZ_CUDA(cudaMalloc((void**)&sc.d_partials, (size_t)norm_partial_slots(g) * 3 * 8));
            OXZ_CUDA(cudaMalloc((void**)&sc.d_acc, ACC_DOUBLES * 8));
            OXZ_CUDA(cudaMalloc((void**)&sc.d_scalars, sizeof(DevScalars)));
            OXZ_CUDA(cudaMallocHost((void**)&sc.h_scalars, sizeof(DevScalars)));
        }
        cudaStream_t s = (cudaStream_t)stream;
        const bool scaled = !std::isnan(loss_scale) && loss_scale != 0.0;
        const int clamp_on = std::isnan(max_grad_value) ? 0 : 1;
        OXZ_TRY(launch_sumsq_plain(s, sc.blocks, device_grads, dtype, n, scaled ? (float)(1.0 / loss_scale) : 1.0f,
                                   clamp_on ? (float)max_grad_value : 0.f, clamp_on, sc.d_partials));
        OXZ_TRY(launch_reduce_partials(s, sc.d_partials, sc.slots, sc.d_acc, nullptr));
        FinalizeParams fp{};
        fp.max_grad_norm = 1.7976931348623157e308;  // a pure measurement: nothing is rescaled
        OXZ_TRY(launch_finalize(s, sc.d_acc, fp, sc.d_scalars));
        OXZ_CUDA(cudaMemcpyAsync(sc.h_scalars, sc.d_scalars, sizeof(DevScalars), cudaMemcpyDeviceToHost, s));
        OXZ_CUDA(cudaStreamSynchronize(s));
        *norm = sc.h_scalars->norm;
        return OXZ_OK;
    });
}

}  // extern "C"
