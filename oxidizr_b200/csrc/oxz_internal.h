// Internal declarations shared by the translation units of liboxz_dpstep.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <memory>
#include <new>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/oxz_dpstep.h"

namespace oxz {

// ---- errors: thread-local text behind oxz_last_error() ----
int32_t fail(int32_t status, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();

// Runs the body of a C entry point: whatever C++ throws inside (an allocation that fails, say) becomes a status and a
// message; no exception leaves the library, as a caller across a C boundary cannot catch one.
template <class F>
inline int32_t guarded(const char* who, F&& body) noexcept {
    try {
        return body();
    } catch (const std::bad_alloc&) {
        return fail(OXZ_ERR_STATE, "%s: out of host memory", who);
    } catch (const std::exception& e) {
        return fail(OXZ_ERR_STATE, "%s: %s", who, e.what());
    } catch (...) {
        return fail(OXZ_ERR_STATE, "%s: an unknown C++ exception", who);
    }
}

#define OXZ_CUDA(expr)                                                                              \
    do {                                                                                            \
        cudaError_t e__ = (expr);                                                                   \
        if (e__ != cudaSuccess)                                                                     \
            return ::oxz::fail(OXZ_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                               __FILE__, __LINE__);                                                 \
    } while (0)

#define OXZ_TRY(expr)                  \
    do {                               \
        int32_t s__ = (expr);          \
        if (s__ != OXZ_OK) return s__; \
    } while (0)

constexpr uint32_t TILE = 256;           // elements per tile: one 8-element vector per lane of a warp
constexpr uint32_t MAX_GROUPS = 8;       // distinct (lr_scale, decay) groups a plan may hold
constexpr uint32_t PAD_TILE = 0xFFFFFFFFu;  // tile_meta of a tile past the last tensor
constexpr uint32_t MAX_PEERS = 16;
constexpr uint32_t MAX_EXTRAS = 13;
constexpr uint32_t MAX_PIPE = 8;         // groups of buckets a copy-engine step is pipelined in
// The doubles that cross the ranks once per step: {sum of squares, infinities seen, NaNs seen, a bounded wait ran out
// on some rank, extras...}.
constexpr uint32_t ACC_EXPIRED = 3;
constexpr uint32_t ACC_EXTRAS = 4;
constexpr uint32_t ACC_DOUBLES = ACC_EXTRAS + MAX_EXTRAS;

// A rank's mailbox: one slot per sending rank and parity of the exchange number, in device memory every peer can
// write. An exchange is: write the payload into my slot of every rank's mailbox, then the exchange number (release);
// wait until every slot of my own mailbox carries that number (acquire); read the payloads. Two parities suffice: a
// rank can enter exchange k+2, which reuses the slots of k, only after every rank has entered k+1 and so has finished
// reading k. It stands in for a small NCCL all-reduce or barrier (tens of microseconds) at a few microseconds, and
// the sum over the slots runs in rank order on every rank.
constexpr uint32_t MAIL_PAYLOAD = 4096;  // bytes: the tensors' present flags, or ACC_DOUBLES doubles
struct alignas(16) MailSlot {
    unsigned long long seq;
    unsigned long long pad;
    unsigned char payload[MAIL_PAYLOAD];
};
struct MailBox {
    MailSlot slot[2][MAX_PEERS];
};
struct MailPeers {
    MailBox* box[MAX_PEERS];  // box[r]: rank r's mailbox as this rank addresses it; box[rank] is local
};

inline size_t dtype_size(int32_t dt) { return dt == OXZ_F32 ? 4 : 2; }

// Maps a tile of this rank's local state arrays to a tile of the flat parameter space.
// Bucket b holds tiles [b*tpb, ...); rank r owns the r-th 1/world of every bucket.
struct TileMap {
    uint32_t tiles_per_shard;       // tiles a rank owns of a full bucket
    uint32_t tiles_per_bucket;      // tiles of a full bucket = world * tiles_per_shard
    uint32_t n_buckets;
    uint32_t last_shard_tiles;      // tiles a rank owns of the last bucket
    uint32_t rank;
    uint32_t n_local_tiles;         // end of the tile range a launch covers
    uint32_t first_tile;            // start of that range (0 for a whole-shard launch)
};

// Per-step scalars of the update, rounded to f32 on the host from f64.
struct AdamParams {
    float beta1, one_minus_beta1, beta2, one_minus_beta2;
    float eps, bias2_sqrt;
    float inv_scale;   // 1/loss_scale, 1.0f without a scaler
    float clamp_hi;    // max_grad_value
    int32_t clamp_on;
    int32_t decay_after, eps_mode;
    int32_t push_hint;  // 0: streaming stores of the working weights (default); 1: plain stores (tuning aid)
    float step_size[MAX_GROUPS];
    float decay_mul[MAX_GROUPS];
};

// Device-resident outcome of the norm pass; the update kernel reads it, no host round trip.
struct DevScalars {
    double norm;        // measured global norm (inf or NaN on overflow)
    double sumsq;
    float c1, c2;       // clip coefficients applied in this order
    int32_t overflow;
    int32_t skip;       // overflow or spike veto: the update kernel returns at once
    int32_t wait_expired;  // a bounded wait inside a kernel ran out, on this rank or (after the exchange) on any rank:
                           // the step changes nothing and is reported failed. 2: the wait was ended by an abort
    int32_t reserved;
};

struct PeerTable {
    const void* grads[MAX_PEERS];
    void* work[MAX_PEERS];
};

struct FinalizeParams {
    double max_grad_norm, target_grad_norm, clip_eps;
    int32_t has_target, spike_skip;
};

// ---- kernel launchers (oxz_kernels.cu) ----
struct LaunchGeom {
    int sm_count;
    int norm_blocks;   // multiple of the cluster size
    int pull_blocks[3];  // per gradient dtype (f32, bf16, f16), never more than norm_blocks
    int bulk_blocks[3];  // bulk-copy pull, per rank count 2 / 4 / 8
    int adam_blocks;
};
int32_t query_geom(int device, LaunchGeom* g);
uint32_t norm_partial_slots(const LaunchGeom& g);
uint32_t pull_partial_slots(const LaunchGeom& g, int32_t dt);

// Sum of squares of unscaled (and optionally clamped) gradients held in one local array of dtype `dt`.
int32_t launch_sumsq(cudaStream_t s, const LaunchGeom& g, const void* grads, int32_t dt, const TileMap& map,
                     const uint32_t* tile_meta, const uint8_t* present, bool check_present, float inv_scale,
                     float clamp_hi, int32_t clamp_on, double* partials);
// Per-tensor {sum, inf, NaN} of the same quantity, added into out[3 * n_tensors] (zeroed by the caller).
int32_t launch_sumsq_tensors(cudaStream_t s, const LaunchGeom& g, const void* grads, int32_t dt, const TileMap& map,
                             const uint32_t* tile_meta, const uint8_t* present, float inv_scale, float clamp_hi,
                             int32_t clamp_on, double* out);
// Same over a plain array of n elements (no plan): the standalone norm entry point.
int32_t launch_sumsq_plain(cudaStream_t s, int blocks, const void* grads, int32_t dt, uint64_t n, float inv_scale,
                           float clamp_hi, int32_t clamp_on, double* partials);
// Pull-reduce: sums this rank's tiles of every peer's gradient buffer in f32 in rank order, stores the sum
// in `reduced` (local, f32) and accumulates the squares as launch_sumsq does.
int32_t launch_pull_sumsq(cudaStream_t s, const LaunchGeom& g, const PeerTable& peers, int32_t world, int staged, int32_t dt,
                          const TileMap& map, const uint32_t* tile_meta, const uint8_t* present, bool check_present,
                          float inv_scale, float clamp_hi, int32_t clamp_on, float* reduced, double* partials);
// The pull-reduce with 1-D bulk asynchronous copies into shared memory (16-bit gradients, 2/4/8 ranks, every tensor
// present, shard and range boundaries on multiples of 8 tiles). Returns OXZ_ERR_UNSUPPORTED when the shape does not fit.
bool pull_bulk_fits(const TileMap& map, int32_t world, int32_t dt);
int32_t launch_pull_bulk(cudaStream_t s, const LaunchGeom& g, const PeerTable& peers, int32_t world, int32_t dt,
                         const TileMap& map, const uint32_t* tile_meta, const uint8_t* present, bool check_present,
                         float inv_scale, float clamp_hi, int32_t clamp_on, float* reduced, double* partials,
                         uint32_t slots, DevScalars* scalars);
// partials[slots][3] -> acc[0..3) = {sum, inf count, nan count}; acc[ACC_EXPIRED] = 1 when scalars (may be null) says a
// bounded wait of this rank ran out
int32_t launch_reduce_partials(cudaStream_t s, const double* partials, uint32_t slots, double* acc, const DevScalars* scalars);
// acc -> scalars (norm, clip coefficients, decisions); acc[ACC_EXPIRED] > 0 makes the step a reported failure
int32_t launch_finalize(cudaStream_t s, const double* acc, const FinalizeParams& fp, DevScalars* scalars);
// Exchange `seq` as a barrier, optionally carrying the tensors' present flags: present_out[i] = OR over ranks of their
// present_in[i] (T 0: barrier only). Every wait is bounded by limit_ns and ended early by *abort_flag != 0.
int32_t launch_gate(cudaStream_t s, const MailPeers& mail, int32_t world, int32_t rank, uint64_t seq, const uint8_t* present_in,
                    uint8_t* present_out, uint32_t T, DevScalars* scalars, uint64_t limit_ns, const int32_t* abort_flag);
// The step's one data exchange, fused with the sums either side of it: partials -> this rank's {sum, inf, NaN} ->
// exchange `seq` with acc[ACC_EXPIRED..ACC_EXTRAS + n_extras) riding along -> sums over ranks in rank order ->
// acc and the scalars. sum_norm 0 (full replicas): the three norm terms stay this rank's own.
int32_t launch_decide(cudaStream_t s, const MailPeers& mail, int32_t world, int32_t rank, uint64_t seq, const double* partials,
                      uint32_t slots, double* acc, uint32_t n_extras, int32_t sum_norm, const FinalizeParams& fp,
                      DevScalars* scalars, uint64_t limit_ns, const int32_t* abort_flag);
// The fused update. gsrc is indexed in local space (dtype gdt); master/m/v local f32; work is written in flat space
// to every pointer of `peers.work[0..n_work)` (n_work 0: no working copy).
int32_t launch_adamw(cudaStream_t s, const LaunchGeom& g, const void* gsrc, int32_t gdt, float* master, float* m,
                     float* v, const PeerTable& peers, int32_t n_work, int32_t pdt, const TileMap& map,
                     const uint32_t* tile_meta, const uint8_t* present, bool check_present, const DevScalars* scalars,
                     const AdamParams& ap);
// Which form of the update kernel the calling thread's last launch_adamw took (OXZ_UPDATE_KERNEL_*).
int32_t last_update_kernel();
// Packs per-tensor gradients into the flat buffer.
int32_t launch_flatten(cudaStream_t s, const LaunchGeom& g, void* flat, int32_t dt, uint32_t n_tiles,
                       const uint32_t* tile_meta, const uint64_t* d_offsets, const uint64_t* d_numel,
                       const void* const* d_src, int32_t accumulate);

}  // namespace oxz

namespace oxz {
// In-process rendezvous of a local group: the counterpart of boostr's LocalCommunicator (src/dp/launch.rs:52-71).
struct LocalGroup;
}  // namespace oxz

// ---- opaque handles ----
struct oxz_comm {
    int32_t kind = 0;      // 0 = NCCL, 1 = local (in-process threads, host rendezvous with timeout and abort)
    std::shared_ptr<oxz::LocalGroup> local;
    void* nccl = nullptr;  // ncclComm_t
    int32_t rank = 0, world = 1, device = 0;
    cudaStream_t stream = nullptr;  // for the small blocking collectives
    void* d_small = nullptr;        // 512 bytes of device scratch for them
    int32_t* h_abort_flag = nullptr;  // pinned, mapped: kernels that wait on other ranks poll it; oxz_comm_abort sets it
    std::atomic<int> aborted{0};
};

struct oxz_plan {
    // layout (host)
    uint64_t T = 0;
    std::vector<uint64_t> numel, offset;
    std::vector<uint8_t> group_of;
    std::vector<float> group_lr_scale;
    std::vector<uint8_t> group_no_decay;
    // world / rank: how the state is sharded (1 / 0 for OXZ_SYNC_REPLICATED); cw / cr: the communicator's size and
    // this rank's place in it, which is what the gradient sum runs over
    int32_t gdt = 0, pdt = 0, world = 1, rank = 0, cw = 1, cr = 0, mode = 0, device = 0;
    uint64_t numel_total = 0, total_tiles = 0;
    uint64_t bucket_tiles = 0, n_buckets = 0, last_bucket_tiles = 0, local_tiles = 0;
    std::vector<uint32_t> tile_meta;  // per flat tile: tensor | group << 24

    // device state
    bool allocated = false;
    cudaStream_t own_stream = nullptr, stream = nullptr;
    oxz::LaunchGeom geom{};
    void* grads = nullptr;
    void* work = nullptr;
    float *master = nullptr, *exp_avg = nullptr, *exp_avg_sq = nullptr;
    void* reduced = nullptr;  // W>1: the summed gradients of this rank's tiles (f32 for P2P, grad dtype for NCCL)
    uint32_t* d_tile_meta = nullptr;
    uint8_t* d_present = nullptr;     // per tensor: some rank has a gradient this step (what the kernels read)
    uint8_t* d_present_in = nullptr;  // this rank's own flags (more than one rank)
    uint64_t *d_offsets = nullptr, *d_numel = nullptr;
    const void** d_src = nullptr;
    double* d_partials = nullptr;
    double* d_acc = nullptr;  // 3 + MAX_EXTRAS doubles
    oxz::DevScalars* d_scalars = nullptr;
    // pinned host mirrors
    oxz::DevScalars* h_scalars = nullptr;
    double* h_acc = nullptr;
    double* h_extras = nullptr;
    uint8_t* h_present = nullptr;     // this rank's own flags as last given
    uint8_t* h_union = nullptr;       // the union over ranks, where the host learns it (a local group)
    const void** h_src = nullptr;
    cudaEvent_t done = nullptr;
    bool profile = false;
    cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    oxz::PeerTable peers{};
    oxz::PeerTable own_work{};  // work[0] = this rank's weights, nothing else
    // a second gradient buffer (oxz_grads_double_buffer): `grads` is the one the next step reads, `grads_alt` the one
    // the host may fill meanwhile; oxz_grads_swap exchanges them (and the peers' addresses of them)
    void* grads_alt = nullptr;
    bool double_buffered = false;  // the second buffer is complete: allocated, events made, mapped by the peers
    const void* peer_grads_alt[oxz::MAX_PEERS] = {};
    cudaStream_t upload_stream = nullptr;
    cudaEvent_t ev_uploaded = nullptr, ev_last_read[2] = {nullptr, nullptr};
    int cur_grads = 0;          // which of the two buffers `grads` is
    bool upload_pending = false;  // uploads into the current buffer that the next step must wait for
    std::vector<void*> ipc_opened;
    // OXZ_SYNC_COPY: staging for the peers' gradient slices, one copy stream per peer, pipeline events
    void* stage = nullptr;
    oxz::PeerTable staged_src{};
    cudaStream_t copy_stream[oxz::MAX_PEERS] = {};
    cudaEvent_t ev_go = nullptr, ev_copied[oxz::MAX_PEERS][oxz::MAX_PIPE] = {}, ev_updated[oxz::MAX_PIPE] = {}, ev_pushed[oxz::MAX_PEERS] = {};
    uint32_t pipe_groups = 1;
    oxz_comm* comm = nullptr;
    // exchanges between ranks through peer memory (ranks on distinct GPUs behind an NCCL communicator)
    bool use_mail = false;
    oxz::MailBox* mail = nullptr;
    oxz::MailPeers mail_peers{};
    uint64_t mail_seq = 0;        // exchanges made so far; every rank makes the same ones in the same order
    uint64_t mail_limit_ns = 0;

    // buckets reduced ahead of the step (oxz_grads_ready_async)
    cudaStream_t early_stream = nullptr;
    cudaEvent_t ev_produced = nullptr, ev_early = nullptr;
    std::vector<uint8_t> early_done;   // per bucket
    uint32_t early_groups = 0;         // partial-sum groups already written this step
    int32_t last_pull_kernel = 0;      // OXZ_PULL_KERNEL_* of the most recent peer pull
    int32_t last_update_kernel = 0;    // OXZ_UPDATE_KERNEL_* of the most recent update
    double early_scale = 0.0, early_clamp = 0.0;

    // step bookkeeping
    uint64_t timestep = 0;
    bool inflight = false;
    bool present_all = true;
    oxz_hyper inflight_hyper{};
    double* inflight_extras = nullptr;
    uint32_t inflight_n_extras = 0;
};
