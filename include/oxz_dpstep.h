/*
 * oxz_dpstep — C ABI of a B200-native data-parallel optimizer step for oxidizr.
 *
 * The library replaces, behind oxidizr's LitTrainer::training_step, the work between
 * "AFTER ACCUMULATION LOOP" (src/trainer.rs:515) and the end of step_once (src/trainer.rs:695):
 * the gradient sum over ranks, the loss-scale unscale, the inf/NaN decision, the value and
 * global-norm clips, the fused AdamW update with the weight-decay groups, and the write-back of
 * f32 master and narrow working weights.
 *
 * Conventions
 *   - Every function returns an oxz_status (0 = OK) and never throws or aborts the process.
 *     oxz_last_error() returns the calling thread's last error text.
 *   - One oxz_plan (and one oxz_comm) per rank. A plan is used by one thread at a time; different
 *     ranks' plans may be driven from different threads of one process (the reference runs one OS
 *     thread per rank, src/dp/launch.rs:207-240) or from one process per rank.
 *   - Device work is enqueued on the plan's stream. Calls named *_async return before it ends.
 *   - There is no CPU fallback: a call that needs the GPU fails with OXZ_ERR_CUDA without one.
 */
#ifndef OXZ_DPSTEP_H
#define OXZ_DPSTEP_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OXZ_ABI_VERSION 1u

typedef enum oxz_status {
    OXZ_OK = 0,
    OXZ_ERR_INVALID = 1,     /* bad argument; mirrors boostr Error::InvalidArgument / TrainingError */
    OXZ_ERR_CUDA = 2,        /* a CUDA runtime call failed */
    OXZ_ERR_NCCL = 3,        /* a collective failed; mirrors Error::DistributedError. Peers may be waiting:
                                the caller must abort the group (src/dp/reduce.rs:27-29) */
    OXZ_ERR_STATE = 4,       /* call order: state not allocated, a step still in flight, ... */
    OXZ_ERR_ABORTED = 5,     /* the communicator was aborted (src/dp/launch.rs:97-103) */
    OXZ_ERR_UNSUPPORTED = 6, /* NCCL library or peer access unavailable */
    OXZ_ERR_DATA = 7,        /* mirrors Error::DataError of the row arithmetic */
    OXZ_ERR_TIMEOUT = 8      /* a rank never joined a collective of a local group within its timeout, or a bounded
                                wait inside a kernel of the step ran out (on any rank: every rank reports it) */
} oxz_status;

typedef enum oxz_dtype { OXZ_F32 = 0, OXZ_BF16 = 1, OXZ_F16 = 2 } oxz_dtype;

/* How the gradients of different ranks meet. */
typedef enum oxz_sync_mode {
    OXZ_SYNC_SINGLE = 0, /* world 1: no collective (NoOpCommunicator, src/trainer.rs:234) */
    OXZ_SYNC_P2P = 1,    /* fused kernels over NVLink peer memory: pull-reduce in f32 in rank order, push of the narrow
                            weights; the step's barriers and its one small sum (norm terms, loss) also cross through
                            peer memory, in rank order, when up to four ranks sit on distinct GPUs behind an NCCL
                            communicator (OXZ_MAIL=1 in the environment: at any rank count; OXZ_MAIL=0: never; small
                            NCCL all-reduces serve otherwise, at the same speed) */
    OXZ_SYNC_NCCL = 2,   /* ncclReduceScatter / ncclAllGather in the gradient's own dtype */
    OXZ_SYNC_COPY = 3,   /* copy engines move the bytes over NVLink (peers' gradient slices into local staging,
                            the updated weights out to every peer), pipelined by groups of buckets with the
                            kernels that sum in f32 in rank order, measure the norm and update */
    OXZ_SYNC_REPLICATED = 4 /* the reference's own layout (full replicas, README.md:284; src/dp/reduce.rs:30-60):
                            every rank sums every rank's gradients in f32 in rank order and runs the whole
                            update on its own full copy of the state; nothing is sharded, no weights travel.
                            Kept as the parity mode for the sharded ones: W times their memory and update work */
} oxz_sync_mode;

typedef struct oxz_comm oxz_comm;
typedef struct oxz_plan oxz_plan;

uint32_t oxz_abi_version(void);
const char* oxz_last_error(void);
const char* oxz_status_name(int32_t status);

/* ------------------------------------------------------------------ communicator
 * Replaces boostr's NcclCommunicator as oxidizr creates and ends it:
 * NcclCommunicator::from_streams (src/dp/launch.rs:82-95) and abort (src/dp/launch.rs:97-103). */

/* 128-byte rendezvous token for oxz_comm_init_rank; make it on one rank and hand it to the others. */
int32_t oxz_comm_unique_id(uint8_t id[128]);
/* One communicator for this rank, on `device`. Collective over all ranks. One process per rank or one thread per rank. */
int32_t oxz_comm_init_rank(int32_t device, int32_t rank, int32_t world, const uint8_t id[128], oxz_comm** out);
/* All communicators of a single-process group at once, as from_streams does (src/dp/launch.rs:82-95). */
int32_t oxz_comm_init_all(int32_t n, const int32_t* devices, oxz_comm** out);
/* An in-process group of n rank threads that meet on the host, with a collective timeout and abort: the counterpart
 * of boostr's LocalCommunicator::with_timeout (src/dp/launch.rs:52-71, tests/data_parallel.rs:158-185). Ranks may
 * share one GPU (devices[i] equal) or use none (devices NULL or -1: host collectives only). Device collectives
 * drain the stream and go through host memory; it serves OXZ_SYNC_P2P, OXZ_SYNC_COPY and OXZ_SYNC_REPLICATED plans,
 * not OXZ_SYNC_NCCL ones. */
int32_t oxz_comm_init_local(int32_t n, const int32_t* devices, double timeout_seconds, oxz_comm** out);
int32_t oxz_comm_world_size(const oxz_comm* comm, int32_t* world);
int32_t oxz_comm_rank(const oxz_comm* comm, int32_t* rank);
/* Ends every pending and future collective of this rank with an error; callable from any thread. */
int32_t oxz_comm_abort(oxz_comm* comm);
int32_t oxz_comm_destroy(oxz_comm* comm);
/* Sum of two host counts over every rank: the step-weighting collective (src/dp/weighting.rs:63-101). Blocking. */
int32_t oxz_allreduce_i64x2(oxz_comm* comm, int64_t inout[2]);
/* Sum of up to 16 host doubles over every rank: the logged loss when it must be known before the update is
 * enqueued (the `extras` of boostr all_reduce_flat_sum, src/dp/reduce.rs:57-59). Blocking. */
int32_t oxz_allreduce_f64(oxz_comm* comm, double* inout, uint32_t n);
/* Broadcast of device memory from `root`: initial replica sync and the stop flag (src/dp/broadcast.rs:54,77). */
int32_t oxz_broadcast(oxz_comm* comm, void* device_ptr, uint64_t bytes, int32_t root);
/* Barrier over every rank (src/dp/trainer_hooks.rs:104). Blocking. */
int32_t oxz_barrier(oxz_comm* comm);

/* One thread per rank with a first-failure abort: run_ranks (src/dp/launch.rs:183-272). `body` runs once per rank
 * (on the calling thread when world is 1). The first rank whose body returns a non-zero status aborts every
 * communicator in comms (may be NULL) once, so peers blocked in a collective return; all threads are joined; the
 * status and text of the rank that failed first are returned as "rank r of w failed first: ...", later errors are
 * dropped. *failed_rank receives that rank, or -1. */
typedef int32_t (*oxz_rank_body)(int32_t rank, int32_t world, void* user);
int32_t oxz_run_ranks(int32_t world, oxz_comm* const* comms, oxz_rank_body body, void* user, int32_t* failed_rank);
/* Sets the calling thread's error text, for a body whose failure did not come from this library. */
int32_t oxz_set_last_error(const char* message);

/* ------------------------------------------------------------------ plan
 * The flat layout of the trainable parameters and their AdamW groups. Replaces the `declared`
 * (id, shape) list of reduce_step_gradients (src/dp/reduce.rs:45-56) and DecayPlan::param_groups
 * (src/weight_decay/plan.rs:113-122). Tensors keep parameter_ids order (src/trainer.rs:208). */

typedef struct oxz_plan_desc {
    uint64_t n_tensors;
    const uint64_t* numel;       /* [n_tensors] elements per tensor */
    const uint8_t* no_decay;     /* [n_tensors] 1 = member of the zero-decay group; NULL = none */
    const float* lr_scale;       /* [n_tensors] ParamGroup::lr_scale; NULL = 1.0 */
    int32_t grad_dtype;          /* oxz_dtype of the gradients a rank produces */
    int32_t param_dtype;         /* oxz_dtype of the working weights; OXZ_F32 keeps no separate master */
    int32_t world, rank;
    int32_t sync_mode;           /* oxz_sync_mode; OXZ_SYNC_SINGLE requires world 1 */
    int32_t device;              /* CUDA device ordinal */
    uint64_t bucket_bytes;       /* gradient bytes per bucket; 0 = 64 MiB */
} oxz_plan_desc;

typedef struct oxz_plan_info {
    uint64_t n_tensors;
    uint64_t numel_total;     /* trainable elements */
    uint64_t padded_total;    /* elements of the flat space (tensor starts are tile-aligned) */
    uint64_t tile_elems;      /* alignment of every tensor start, bucket and shard, in elements */
    uint64_t n_buckets;
    uint64_t bucket_elems;    /* elements per bucket, the last bucket may be shorter */
    uint64_t local_elems;     /* elements of optimizer state this rank owns (1/world of every bucket) */
    uint64_t n_groups;        /* distinct (lr_scale, decay) groups */
} oxz_plan_info;

int32_t oxz_plan_create(const oxz_plan_desc* desc, oxz_plan** out); /* host only: runs without a GPU */
int32_t oxz_plan_destroy(oxz_plan* plan);
int32_t oxz_plan_query(const oxz_plan* plan, oxz_plan_info* info);
/* offsets[i]: first flat element of tensor i */
int32_t oxz_plan_tensor_offsets(const oxz_plan* plan, uint64_t* offsets);
/* For bucket b: its flat start, its length, and the start and length of the part rank `rank` owns. */
int32_t oxz_plan_bucket(const oxz_plan* plan, uint64_t b, int32_t rank, uint64_t* start, uint64_t* len,
                        uint64_t* shard_start, uint64_t* shard_len);
/* Flat element -> element of `rank`'s local state arrays, or UINT64_MAX when another rank owns it. */
int32_t oxz_plan_local_index(const oxz_plan* plan, int32_t rank, uint64_t flat_index, uint64_t* local_index);
/* The CUDA stream (cudaStream_t) the plan enqueues on; NULL restores the plan's own stream. */
int32_t oxz_plan_set_stream(oxz_plan* plan, void* stream);

/* ------------------------------------------------------------------ state
 * Replaces the state boostr's AdamW owns: exp_avg, exp_avg_sq, the f32 master and the applied-step
 * count (src/checkpoint_set/optimizer_io.rs:1-5), plus the flat gradient and working-weight buffers. */

/* Allocates the device buffers (zero-filled). `comm` may be NULL at world 1. With OXZ_SYNC_P2P and OXZ_SYNC_COPY
 * this is collective: ranks exchange peer mappings of their gradient and weight buffers. */
int32_t oxz_state_alloc(oxz_plan* plan, oxz_comm* comm);
/* Device pointers of the flat buffers. grads: padded_total x grad_dtype. work: padded_total x param_dtype
 * (at world 1 with param_dtype F32 it is the master itself: no separate copy is kept). master/exp_avg/exp_avg_sq:
 * local_elems x f32. A backward pass may write its gradients straight into grads + offsets[i]. */
int32_t oxz_state_pointers(const oxz_plan* plan, void** grads, void** work, void** master, void** exp_avg,
                           void** exp_avg_sq);
typedef enum oxz_state_kind { OXZ_STATE_MASTER = 0, OXZ_STATE_EXP_AVG = 1, OXZ_STATE_EXP_AVG_SQ = 2,
                              OXZ_STATE_WORK = 3, OXZ_STATE_GRADS = 4 } oxz_state_kind;
/* Copies one whole tensor from host memory (f32 for master/moments; the buffer's dtype for work and grads).
 * A rank keeps the elements it owns and ignores the rest (work and grads are whole on every rank). Blocking. */
int32_t oxz_state_import(oxz_plan* plan, int32_t kind, uint64_t tensor, const void* host);
/* Copies the elements this rank owns of one tensor into host memory and leaves the others untouched. Blocking.
 * Mirrors optimizer.state_dict / load_state_dict (src/checkpoint_set/optimizer_io.rs:41-63,116-136). */
int32_t oxz_state_export(oxz_plan* plan, int32_t kind, uint64_t tensor, void* host);
int32_t oxz_state_set_timestep(oxz_plan* plan, uint64_t applied_steps);
int32_t oxz_state_timestep(const oxz_plan* plan, uint64_t* applied_steps); /* optimizer_timestep, src/trainer.rs:906-908 */

/* Writes the optimizer state file of a checkpoint set in the reference's layout (src/checkpoint_set/optimizer_io.rs:1-5,
 * 62-74): SafeTensors keyed `<name>.exp_avg`, `<name>.exp_avg_sq`, `<name>.master` (F32; master only for parameters
 * narrower than f32) and `__step` (F64), metadata format = "oxidizr-optimizer". names[i] is tensor i's checkpoint name,
 * ndim[i] its rank and dims its shapes back to back. Collective with more than one rank: the slices are merged bit
 * for bit and rank 0 writes. The write is atomic (temporary file, then rename), and every rank returns the same answer:
 * a file error on the writing rank is an error on all of them. Blocking. */
int32_t oxz_optimizer_save(oxz_plan* plan, oxz_comm* comm, const char* path, const char* const* names,
                           const uint32_t* ndim, const uint64_t* dims);
/* Reads such a file into the plan's state (src/checkpoint_set/optimizer_io.rs:113-137): strict - an unknown name, a
 * missing key, a shape or dtype mismatch, or a file shorter than its header says is found before anything is loaded and
 * leaves the state unchanged. A read or copy error after those checks (the disk or the device failing midway) leaves the
 * state partly loaded: load again, or create the plan afresh. Every rank reads the file and keeps the elements it owns, so
 * a file written at one world size loads at another. Blocking. */
int32_t oxz_optimizer_load(oxz_plan* plan, const char* path, const char* const* names, const uint32_t* ndim,
                           const uint64_t* dims);

/* ------------------------------------------------------------------ gradients in
 * Replaces the flatten half of boostr all_reduce_flat_sum (called at src/dp/reduce.rs:58). */

/* Packs per-tensor device gradients (grad_dtype, 16-byte aligned) into the flat buffer. grad_ptrs[i] NULL = this
 * rank has no gradient for tensor i: its span is zero-filled. accumulate != 0 adds instead of storing, in f32,
 * which is the micro-batch accumulation of src/trainer.rs:1087-1107. Asynchronous. */
int32_t oxz_grads_flatten_async(oxz_plan* plan, const void* const* grad_ptrs, int32_t accumulate);
/* Host gradients of one tensor (grad_dtype; pinned memory copies asynchronously) into the flat buffer. */
int32_t oxz_grads_upload_async(oxz_plan* plan, uint64_t tensor, const void* host);
/* A second gradient buffer, so that a step's gradients can arrive from the host while the step before still reads its
 * own: allocates it (and, with peers, maps it into every rank: collective for OXZ_SYNC_P2P / OXZ_SYNC_REPLICATED).
 * oxz_grads_upload_next_async copies one tensor into the buffer that is NOT current, on the plan's own upload stream,
 * also while a step is in flight; it starts after the step that last read that buffer. oxz_grads_swap makes that
 * buffer the current one (oxz_state_pointers then reports it): the next oxz_step_async or oxz_grads_ready_async waits
 * for the uploads. With several ranks every rank swaps between the same two steps. No reference counterpart: the
 * reference's gradients are produced on the device. */
int32_t oxz_grads_double_buffer(oxz_plan* plan, oxz_comm* comm);
int32_t oxz_grads_upload_next_async(oxz_plan* plan, uint64_t tensor, const void* host);
int32_t oxz_grads_swap(oxz_plan* plan);

/* ------------------------------------------------------------------ the step */

typedef struct oxz_hyper {
    double lr;               /* this step's learning rate, LrPlan::lr_at (src/trainer.rs:254) */
    double beta1, beta2, eps, weight_decay; /* AdamWConfig, src/trainer.rs:184-191 */
    double max_grad_norm;    /* src/trainer.rs:581-587 */
    double max_grad_value;   /* NaN = off (src/grad_clip.rs:47) */
    double target_grad_norm; /* NaN = off (src/trainer.rs:635-645) */
    double loss_scale;       /* LossScaler::scale; NaN or 0 = no scaler (src/trainer.rs:573-575) */
    double clip_eps;         /* epsilon of the clip coefficient max/(norm+eps); 1e-6 conventional */
    int32_t decay_after;     /* 0 = weight decay before the Adam term (default) */
    int32_t eps_mode;        /* 0 = sqrt(v)/sqrt(1-beta2^t) + eps (default), 1 = sqrt(v) + eps */
    int32_t spike_skip;      /* the spike guard vetoed this step (src/trainer.rs:612) */
    int32_t reserved;
} oxz_hyper;

typedef struct oxz_step_result {
    double grad_norm;     /* the norm clip_gradients measured (src/grad_clip.rs:28-35) */
    double reported_norm; /* what training_step returns (src/trainer.rs:629-632, 657-661) */
    double clip_coef;     /* product of the applied clip coefficients */
    int32_t overflow;     /* !grad_norm.is_finite() (src/trainer.rs:619) */
    int32_t applied;      /* optimizer.step ran */
    uint64_t timestep;    /* applied steps after this one */
} oxz_step_result;

/* One optimizer step on the gradients now in the flat buffer: src/trainer.rs:520-661 in one call.
 * present: [n_tensors] 0 = THIS rank produced no gradient for the tensor this step; NULL = it has all of them. The
 *          ranks' flags may differ (an expert only some ranks routed to): the library forms their union, and a tensor
 *          is left untouched only when NO rank has a gradient for it (src/dp/reduce.rs:20). Where a rank's flag is 0
 *          but another's is 1, that rank's span of the gradient buffer must hold zeros (oxz_grads_flatten_async with
 *          a NULL pointer for the tensor writes them); a span no rank has a gradient for may hold anything.
 * extras:  n_extras host doubles summed over ranks in place (the logged loss, src/dp/reduce.rs:57-59).
 * The decision to skip is taken on the device; nothing is read back between the norm and the update. */
int32_t oxz_step_async(oxz_plan* plan, oxz_comm* comm, const oxz_hyper* hyper, const uint8_t* present,
                       double* extras, uint32_t n_extras);
/* Overlap with the tail of backward: reduces over ranks (at world 1: measures) the gradient buckets
 * [first_bucket, first_bucket + n_buckets) now, on a side stream, while backward still produces the others. The
 * buckets must be complete on every rank once the work enqueued so far on `producer_stream` (the stream backward
 * writes the gradients on; NULL = the legacy default stream) has finished. Collective: every rank makes the same calls
 * in the same order. hyper (its loss_scale and max_grad_value) and present must be the ones the step's
 * oxz_step_async is then given; that call reduces whatever buckets are left and finishes the step. Up to 6 calls per
 * step. Serves OXZ_SYNC_SINGLE and OXZ_SYNC_P2P. (The reference reduces once, after backward: src/trainer.rs:520-527.) */
int32_t oxz_grads_ready_async(oxz_plan* plan, oxz_comm* comm, const oxz_hyper* hyper, const uint8_t* present,
                              uint64_t first_bucket, uint64_t n_buckets, void* producer_stream);
/* Waits for the step in flight, fills `result` and the extras, and advances the applied-step count. */
int32_t oxz_step_wait(oxz_plan* plan, oxz_step_result* result);
/* oxz_step_async followed by oxz_step_wait. */
int32_t oxz_step(oxz_plan* plan, oxz_comm* comm, const oxz_hyper* hyper, const uint8_t* present, double* extras,
                 uint32_t n_extras, oxz_step_result* result);

/* Per-phase device times of the last finished step, measured with CUDA events on the plan's stream: the
 * counterpart of the reference's PROFILE_TRAIN wall-clock lines (src/trainer.rs:579-593, 648-655). */
typedef struct oxz_step_profile {
    float collect_ms; /* waiting for / reducing the ranks' gradients before the norm kernel (0 at world 1) */
    float norm_ms;    /* the unscale + inf check + sum-of-squares kernel (with the peer pull in P2P mode) */
    float decide_ms;  /* partials -> norm all-reduce -> decision and clip coefficients */
    float update_ms;  /* the fused AdamW kernel (with the peer push in P2P mode) */
    float publish_ms; /* all-gather or closing barrier (0 at world 1) */
    float total_ms;
} oxz_step_profile;
/* Grid sizes the plan launches with (blocks of 256 threads) and the device's SM count. */
int32_t oxz_plan_launch_geometry(const oxz_plan* plan, int32_t* sm_count, int32_t* norm_blocks, int32_t* update_blocks);
/* Which kernel did the most recent pull of the peers' gradients (OXZ_SYNC_P2P): per-lane loads, or bulk
 * asynchronous copies into shared memory (16-bit gradients, 2, 4 or 8 ranks, a bucket's
 * shard a multiple of 8 tiles; OXZ_PULL_BULK=0 in the environment turns it off). Both give the same bits. No
 * reference counterpart: a tuning and test aid. */
#define OXZ_PULL_KERNEL_NONE 0
#define OXZ_PULL_KERNEL_LOADS 1
#define OXZ_PULL_KERNEL_BULK 2
int32_t oxz_plan_last_pull_kernel(const oxz_plan* plan, int32_t* kind);
/* Which form of the update kernel the most recent step launched: one tile per warp (the default), two tiles per warp
 * with 256-bit stores of the 16-bit weights (the default with two ranks), or inputs staged through shared memory
 * (OXZ_ADAM_VARIANT=4|5 in the environment; measured slower, kept for the comparison). All give the same bits. No
 * reference counterpart: a tuning and test aid. */
#define OXZ_UPDATE_KERNEL_NONE 0
#define OXZ_UPDATE_KERNEL_TILE 1
#define OXZ_UPDATE_KERNEL_WIDE 2
#define OXZ_UPDATE_KERNEL_STAGED 3
int32_t oxz_plan_last_update_kernel(const oxz_plan* plan, int32_t* kind);
/* How the plan's ranks meet for the step's barriers and its small sum: 0 = not at all (one rank), 1 = collectives of
 * the communicator (NCCL all-reduces, or the host rendezvous of a local group), 2 = through mailboxes in peer memory
 * (one kernel per exchange, every wait bounded: OXZ_MAIL_TIMEOUT_MS in the environment, 30000 by default, after which
 * the step changes nothing and oxz_step_wait returns OXZ_ERR_TIMEOUT; oxz_comm_abort ends such a wait at once).
 * No reference counterpart: a tuning and test aid. */
#define OXZ_EXCHANGE_NONE 0
#define OXZ_EXCHANGE_COMM 1
#define OXZ_EXCHANGE_MAILBOX 2
int32_t oxz_plan_exchange_kind(const oxz_plan* plan, int32_t* kind);
/* Shows on one GPU, without any fault, what a rank sees when a peer never arrives: launches the gate kernel as rank 0 of
 * two ranks whose other rank does not exist, with its wait bounded to limit_ms. *outcome receives what the kernel
 * recorded (1 = the wait ran out, which is the expected answer); the call then runs the same kernel alone (world 1) to
 * show the context still works, and returns OXZ_OK only if both went as expected. No reference counterpart: a test aid. */
int32_t oxz_selftest_bounded_wait(int32_t device, uint32_t limit_ms, int32_t* outcome);
/* on != 0: record the events every step (a few microseconds); off by default. */
int32_t oxz_plan_set_profile(oxz_plan* plan, int32_t on);
int32_t oxz_step_profile_read(oxz_plan* plan, oxz_step_profile* out);

/* Global L2 norm of n device gradients after the unscale (and after the clamp when max_grad_value is not NaN),
 * as a pure measurement: compute_grad_norm(.., f64::MAX) of src/grad_clip.rs:49. A non-finite element gives a
 * non-finite norm (src/grad_clip.rs:130-143). Blocking; allocates its partial-sum scratch on first use per device. */
int32_t oxz_grad_norm(const void* device_grads, int32_t dtype, uint64_t n, double loss_scale, double max_grad_value,
                      void* stream, double* norm);

/* The L2 norm of every tensor's gradient as the last step saw it: summed over ranks, unscaled by loss_scale (NaN or 0:
 * no scaler), clamped to max_grad_value when that is not NaN. It is grad_norm_for_tensor (src/trainer.rs:933-937), which
 * the reference calls per parameter to name the offending tensors after a non-finite norm (diagnose_bad_gradients,
 * src/trainer.rs:990-1020) and for its DEBUG_GRAD breakdown (src/trainer.rs:940-988). norms[n_tensors]: a tensor with a
 * non-finite element gives inf or NaN as the global norm does; a tensor no rank had a gradient for gives -1. Call it
 * after oxz_step_wait and before the gradient buffer changes; collective with more than one rank (each rank measures
 * the part it owns); blocking; off the step's path (it is only needed after a skipped step or for debugging). The
 * per-tensor sums are accumulated with atomic adds: their last bits may differ from run to run. */
int32_t oxz_grad_norms_per_tensor(oxz_plan* plan, oxz_comm* comm, double loss_scale, double max_grad_value, double* norms);

/* The same measurement as oxz_grad_norm for hosts that must not allocate. It has no counterpart in the reference:
 * it exists for callers of this library whose device memory is already spoken for (a trainer whose caching
 * allocator owns the whole GPU, a process with a fixed memory budget) or whose step loop must not meet the
 * device-wide synchronisation of cudaMalloc/cudaFree. The partial sums live in a static device array inside the
 * library image (about 7 KiB, held by every GPU that loads the library until the process exits); the call makes
 * no cudaMalloc, cudaMallocHost or cudaFree, and the result is copied straight into *norm.
 *   clusters: how many 4-block clusters to launch; 0 = as many as the device holds at once. The array holds the
 *             partial sums of at most OXZ_STATIC_NORM_MAX_CLUSTERS clusters: a larger request is OXZ_ERR_INVALID.
 * The first call on each device looks up the array's device address and the launch geometry (with that device
 * current) and keeps them; make that first call outside any stream capture. All calls on one device share the one
 * array, and it keeps the last call's contents (no stage depends on them): two calls whose kernels overlap on the
 * GPU, from different streams or threads, race on it and must be serialised by the caller. Blocking. */
#define OXZ_STATIC_NORM_MAX_CLUSTERS 256u
int32_t oxz_grad_norm_static(const void* device_grads, int32_t dtype, uint64_t n, double loss_scale,
                             double max_grad_value, uint32_t clusters, void* stream, double* norm);

/* ------------------------------------------------------------------ host decisions (pure, no GPU) */

typedef struct oxz_scaler_config { double initial, growth_factor, backoff_factor; uint64_t growth_interval; } oxz_scaler_config;
typedef struct oxz_scaler_state { double scale; uint64_t consecutive_ok; } oxz_scaler_state;
/* LossScaleConfig::check (src/loss_scale/config.rs:66-100). */
int32_t oxz_scaler_check(const oxz_scaler_config* cfg);
/* LossScaler::new / restore (src/loss_scale/scaler.rs:19-37). */
int32_t oxz_scaler_init(const oxz_scaler_config* cfg, oxz_scaler_state* state);
int32_t oxz_scaler_restore(const oxz_scaler_state* saved, oxz_scaler_state* state);
/* The scaler update at the end of a step (src/trainer.rs:666-681): untouched on a finite-gradient spike skip. */
int32_t oxz_scaler_record_step(const oxz_scaler_config* cfg, oxz_scaler_state* state, int32_t overflow,
                               int32_t spike_skip);

typedef enum oxz_decay_rule { OXZ_DECAY_ALL = 0, OXZ_SKIP_1D = 1, OXZ_SKIP_ALL = 2 } oxz_decay_rule;
/* WeightDecaySpec::check and ::excludes (src/weight_decay/rule.rs:78-118). *excluded = 1: no weight decay. */
int32_t oxz_decay_check(int32_t rule, const char* const* patterns, uint32_t n_patterns);
int32_t oxz_decay_excludes(int32_t rule, const char* const* patterns, uint32_t n_patterns, const char* name,
                           uint32_t rank, int32_t* excluded);

typedef struct oxz_spike_config { uint64_t window; double z_threshold; uint64_t min_steps; int32_t action_warn; int32_t reserved; } oxz_spike_config;
typedef struct oxz_spike_state { double mean, variance; uint64_t observed, detected, skipped; } oxz_spike_state;
/* TrainMetrics::judge over SpikeGuard::observe (src/metrics/state.rs:79-86, src/metrics/spike.rs:124-168).
 * index is the 0-based step; *skip = 1 when the step must skip the optimizer; *flagged = 1 for any spike. */
int32_t oxz_spike_judge(const oxz_spike_config* cfg, oxz_spike_state* state, uint64_t index, double loss,
                        int32_t* skip, int32_t* flagged);

typedef enum oxz_lr_schedule { OXZ_LR_CONSTANT = 0, OXZ_LR_COSINE = 1, OXZ_LR_LINEAR = 2, OXZ_LR_WSD = 3 } oxz_lr_schedule;
typedef enum oxz_decay_shape { OXZ_SHAPE_LINEAR = 0, OXZ_SHAPE_COSINE = 1, OXZ_SHAPE_SQRT = 2 } oxz_decay_shape;
typedef struct oxz_lr_plan {
    double base_lr, min_lr_ratio;
    uint64_t warmup_steps, total_steps;
    uint64_t decay_steps;  /* wsd only: resolved span (src/schedule.rs:124-132) */
    int32_t schedule, decay_shape;
} oxz_lr_plan;
/* LrPlan::lr_at (src/schedule.rs:177-183). */
int32_t oxz_lr_at(const oxz_lr_plan* plan, uint64_t step, double* lr);

typedef struct oxz_row_layout { uint64_t num_rows, rank_batch_size, world_size; } oxz_row_layout;
typedef struct oxz_data_position { uint64_t epoch, row; } oxz_data_position;
/* RowLayout::for_world checks (src/data/rows.rs:66-123). */
int32_t oxz_rows_check(const oxz_row_layout* layout);
/* RowLayout::advance (src/data/rows.rs:167-191). */
int32_t oxz_rows_advance(const oxz_row_layout* layout, oxz_data_position pos, uint64_t batches, oxz_data_position* out);
/* One rank's draw of the next global batch in stream order (src/data/positioning.rs:44-68, src/data/batch.rs:51-71):
 * rows[rank_batch_size] are the global row indices, and when `tokens` (u32 LE stream) is given, inputs/targets
 * [rank_batch_size * seq_len] receive the i64 token ids. *next is the position after the global batch. */
int32_t oxz_rows_next_window(const oxz_row_layout* layout, oxz_data_position pos, uint64_t rank, uint64_t seq_len,
                             uint64_t first_row, const uint32_t* tokens, uint64_t n_tokens, uint64_t* rows,
                             int64_t* inputs, int64_t* targets, oxz_data_position* next);
/* The row order the reference runs by default, RowOrder::Shuffled (trainer.shuffle_rows = true, src/config.rs:80-82): a
 * permutation of the shard's rows per epoch, which the Rust side makes with rand's StdRng and SliceRandom::shuffle
 * (epoch_permutation(num_rows, seed, epoch), src/data/rows.rs:258-272) and hands over; the library maps slot -> perm[slot]
 * as EpochOrder::row does (src/data/rows.rs:240-256) and so reads the reference's rows bit for bit without restating the
 * generator.
 * oxz_rows_batch_epoch: the epoch whose order the batch drawn at `pos` reads - pos.epoch, or the next one when fewer
 * rows than a global batch are left (RowLayout::batch_start, src/data/rows.rs:153-165).
 * oxz_rows_check_permutation: OXZ_ERR_DATA unless perm holds every value of 0..n once.
 * oxz_rows_next_window_ordered: oxz_rows_next_window with the row at each slot taken from perm (n_perm = num_rows
 * values, the order of epoch perm_epoch); OXZ_ERR_DATA when the batch reads another epoch than perm_epoch. Only the
 * entries it reads are range-checked here; check the whole permutation once with oxz_rows_check_permutation. */
int32_t oxz_rows_batch_epoch(const oxz_row_layout* layout, oxz_data_position pos, uint64_t* epoch);
int32_t oxz_rows_check_permutation(const uint32_t* perm, uint64_t n);
int32_t oxz_rows_next_window_ordered(const oxz_row_layout* layout, oxz_data_position pos, uint64_t rank, uint64_t seq_len,
                                     uint64_t first_row, const uint32_t* tokens, uint64_t n_tokens, uint64_t perm_epoch,
                                     const uint32_t* perm, uint64_t n_perm, uint64_t* rows, int64_t* inputs,
                                     int64_t* targets, oxz_data_position* next);
/* ------------------------------------------------------------------ the checkpoint meta's keys on this path
 *
 * `checkpoint_step_N.meta.json` is CheckpointMeta (src/config.rs:1223-1302) as serde_json writes it. These are the keys
 * the optimizer path records and reads back on resume (src/checkpoint_set/snapshot.rs:245-262); every other key is
 * skipped on load and written empty by oxz_meta_save. A has_* flag of 0 is serde's Option::None (key absent or null). */
typedef struct oxz_resume_meta {
    uint64_t step;
    int32_t has_world_size, has_global_batch_rows, has_loss_scale, has_data_position, has_spike_guard;
    int32_t has_weight_decay_rule, has_mixture;
    uint32_t n_mixture_weights;      /* MixtureRecord::weights (src/data/mixture/record.rs:13-19): fetch with oxz_meta_mixture_weights */
    uint64_t mixture_rows_per_epoch;
    int32_t weight_decay_rule;      /* oxz_decay_rule; a meta without the key reads as OXZ_DECAY_ALL, the rule of runs
                                       from before parameter groups (WeightDecaySpec::of_meta, src/weight_decay/rule.rs:68-74) */
    uint32_t n_no_decay_patterns;   /* fetch each with oxz_meta_no_decay_pattern */
    uint64_t world_size, global_batch_rows;
    oxz_scaler_state loss_scale;     /* GradScalerState {scale, consecutive_ok}; f64 at full precision */
    oxz_data_position data_position; /* DataPosition {epoch, row} (src/data/rows.rs:28-34) */
    oxz_spike_state spike_guard;     /* SpikeGuardState (src/metrics/spike.rs:14-26) */
    char checkpoint_file[512];
    char optimizer_file[512];        /* empty: none */
} oxz_resume_meta;
/* CheckpointMeta::load restricted to the keys above. */
int32_t oxz_meta_load(const char* path, oxz_resume_meta* out);
int32_t oxz_meta_no_decay_pattern(const char* path, uint32_t index, char* buf, uint64_t cap);
/* CheckpointMeta::save_to (src/config.rs:1386-1394): pretty JSON, written beside the target and renamed over it.
 * Floats are printed so that they read back to the same bits. */
int32_t oxz_meta_save(const char* path, const oxz_resume_meta* meta, const char* const* no_decay_patterns,
                      const double* mixture_weights);
int32_t oxz_meta_mixture_weights(const char* path, double* weights, uint32_t cap, uint32_t* n_weights);
/* check_mixture_resume (src/data/mixture/record.rs:40-70): the weights (compared by bits) and rows_per_epoch decide the
 * row at every slot, so a resume must run the mixture the meta records; a meta without one resumes only a run without
 * weights. has_current 0: this run sets no weights. Nothing is checked at step 0 or without a meta. */
int32_t oxz_check_mixture_resume(const char* meta_path, uint64_t start_step, int32_t has_current, const double* weights,
                                 uint32_t n_weights, uint64_t rows_per_epoch);
/* check_resume_world (src/dp/resume.rs:19-55): a meta that records another world size is an error naming both (a
 * meta without the key counts as one rank); another global batch only fills `warning` (empty otherwise). A run at
 * step 0 and a null meta_path check nothing. */
int32_t oxz_check_resume_world(const char* meta_path, uint64_t start_step, uint64_t world, uint64_t global_batch_rows,
                               char* warning, uint64_t cap);
/* read_loss_scale_state (src/loss_scale/resume.rs:14-29): the scaler state a run at start_step resumes with;
 * *has_state = 0 at step 0, without a meta, or when the meta has no loss_scale key. */
int32_t oxz_read_loss_scale_state(const char* meta_path, uint64_t start_step, int32_t* has_state, oxz_scaler_state* state);

/* The rank-sliced row loader in stream order (LitDataLoader::with_rank + next_batch, src/data/ranks.rs:25-41,
 * src/data/positioning.rs:44-68, src/data/batch.rs:51-71) over one little-endian u32 token file mapped read-only
 * (src/data/source.rs:7-12, 204-230). Rows are seq_len + 1 tokens; rows [first_row, end_row) form the loader's range
 * (end_row 0 = every whole row; the tail shorter than a row is never read). Opening needs no GPU. */
typedef struct oxz_loader oxz_loader;
int32_t oxz_loader_open(const char* path, uint64_t seq_len, uint64_t rank_batch_size, uint64_t rank, uint64_t world,
                        uint64_t first_row, uint64_t end_row, int32_t device, oxz_loader** out);
/* LitDataLoader::from_files + with_row_ranges + with_rank (src/data/multi_source.rs:17-52, src/data/row_ranges.rs:40-106):
 * the stream is file 0's whole rows, then file 1's, ...; each file drops its own tail. spans holds n_spans pairs
 * (start, end) of GLOBAL rows, end exclusive, ascending without overlap; loader rows count across them in order
 * (n_spans 0: every row). The `.tokens.json` sidecars are the tokenizer's and are not read here. */
int32_t oxz_loader_open_files(const char* const* paths, uint32_t n_paths, uint64_t seq_len, uint64_t rank_batch_size,
                              uint64_t rank, uint64_t world, const uint64_t* spans, uint32_t n_spans, int32_t device,
                              oxz_loader** out);
/* LitDataLoader::source_rows: whole rows of each source in order; *n_sources receives the count, rows up to cap of them. */
int32_t oxz_loader_source_rows(const oxz_loader* loader, uint64_t* rows, uint32_t cap, uint32_t* n_sources);
/* PrefetchDataLoader::new(loader, depth) (src/data/prefetch.rs:37-115): a host thread draws the coming batches in order
 * from the loader's position and copies their rows into pinned buffers (depth + 2 of them) while the device works on
 * the current batch, so that oxz_loader_next_batch_async only has to enqueue the copy and the kernels. The batch
 * sequence is the unprefetched loader's; a seek or a new mixture restarts the thread at the new position; an error
 * the thread meets is returned by the call that reaches that batch. depth 0 turns it off. Needs the device (pinned
 * memory). */
int32_t oxz_loader_set_prefetch(oxz_loader* loader, uint32_t depth);
/* LitDataLoader::with_row_order(RowOrder::Shuffled{seed}) (src/data/construction.rs:140) with the permutation made by the
 * caller: perm[slot] is the loader row (0..oxz_loader_num_rows) read at `slot` of `epoch`. The loader copies it, rejects
 * anything that is not a permutation of its rows, and keeps the orders of two epochs (a third drops the lowest), so the
 * next epoch's can be handed over before the rollover - a prefetch thread draws across it. A batch whose epoch has no
 * order fails with OXZ_ERR_DATA naming the epoch. perm NULL: back to stream order. Restarts a prefetch thread at the
 * loader's position. Not together with a mixture, whose sources are drawn in passes of their own. */
int32_t oxz_loader_set_row_order(oxz_loader* loader, uint64_t epoch, const uint32_t* perm, uint64_t n);
/* Draws the next batch's rows only: rows[rank_batch_size] receive the global rows this rank reads, and the position
 * moves on as after a batch. Host only: what a dry run or a test of the row order needs. */
int32_t oxz_loader_next_rows(oxz_loader* loader, uint64_t* rows);
/* LitDataLoader::with_mixture (src/data/mixture/loader.rs:16-33) in stream order: one weight per source. An epoch is
 * rows_per_epoch slots (has_rows_per_epoch 0: the sources' training rows); source i fills its largest-remainder quota of
 * them (src/data/mixture/quota.rs:22-57), interleaved by smooth weighted round-robin, the same every epoch
 * (src/data/mixture/schedule.rs:103-122), and its k-th draw of the run reads its training row k % n_i
 * (src/data/mixture/draw.rs:44-62), so an upsampled source repeats each row once per pass and a seek is exact. The
 * loader's layout then counts rows_per_epoch rows and the position returns to the start. The shuffled schedule and the
 * per-pass permutations of a shuffled mixture need rand 0.10.3's StdRng on this side and are not offered. */
int32_t oxz_loader_set_mixture(oxz_loader* loader, const double* weights, uint32_t n_weights, int32_t has_rows_per_epoch,
                               uint64_t rows_per_epoch);
typedef struct oxz_mixture_source { double weight; uint64_t rows_per_epoch, train_rows; } oxz_mixture_source; /* MixtureSource */
int32_t oxz_loader_mixture_sources(const oxz_loader* loader, oxz_mixture_source* out, uint32_t cap, uint32_t* n_sources);
/* quotas(weights, rows) by itself (pure, no loader). */
int32_t oxz_mixture_quotas(const double* weights, uint32_t n_weights, uint64_t rows, uint64_t* quotas);
int32_t oxz_loader_close(oxz_loader* loader);
/* LitDataLoader::with_target_mask(TargetMask::PrefixLm{target_base, always_score}) (src/data/mask.rs:21-47): a position
 * scores iff its TARGET id is at least target_base or is listed in always_score. on = 0 turns the mask off.
 * TargetMask::SpeechAudio depends on boostr's SpeechLayout and is not offered. */
#define OXZ_MAX_ALWAYS_SCORE 16u
int32_t oxz_loader_set_target_mask(oxz_loader* loader, int32_t on, uint32_t target_base, const uint32_t* always_score,
                                   uint32_t n_always);
/* LitDataLoader::with_document_mask (src/data/host_masks.rs:28-35): every position whose INPUT is the separator is
 * unscored (ANDed with the target mask), and each batch carries its document segments (src/data/segments.rs:62-101). */
int32_t oxz_loader_set_document_mask(oxz_loader* loader, int32_t on, uint32_t separator_id);
/* The masks of the batch oxz_loader_next_batch_async enqueued last (Batch::loss_mask / scored / segments,
 * src/data/batch.rs:11-26), built on the device in the same stream. Device pointers are null for what is off.
 * scored and n_segments point into pinned host memory that the stream fills: read them once the stream has passed
 * the batch (an unmasked batch scores rows * seq_len, written at once). Valid until the batch after the next. */
typedef struct oxz_batch_masks {
    const float* loss_mask;      /* device [rows, seq_len] f32: 1.0 scored, 0.0 not */
    const int32_t* segment_ids;  /* device [rows, seq_len] i32: segment of each input token, counted over the batch */
    const int32_t* cu_seqlens;   /* device: *n_segments + 1 cumulative offsets over the flattened inputs, from 0 */
    const uint64_t* scored;      /* pinned host */
    const uint64_t* n_segments;  /* pinned host; 0 when the document mask is off */
} oxz_batch_masks;
int32_t oxz_loader_batch_masks(const oxz_loader* loader, oxz_batch_masks* out);
int32_t oxz_loader_num_rows(const oxz_loader* loader, uint64_t* rows);
/* LitDataLoader::position / seek (src/data/positioning.rs:14-42): the position is global, every rank seeks the same one. */
int32_t oxz_loader_position(const oxz_loader* loader, oxz_data_position* pos);
int32_t oxz_loader_seek(oxz_loader* loader, oxz_data_position pos);
/* Draws this rank's rows of the next global batch and advances past the whole global batch. *inputs and *targets
 * are device pointers to [rank_batch_size, seq_len] i64 owned by the loader, valid until the second-next call;
 * rows (may be NULL) receives the global row indices. Asynchronous on `stream`; use one stream for all calls of a
 * loader, the buffers are recycled in its order. */
int32_t oxz_loader_next_batch_async(oxz_loader* loader, void* stream, int64_t** inputs, int64_t** targets, uint64_t* rows);

/* StepWeighting::over_ranks applied to the summed counts (src/dp/weighting.rs:46-61): counts = {scored, masked ranks}
 * after oxz_allreduce_i64x2. *global_scored = -1 for an unmasked step. Mixed masks are OXZ_ERR_INVALID on every rank. */
int32_t oxz_step_weighting(uint64_t local_micro_batches, int32_t world, const int64_t counts[2],
                           uint64_t* micro_batches, int64_t* global_scored);

#ifdef __cplusplus
}
#endif
#endif /* OXZ_DPSTEP_H */
