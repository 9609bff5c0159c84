//! Raw FFI declarations of `liboxz_dpstep.so`, the B200-native data-parallel optimizer step for oxidizr.
//!
//! One `extern "C"` item per declaration of `include/oxz_dpstep.h`, one `#[repr(C)]` struct per struct, one constant
//! per enumerator and `#define`. The header is the reference: read the contract of every call there. What each call
//! replaces inside oxidizr (file:line) is cited in the header next to it.
//!
//! Conventions of the library: every function returns an `oxz_status` as `i32` (0 = `OXZ_OK`) and never unwinds;
//! `oxz_last_error()` returns the calling thread's last error text; one `oxz_plan` and one `oxz_comm` per rank, a plan
//! is driven by one thread at a time (oxidizr runs one OS thread per rank, src/dp/launch.rs:207-240).
//!
//! `safe.rs` holds the thin safe layer `LitTrainer` would call.
#![allow(non_camel_case_types)]

use std::os::raw::{c_char, c_void};

pub mod safe;

// ---- status codes, dtypes, modes and the other small enumerations (all passed as i32 / u32) ----
pub const OXZ_OK: i32 = 0;
pub const OXZ_ERR_INVALID: i32 = 1;
pub const OXZ_ERR_CUDA: i32 = 2;
pub const OXZ_ERR_NCCL: i32 = 3;
pub const OXZ_ERR_STATE: i32 = 4;
pub const OXZ_ERR_ABORTED: i32 = 5;
pub const OXZ_ERR_UNSUPPORTED: i32 = 6;
pub const OXZ_ERR_DATA: i32 = 7;
pub const OXZ_ERR_TIMEOUT: i32 = 8;
pub const OXZ_F32: i32 = 0;
pub const OXZ_BF16: i32 = 1;
pub const OXZ_F16: i32 = 2;
pub const OXZ_SYNC_SINGLE: i32 = 0;
pub const OXZ_SYNC_P2P: i32 = 1;
pub const OXZ_SYNC_NCCL: i32 = 2;
pub const OXZ_SYNC_COPY: i32 = 3;
pub const OXZ_SYNC_REPLICATED: i32 = 4;
pub const OXZ_STATE_MASTER: i32 = 0;
pub const OXZ_STATE_EXP_AVG: i32 = 1;
pub const OXZ_STATE_EXP_AVG_SQ: i32 = 2;
pub const OXZ_STATE_WORK: i32 = 3;
pub const OXZ_STATE_GRADS: i32 = 4;
pub const OXZ_DECAY_ALL: i32 = 0;
pub const OXZ_SKIP_1D: i32 = 1;
pub const OXZ_SKIP_ALL: i32 = 2;
pub const OXZ_LR_CONSTANT: i32 = 0;
pub const OXZ_LR_COSINE: i32 = 1;
pub const OXZ_LR_LINEAR: i32 = 2;
pub const OXZ_LR_WSD: i32 = 3;
pub const OXZ_SHAPE_LINEAR: i32 = 0;
pub const OXZ_SHAPE_COSINE: i32 = 1;
pub const OXZ_SHAPE_SQRT: i32 = 2;
pub const OXZ_ABI_VERSION: u32 = 1;
pub const OXZ_PULL_KERNEL_NONE: i32 = 0;
pub const OXZ_PULL_KERNEL_LOADS: i32 = 1;
pub const OXZ_PULL_KERNEL_BULK: i32 = 2;
pub const OXZ_UPDATE_KERNEL_NONE: i32 = 0;
pub const OXZ_UPDATE_KERNEL_TILE: i32 = 1;
pub const OXZ_UPDATE_KERNEL_WIDE: i32 = 2;
pub const OXZ_UPDATE_KERNEL_STAGED: i32 = 3;
pub const OXZ_EXCHANGE_NONE: i32 = 0;
pub const OXZ_EXCHANGE_COMM: i32 = 1;
pub const OXZ_EXCHANGE_MAILBOX: i32 = 2;
pub const OXZ_STATIC_NORM_MAX_CLUSTERS: u32 = 256;
pub const OXZ_MAX_ALWAYS_SCORE: u32 = 16;

// ---- opaque handles ----
/// One rank's communicator (NCCL, or an in-process group that meets on the host).
#[repr(C)]
pub struct oxz_comm {
    _private: [u8; 0],
}
/// The flat layout of the trainable parameters, their AdamW groups and, once allocated, the device state.
#[repr(C)]
pub struct oxz_plan {
    _private: [u8; 0],
}
/// The rank-sliced row loader over u32 token files.
#[repr(C)]
pub struct oxz_loader {
    _private: [u8; 0],
}

/// `run_ranks` body: called once per rank with (rank, world, user); non-zero = that rank failed.
pub type oxz_rank_body = Option<unsafe extern "C" fn(rank: i32, world: i32, user: *mut c_void) -> i32>;

// ---- plain structs, field for field as in the header ----
#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_plan_desc {
    pub n_tensors: u64,
    pub numel: *const u64,
    pub no_decay: *const u8,
    pub lr_scale: *const f32,
    pub grad_dtype: i32,
    pub param_dtype: i32,
    pub world: i32,
    pub rank: i32,
    pub sync_mode: i32,
    pub device: i32,
    pub bucket_bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_plan_info {
    pub n_tensors: u64,
    pub numel_total: u64,
    pub padded_total: u64,
    pub tile_elems: u64,
    pub n_buckets: u64,
    pub bucket_elems: u64,
    pub local_elems: u64,
    pub n_groups: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_hyper {
    pub lr: f64,
    pub beta1: f64,
    pub beta2: f64,
    pub eps: f64,
    pub weight_decay: f64,
    pub max_grad_norm: f64,
    pub max_grad_value: f64,
    pub target_grad_norm: f64,
    pub loss_scale: f64,
    pub clip_eps: f64,
    pub decay_after: i32,
    pub eps_mode: i32,
    pub spike_skip: i32,
    pub reserved: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_step_result {
    pub grad_norm: f64,
    pub reported_norm: f64,
    pub clip_coef: f64,
    pub overflow: i32,
    pub applied: i32,
    pub timestep: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_step_profile {
    pub collect_ms: f32,
    pub norm_ms: f32,
    pub decide_ms: f32,
    pub update_ms: f32,
    pub publish_ms: f32,
    pub total_ms: f32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_scaler_config {
    pub initial: f64,
    pub growth_factor: f64,
    pub backoff_factor: f64,
    pub growth_interval: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_scaler_state {
    pub scale: f64,
    pub consecutive_ok: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_spike_config {
    pub window: u64,
    pub z_threshold: f64,
    pub min_steps: u64,
    pub action_warn: i32,
    pub reserved: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_spike_state {
    pub mean: f64,
    pub variance: f64,
    pub observed: u64,
    pub detected: u64,
    pub skipped: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_lr_plan {
    pub base_lr: f64,
    pub min_lr_ratio: f64,
    pub warmup_steps: u64,
    pub total_steps: u64,
    pub decay_steps: u64,
    pub schedule: i32,
    pub decay_shape: i32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_row_layout {
    pub num_rows: u64,
    pub rank_batch_size: u64,
    pub world_size: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_data_position {
    pub epoch: u64,
    pub row: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_resume_meta {
    pub step: u64,
    pub has_world_size: i32,
    pub has_global_batch_rows: i32,
    pub has_loss_scale: i32,
    pub has_data_position: i32,
    pub has_spike_guard: i32,
    pub has_weight_decay_rule: i32,
    pub has_mixture: i32,
    pub n_mixture_weights: u32,
    pub mixture_rows_per_epoch: u64,
    pub weight_decay_rule: i32,
    pub n_no_decay_patterns: u32,
    pub world_size: u64,
    pub global_batch_rows: u64,
    pub loss_scale: oxz_scaler_state,
    pub data_position: oxz_data_position,
    pub spike_guard: oxz_spike_state,
    pub checkpoint_file: [c_char; 512],
    pub optimizer_file: [c_char; 512],
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_mixture_source {
    pub weight: f64,
    pub rows_per_epoch: u64,
    pub train_rows: u64,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct oxz_batch_masks {
    pub loss_mask: *const f32,
    pub segment_ids: *const i32,
    pub cu_seqlens: *const i32,
    pub scored: *const u64,
    pub n_segments: *const u64,
}

extern "C" {
    pub fn oxz_abi_version() -> u32;
    pub fn oxz_last_error() -> *const c_char;
    pub fn oxz_status_name(status: i32) -> *const c_char;
    pub fn oxz_comm_unique_id(id: *mut u8) -> i32;
    pub fn oxz_comm_init_rank(device: i32, rank: i32, world: i32, id: *const u8, out: *mut *mut oxz_comm) -> i32;
    pub fn oxz_comm_init_all(n: i32, devices: *const i32, out: *mut *mut oxz_comm) -> i32;
    pub fn oxz_comm_init_local(n: i32, devices: *const i32, timeout_seconds: f64, out: *mut *mut oxz_comm) -> i32;
    pub fn oxz_comm_world_size(comm: *const oxz_comm, world: *mut i32) -> i32;
    pub fn oxz_comm_rank(comm: *const oxz_comm, rank: *mut i32) -> i32;
    pub fn oxz_comm_abort(comm: *mut oxz_comm) -> i32;
    pub fn oxz_comm_destroy(comm: *mut oxz_comm) -> i32;
    pub fn oxz_allreduce_i64x2(comm: *mut oxz_comm, inout: *mut i64) -> i32;
    pub fn oxz_allreduce_f64(comm: *mut oxz_comm, inout: *mut f64, n: u32) -> i32;
    pub fn oxz_broadcast(comm: *mut oxz_comm, device_ptr: *mut c_void, bytes: u64, root: i32) -> i32;
    pub fn oxz_barrier(comm: *mut oxz_comm) -> i32;
    pub fn oxz_run_ranks(
        world: i32,
        comms: *const *mut oxz_comm,
        body: oxz_rank_body,
        user: *mut c_void,
        failed_rank: *mut i32,
    ) -> i32;
    pub fn oxz_set_last_error(message: *const c_char) -> i32;
    pub fn oxz_plan_create(desc: *const oxz_plan_desc, out: *mut *mut oxz_plan) -> i32;
    pub fn oxz_plan_destroy(plan: *mut oxz_plan) -> i32;
    pub fn oxz_plan_query(plan: *const oxz_plan, info: *mut oxz_plan_info) -> i32;
    pub fn oxz_plan_tensor_offsets(plan: *const oxz_plan, offsets: *mut u64) -> i32;
    pub fn oxz_plan_bucket(
        plan: *const oxz_plan,
        b: u64,
        rank: i32,
        start: *mut u64,
        len: *mut u64,
        shard_start: *mut u64,
        shard_len: *mut u64,
    ) -> i32;
    pub fn oxz_plan_local_index(plan: *const oxz_plan, rank: i32, flat_index: u64, local_index: *mut u64) -> i32;
    pub fn oxz_plan_set_stream(plan: *mut oxz_plan, stream: *mut c_void) -> i32;
    pub fn oxz_state_alloc(plan: *mut oxz_plan, comm: *mut oxz_comm) -> i32;
    pub fn oxz_state_pointers(
        plan: *const oxz_plan,
        grads: *mut *mut c_void,
        work: *mut *mut c_void,
        master: *mut *mut c_void,
        exp_avg: *mut *mut c_void,
        exp_avg_sq: *mut *mut c_void,
    ) -> i32;
    pub fn oxz_state_import(plan: *mut oxz_plan, kind: i32, tensor: u64, host: *const c_void) -> i32;
    pub fn oxz_state_export(plan: *mut oxz_plan, kind: i32, tensor: u64, host: *mut c_void) -> i32;
    pub fn oxz_state_set_timestep(plan: *mut oxz_plan, applied_steps: u64) -> i32;
    pub fn oxz_state_timestep(plan: *const oxz_plan, applied_steps: *mut u64) -> i32;
    pub fn oxz_optimizer_save(
        plan: *mut oxz_plan,
        comm: *mut oxz_comm,
        path: *const c_char,
        names: *const *const c_char,
        ndim: *const u32,
        dims: *const u64,
    ) -> i32;
    pub fn oxz_optimizer_load(
        plan: *mut oxz_plan,
        path: *const c_char,
        names: *const *const c_char,
        ndim: *const u32,
        dims: *const u64,
    ) -> i32;
    pub fn oxz_grads_flatten_async(plan: *mut oxz_plan, grad_ptrs: *const *const c_void, accumulate: i32) -> i32;
    pub fn oxz_grads_upload_async(plan: *mut oxz_plan, tensor: u64, host: *const c_void) -> i32;
    pub fn oxz_grads_double_buffer(plan: *mut oxz_plan, comm: *mut oxz_comm) -> i32;
    pub fn oxz_grads_upload_next_async(plan: *mut oxz_plan, tensor: u64, host: *const c_void) -> i32;
    pub fn oxz_grads_swap(plan: *mut oxz_plan) -> i32;
    pub fn oxz_step_async(
        plan: *mut oxz_plan,
        comm: *mut oxz_comm,
        hyper: *const oxz_hyper,
        present: *const u8,
        extras: *mut f64,
        n_extras: u32,
    ) -> i32;
    pub fn oxz_grads_ready_async(
        plan: *mut oxz_plan,
        comm: *mut oxz_comm,
        hyper: *const oxz_hyper,
        present: *const u8,
        first_bucket: u64,
        n_buckets: u64,
        producer_stream: *mut c_void,
    ) -> i32;
    pub fn oxz_step_wait(plan: *mut oxz_plan, result: *mut oxz_step_result) -> i32;
    pub fn oxz_step(
        plan: *mut oxz_plan,
        comm: *mut oxz_comm,
        hyper: *const oxz_hyper,
        present: *const u8,
        extras: *mut f64,
        n_extras: u32,
        result: *mut oxz_step_result,
    ) -> i32;
    pub fn oxz_plan_launch_geometry(
        plan: *const oxz_plan,
        sm_count: *mut i32,
        norm_blocks: *mut i32,
        update_blocks: *mut i32,
    ) -> i32;
    pub fn oxz_plan_last_pull_kernel(plan: *const oxz_plan, kind: *mut i32) -> i32;
    pub fn oxz_plan_last_update_kernel(plan: *const oxz_plan, kind: *mut i32) -> i32;
    pub fn oxz_plan_exchange_kind(plan: *const oxz_plan, kind: *mut i32) -> i32;
    pub fn oxz_selftest_bounded_wait(device: i32, limit_ms: u32, outcome: *mut i32) -> i32;
    pub fn oxz_plan_set_profile(plan: *mut oxz_plan, on: i32) -> i32;
    pub fn oxz_step_profile_read(plan: *mut oxz_plan, out: *mut oxz_step_profile) -> i32;
    pub fn oxz_grad_norm(
        device_grads: *const c_void,
        dtype: i32,
        n: u64,
        loss_scale: f64,
        max_grad_value: f64,
        stream: *mut c_void,
        norm: *mut f64,
    ) -> i32;
    pub fn oxz_grad_norms_per_tensor(
        plan: *mut oxz_plan,
        comm: *mut oxz_comm,
        loss_scale: f64,
        max_grad_value: f64,
        norms: *mut f64,
    ) -> i32;
    pub fn oxz_grad_norm_static(
        device_grads: *const c_void,
        dtype: i32,
        n: u64,
        loss_scale: f64,
        max_grad_value: f64,
        clusters: u32,
        stream: *mut c_void,
        norm: *mut f64,
    ) -> i32;
    pub fn oxz_scaler_check(cfg: *const oxz_scaler_config) -> i32;
    pub fn oxz_scaler_init(cfg: *const oxz_scaler_config, state: *mut oxz_scaler_state) -> i32;
    pub fn oxz_scaler_restore(saved: *const oxz_scaler_state, state: *mut oxz_scaler_state) -> i32;
    pub fn oxz_scaler_record_step(
        cfg: *const oxz_scaler_config,
        state: *mut oxz_scaler_state,
        overflow: i32,
        spike_skip: i32,
    ) -> i32;
    pub fn oxz_decay_check(rule: i32, patterns: *const *const c_char, n_patterns: u32) -> i32;
    pub fn oxz_decay_excludes(
        rule: i32,
        patterns: *const *const c_char,
        n_patterns: u32,
        name: *const c_char,
        rank: u32,
        excluded: *mut i32,
    ) -> i32;
    pub fn oxz_spike_judge(
        cfg: *const oxz_spike_config,
        state: *mut oxz_spike_state,
        index: u64,
        loss: f64,
        skip: *mut i32,
        flagged: *mut i32,
    ) -> i32;
    pub fn oxz_lr_at(plan: *const oxz_lr_plan, step: u64, lr: *mut f64) -> i32;
    pub fn oxz_rows_check(layout: *const oxz_row_layout) -> i32;
    pub fn oxz_rows_advance(
        layout: *const oxz_row_layout,
        pos: oxz_data_position,
        batches: u64,
        out: *mut oxz_data_position,
    ) -> i32;
    pub fn oxz_rows_next_window(
        layout: *const oxz_row_layout,
        pos: oxz_data_position,
        rank: u64,
        seq_len: u64,
        first_row: u64,
        tokens: *const u32,
        n_tokens: u64,
        rows: *mut u64,
        inputs: *mut i64,
        targets: *mut i64,
        next: *mut oxz_data_position,
    ) -> i32;
    pub fn oxz_rows_batch_epoch(layout: *const oxz_row_layout, pos: oxz_data_position, epoch: *mut u64) -> i32;
    pub fn oxz_rows_check_permutation(perm: *const u32, n: u64) -> i32;
    pub fn oxz_rows_next_window_ordered(
        layout: *const oxz_row_layout,
        pos: oxz_data_position,
        rank: u64,
        seq_len: u64,
        first_row: u64,
        tokens: *const u32,
        n_tokens: u64,
        perm_epoch: u64,
        perm: *const u32,
        n_perm: u64,
        rows: *mut u64,
        inputs: *mut i64,
        targets: *mut i64,
        next: *mut oxz_data_position,
    ) -> i32;
    pub fn oxz_meta_load(path: *const c_char, out: *mut oxz_resume_meta) -> i32;
    pub fn oxz_meta_no_decay_pattern(path: *const c_char, index: u32, buf: *mut c_char, cap: u64) -> i32;
    pub fn oxz_meta_save(
        path: *const c_char,
        meta: *const oxz_resume_meta,
        no_decay_patterns: *const *const c_char,
        mixture_weights: *const f64,
    ) -> i32;
    pub fn oxz_meta_mixture_weights(path: *const c_char, weights: *mut f64, cap: u32, n_weights: *mut u32) -> i32;
    pub fn oxz_check_mixture_resume(
        meta_path: *const c_char,
        start_step: u64,
        has_current: i32,
        weights: *const f64,
        n_weights: u32,
        rows_per_epoch: u64,
    ) -> i32;
    pub fn oxz_check_resume_world(
        meta_path: *const c_char,
        start_step: u64,
        world: u64,
        global_batch_rows: u64,
        warning: *mut c_char,
        cap: u64,
    ) -> i32;
    pub fn oxz_read_loss_scale_state(
        meta_path: *const c_char,
        start_step: u64,
        has_state: *mut i32,
        state: *mut oxz_scaler_state,
    ) -> i32;
    pub fn oxz_loader_open(
        path: *const c_char,
        seq_len: u64,
        rank_batch_size: u64,
        rank: u64,
        world: u64,
        first_row: u64,
        end_row: u64,
        device: i32,
        out: *mut *mut oxz_loader,
    ) -> i32;
    pub fn oxz_loader_open_files(
        paths: *const *const c_char,
        n_paths: u32,
        seq_len: u64,
        rank_batch_size: u64,
        rank: u64,
        world: u64,
        spans: *const u64,
        n_spans: u32,
        device: i32,
        out: *mut *mut oxz_loader,
    ) -> i32;
    pub fn oxz_loader_source_rows(loader: *const oxz_loader, rows: *mut u64, cap: u32, n_sources: *mut u32) -> i32;
    pub fn oxz_loader_set_prefetch(loader: *mut oxz_loader, depth: u32) -> i32;
    pub fn oxz_loader_set_row_order(loader: *mut oxz_loader, epoch: u64, perm: *const u32, n: u64) -> i32;
    pub fn oxz_loader_next_rows(loader: *mut oxz_loader, rows: *mut u64) -> i32;
    pub fn oxz_loader_set_mixture(
        loader: *mut oxz_loader,
        weights: *const f64,
        n_weights: u32,
        has_rows_per_epoch: i32,
        rows_per_epoch: u64,
    ) -> i32;
    pub fn oxz_loader_mixture_sources(
        loader: *const oxz_loader,
        out: *mut oxz_mixture_source,
        cap: u32,
        n_sources: *mut u32,
    ) -> i32;
    pub fn oxz_mixture_quotas(weights: *const f64, n_weights: u32, rows: u64, quotas: *mut u64) -> i32;
    pub fn oxz_loader_close(loader: *mut oxz_loader) -> i32;
    pub fn oxz_loader_set_target_mask(
        loader: *mut oxz_loader,
        on: i32,
        target_base: u32,
        always_score: *const u32,
        n_always: u32,
    ) -> i32;
    pub fn oxz_loader_set_document_mask(loader: *mut oxz_loader, on: i32, separator_id: u32) -> i32;
    pub fn oxz_loader_batch_masks(loader: *const oxz_loader, out: *mut oxz_batch_masks) -> i32;
    pub fn oxz_loader_num_rows(loader: *const oxz_loader, rows: *mut u64) -> i32;
    pub fn oxz_loader_position(loader: *const oxz_loader, pos: *mut oxz_data_position) -> i32;
    pub fn oxz_loader_seek(loader: *mut oxz_loader, pos: oxz_data_position) -> i32;
    pub fn oxz_loader_next_batch_async(
        loader: *mut oxz_loader,
        stream: *mut c_void,
        inputs: *mut *mut i64,
        targets: *mut *mut i64,
        rows: *mut u64,
    ) -> i32;
    pub fn oxz_step_weighting(
        local_micro_batches: u64,
        world: i32,
        counts: *const i64,
        micro_batches: *mut u64,
        global_scored: *mut i64,
    ) -> i32;
}
