"""ctypes declarations of every entry point in include/oxz_dpstep.h.

The library is the product; this file only binds it. There is no fallback: when liboxz_dpstep.so is missing
the import fails with the build command to run.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboxz_dpstep.so")

OK, ERR_INVALID, ERR_CUDA, ERR_NCCL, ERR_STATE, ERR_ABORTED, ERR_UNSUPPORTED, ERR_DATA, ERR_TIMEOUT = range(9)
F32, BF16, F16 = 0, 1, 2
SYNC_SINGLE, SYNC_P2P, SYNC_NCCL, SYNC_COPY, SYNC_REPLICATED = 0, 1, 2, 3, 4
EXCHANGE_NONE, EXCHANGE_COMM, EXCHANGE_MAILBOX = 0, 1, 2
STATE_MASTER, STATE_EXP_AVG, STATE_EXP_AVG_SQ, STATE_WORK, STATE_GRADS = range(5)
DECAY_ALL, SKIP_1D, SKIP_ALL = 0, 1, 2
LR_CONSTANT, LR_COSINE, LR_LINEAR, LR_WSD = range(4)
SHAPE_LINEAR, SHAPE_COSINE, SHAPE_SQRT = range(3)

u8p, u64p, f32p, f64p, i64p, vp = (C.POINTER(C.c_uint8), C.POINTER(C.c_uint64), C.POINTER(C.c_float),
                                   C.POINTER(C.c_double), C.POINTER(C.c_int64), C.c_void_p)


class PlanDesc(C.Structure):
    _fields_ = [("n_tensors", C.c_uint64), ("numel", u64p), ("no_decay", u8p), ("lr_scale", f32p),
                ("grad_dtype", C.c_int32), ("param_dtype", C.c_int32), ("world", C.c_int32), ("rank", C.c_int32),
                ("sync_mode", C.c_int32), ("device", C.c_int32), ("bucket_bytes", C.c_uint64)]


class PlanInfo(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("n_tensors", "numel_total", "padded_total", "tile_elems", "n_buckets",
                                          "bucket_elems", "local_elems", "n_groups")]


class Hyper(C.Structure):
    _fields_ = [(n, C.c_double) for n in ("lr", "beta1", "beta2", "eps", "weight_decay", "max_grad_norm",
                                          "max_grad_value", "target_grad_norm", "loss_scale", "clip_eps")] + \
               [(n, C.c_int32) for n in ("decay_after", "eps_mode", "spike_skip", "reserved")]


class StepResult(C.Structure):
    _fields_ = [("grad_norm", C.c_double), ("reported_norm", C.c_double), ("clip_coef", C.c_double),
                ("overflow", C.c_int32), ("applied", C.c_int32), ("timestep", C.c_uint64)]


class StepProfile(C.Structure):
    _fields_ = [(n, C.c_float) for n in ("collect_ms", "norm_ms", "decide_ms", "update_ms", "publish_ms", "total_ms")]


class ScalerConfig(C.Structure):
    _fields_ = [("initial", C.c_double), ("growth_factor", C.c_double), ("backoff_factor", C.c_double),
                ("growth_interval", C.c_uint64)]


class ScalerState(C.Structure):
    _fields_ = [("scale", C.c_double), ("consecutive_ok", C.c_uint64)]


class SpikeConfig(C.Structure):
    _fields_ = [("window", C.c_uint64), ("z_threshold", C.c_double), ("min_steps", C.c_uint64),
                ("action_warn", C.c_int32), ("reserved", C.c_int32)]


class SpikeState(C.Structure):
    _fields_ = [("mean", C.c_double), ("variance", C.c_double), ("observed", C.c_uint64), ("detected", C.c_uint64),
                ("skipped", C.c_uint64)]


class LrPlanC(C.Structure):
    _fields_ = [("base_lr", C.c_double), ("min_lr_ratio", C.c_double), ("warmup_steps", C.c_uint64),
                ("total_steps", C.c_uint64), ("decay_steps", C.c_uint64), ("schedule", C.c_int32),
                ("decay_shape", C.c_int32)]


class RowLayoutC(C.Structure):
    _fields_ = [("num_rows", C.c_uint64), ("rank_batch_size", C.c_uint64), ("world_size", C.c_uint64)]


class DataPositionC(C.Structure):
    _fields_ = [("epoch", C.c_uint64), ("row", C.c_uint64)]


class ResumeMeta(C.Structure):
    _fields_ = [("step", C.c_uint64), ("has_world_size", C.c_int32), ("has_global_batch_rows", C.c_int32),
                ("has_loss_scale", C.c_int32), ("has_data_position", C.c_int32), ("has_spike_guard", C.c_int32),
                ("has_weight_decay_rule", C.c_int32), ("has_mixture", C.c_int32), ("n_mixture_weights", C.c_uint32),
                ("mixture_rows_per_epoch", C.c_uint64), ("weight_decay_rule", C.c_int32), ("n_no_decay_patterns", C.c_uint32),
                ("world_size", C.c_uint64), ("global_batch_rows", C.c_uint64), ("loss_scale", ScalerState),
                ("data_position", DataPositionC), ("spike_guard", SpikeState), ("checkpoint_file", C.c_char * 512),
                ("optimizer_file", C.c_char * 512)]


class MixtureSource(C.Structure):
    _fields_ = [("weight", C.c_double), ("rows_per_epoch", C.c_uint64), ("train_rows", C.c_uint64)]


class BatchMasks(C.Structure):
    _fields_ = [("loss_mask", C.c_void_p), ("segment_ids", C.c_void_p), ("cu_seqlens", C.c_void_p),
                ("scored", C.POINTER(C.c_uint64)), ("n_segments", C.POINTER(C.c_uint64))]


RankBody = C.CFUNCTYPE(C.c_int32, C.c_int32, C.c_int32, C.c_void_p)

# name -> (restype, argtypes): one row per declaration of include/oxz_dpstep.h
SIGNATURES = {
    "oxz_abi_version": (C.c_uint32, []),
    "oxz_last_error": (C.c_char_p, []),
    "oxz_status_name": (C.c_char_p, [C.c_int32]),
    "oxz_comm_unique_id": (C.c_int32, [u8p]),
    "oxz_comm_init_rank": (C.c_int32, [C.c_int32, C.c_int32, C.c_int32, u8p, C.POINTER(vp)]),
    "oxz_comm_init_all": (C.c_int32, [C.c_int32, C.POINTER(C.c_int32), C.POINTER(vp)]),
    "oxz_comm_init_local": (C.c_int32, [C.c_int32, C.POINTER(C.c_int32), C.c_double, C.POINTER(vp)]),
    "oxz_comm_world_size": (C.c_int32, [vp, C.POINTER(C.c_int32)]),
    "oxz_comm_rank": (C.c_int32, [vp, C.POINTER(C.c_int32)]),
    "oxz_comm_abort": (C.c_int32, [vp]),
    "oxz_comm_destroy": (C.c_int32, [vp]),
    "oxz_allreduce_i64x2": (C.c_int32, [vp, i64p]),
    "oxz_allreduce_f64": (C.c_int32, [vp, f64p, C.c_uint32]),
    "oxz_broadcast": (C.c_int32, [vp, vp, C.c_uint64, C.c_int32]),
    "oxz_barrier": (C.c_int32, [vp]),
    "oxz_run_ranks": (C.c_int32, [C.c_int32, C.POINTER(vp), RankBody, vp, C.POINTER(C.c_int32)]),
    "oxz_set_last_error": (C.c_int32, [C.c_char_p]),
    "oxz_plan_create": (C.c_int32, [C.POINTER(PlanDesc), C.POINTER(vp)]),
    "oxz_plan_destroy": (C.c_int32, [vp]),
    "oxz_plan_query": (C.c_int32, [vp, C.POINTER(PlanInfo)]),
    "oxz_plan_tensor_offsets": (C.c_int32, [vp, u64p]),
    "oxz_plan_bucket": (C.c_int32, [vp, C.c_uint64, C.c_int32, u64p, u64p, u64p, u64p]),
    "oxz_plan_local_index": (C.c_int32, [vp, C.c_int32, C.c_uint64, u64p]),
    "oxz_plan_set_stream": (C.c_int32, [vp, vp]),
    "oxz_state_alloc": (C.c_int32, [vp, vp]),
    "oxz_state_pointers": (C.c_int32, [vp] + [C.POINTER(vp)] * 5),
    "oxz_state_import": (C.c_int32, [vp, C.c_int32, C.c_uint64, vp]),
    "oxz_state_export": (C.c_int32, [vp, C.c_int32, C.c_uint64, vp]),
    "oxz_state_set_timestep": (C.c_int32, [vp, C.c_uint64]),
    "oxz_state_timestep": (C.c_int32, [vp, u64p]),
    "oxz_optimizer_save": (C.c_int32, [vp, vp, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(C.c_uint32), u64p]),
    "oxz_optimizer_load": (C.c_int32, [vp, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(C.c_uint32), u64p]),
    "oxz_grads_flatten_async": (C.c_int32, [vp, C.POINTER(vp), C.c_int32]),
    "oxz_grads_upload_async": (C.c_int32, [vp, C.c_uint64, vp]),
    "oxz_grads_double_buffer": (C.c_int32, [vp, vp]),
    "oxz_grads_upload_next_async": (C.c_int32, [vp, C.c_uint64, C.c_void_p]),
    "oxz_grads_swap": (C.c_int32, [vp]),
    "oxz_step_async": (C.c_int32, [vp, vp, C.POINTER(Hyper), u8p, f64p, C.c_uint32]),
    "oxz_grads_ready_async": (C.c_int32, [vp, vp, C.POINTER(Hyper), u8p, C.c_uint64, C.c_uint64, vp]),
    "oxz_step_wait": (C.c_int32, [vp, C.POINTER(StepResult)]),
    "oxz_step": (C.c_int32, [vp, vp, C.POINTER(Hyper), u8p, f64p, C.c_uint32, C.POINTER(StepResult)]),
    "oxz_plan_launch_geometry": (C.c_int32, [vp] + [C.POINTER(C.c_int32)] * 3),
    "oxz_plan_last_pull_kernel": (C.c_int32, [vp, C.POINTER(C.c_int32)]),
    "oxz_plan_exchange_kind": (C.c_int32, [vp, C.POINTER(C.c_int32)]),
    "oxz_plan_last_update_kernel": (C.c_int32, [vp, C.POINTER(C.c_int32)]),
    "oxz_selftest_bounded_wait": (C.c_int32, [C.c_int32, C.c_uint32, C.POINTER(C.c_int32)]),
    "oxz_grad_norms_per_tensor": (C.c_int32, [vp, vp, C.c_double, C.c_double, f64p]),
    "oxz_plan_set_profile": (C.c_int32, [vp, C.c_int32]),
    "oxz_step_profile_read": (C.c_int32, [vp, C.POINTER(StepProfile)]),
    "oxz_grad_norm": (C.c_int32, [vp, C.c_int32, C.c_uint64, C.c_double, C.c_double, vp, f64p]),
    "oxz_grad_norm_static": (C.c_int32, [vp, C.c_int32, C.c_uint64, C.c_double, C.c_double, C.c_uint32, vp, f64p]),
    "oxz_scaler_check": (C.c_int32, [C.POINTER(ScalerConfig)]),
    "oxz_scaler_init": (C.c_int32, [C.POINTER(ScalerConfig), C.POINTER(ScalerState)]),
    "oxz_scaler_restore": (C.c_int32, [C.POINTER(ScalerState), C.POINTER(ScalerState)]),
    "oxz_scaler_record_step": (C.c_int32, [C.POINTER(ScalerConfig), C.POINTER(ScalerState), C.c_int32, C.c_int32]),
    "oxz_decay_check": (C.c_int32, [C.c_int32, C.POINTER(C.c_char_p), C.c_uint32]),
    "oxz_decay_excludes": (C.c_int32, [C.c_int32, C.POINTER(C.c_char_p), C.c_uint32, C.c_char_p, C.c_uint32,
                                       C.POINTER(C.c_int32)]),
    "oxz_spike_judge": (C.c_int32, [C.POINTER(SpikeConfig), C.POINTER(SpikeState), C.c_uint64, C.c_double,
                                    C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "oxz_lr_at": (C.c_int32, [C.POINTER(LrPlanC), C.c_uint64, f64p]),
    "oxz_loader_open_files": (C.c_int32, [C.POINTER(C.c_char_p), C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64,
                                          C.POINTER(C.c_uint64), C.c_uint32, C.c_int32, C.POINTER(vp)]),
    "oxz_loader_source_rows": (C.c_int32, [vp, C.POINTER(C.c_uint64), C.c_uint32, C.POINTER(C.c_uint32)]),
    "oxz_loader_set_prefetch": (C.c_int32, [vp, C.c_uint32]),
    "oxz_loader_next_rows": (C.c_int32, [vp, C.POINTER(C.c_uint64)]),
    "oxz_loader_set_mixture": (C.c_int32, [vp, C.POINTER(C.c_double), C.c_uint32, C.c_int32, C.c_uint64]),
    "oxz_loader_mixture_sources": (C.c_int32, [vp, C.POINTER(MixtureSource), C.c_uint32, C.POINTER(C.c_uint32)]),
    "oxz_mixture_quotas": (C.c_int32, [C.POINTER(C.c_double), C.c_uint32, C.c_uint64, C.POINTER(C.c_uint64)]),
    "oxz_loader_set_target_mask": (C.c_int32, [vp, C.c_int32, C.c_uint32, C.POINTER(C.c_uint32), C.c_uint32]),
    "oxz_loader_set_document_mask": (C.c_int32, [vp, C.c_int32, C.c_uint32]),
    "oxz_loader_batch_masks": (C.c_int32, [vp, C.POINTER(BatchMasks)]),
    "oxz_meta_load": (C.c_int32, [C.c_char_p, C.POINTER(ResumeMeta)]),
    "oxz_meta_no_decay_pattern": (C.c_int32, [C.c_char_p, C.c_uint32, C.c_char_p, C.c_uint64]),
    "oxz_meta_save": (C.c_int32, [C.c_char_p, C.POINTER(ResumeMeta), C.POINTER(C.c_char_p), C.POINTER(C.c_double)]),
    "oxz_meta_mixture_weights": (C.c_int32, [C.c_char_p, C.POINTER(C.c_double), C.c_uint32, C.POINTER(C.c_uint32)]),
    "oxz_check_mixture_resume": (C.c_int32, [C.c_char_p, C.c_uint64, C.c_int32, C.POINTER(C.c_double), C.c_uint32, C.c_uint64]),
    "oxz_check_resume_world": (C.c_int32, [C.c_char_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_char_p, C.c_uint64]),
    "oxz_read_loss_scale_state": (C.c_int32, [C.c_char_p, C.c_uint64, C.POINTER(C.c_int32), C.POINTER(ScalerState)]),
    "oxz_rows_check": (C.c_int32, [C.POINTER(RowLayoutC)]),
    "oxz_rows_advance": (C.c_int32, [C.POINTER(RowLayoutC), DataPositionC, C.c_uint64, C.POINTER(DataPositionC)]),
    "oxz_rows_next_window": (C.c_int32, [C.POINTER(RowLayoutC), DataPositionC, C.c_uint64, C.c_uint64, C.c_uint64,
                                         C.POINTER(C.c_uint32), C.c_uint64, u64p, i64p, i64p,
                                         C.POINTER(DataPositionC)]),
    "oxz_rows_batch_epoch": (C.c_int32, [C.POINTER(RowLayoutC), DataPositionC, u64p]),
    "oxz_rows_check_permutation": (C.c_int32, [C.POINTER(C.c_uint32), C.c_uint64]),
    "oxz_rows_next_window_ordered": (C.c_int32, [C.POINTER(RowLayoutC), DataPositionC, C.c_uint64, C.c_uint64, C.c_uint64,
                                                 C.POINTER(C.c_uint32), C.c_uint64, C.c_uint64, C.POINTER(C.c_uint32), C.c_uint64,
                                                 u64p, i64p, i64p, C.POINTER(DataPositionC)]),
    "oxz_loader_set_row_order": (C.c_int32, [vp, C.c_uint64, C.POINTER(C.c_uint32), C.c_uint64]),
    "oxz_loader_open": (C.c_int32, [C.c_char_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64,
                                    C.c_int32, C.POINTER(vp)]),
    "oxz_loader_close": (C.c_int32, [vp]),
    "oxz_loader_num_rows": (C.c_int32, [vp, u64p]),
    "oxz_loader_position": (C.c_int32, [vp, C.POINTER(DataPositionC)]),
    "oxz_loader_seek": (C.c_int32, [vp, DataPositionC]),
    "oxz_loader_next_batch_async": (C.c_int32, [vp, vp, C.POINTER(vp), C.POINTER(vp), u64p]),
    "oxz_step_weighting": (C.c_int32, [C.c_uint64, C.c_int32, i64p, u64p, i64p]),
}


class OxzError(RuntimeError):
    """A non-zero oxz_status, with the library's message. Mirrors boostr::error::Error on the Rust side."""

    def __init__(self, status: int, message: str):
        super().__init__(f"{status_name(status)}: {message}")
        self.status = status
        self.message = message


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m oxidizr_b200.build` (nvcc, sm_100a). "
                "There is no CPU fallback for this path.")
        L = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        if L.oxz_abi_version() != 1:
            raise ImportError(f"liboxz_dpstep.so has ABI {L.oxz_abi_version()}, this binding expects 1")
        _lib = L
    return _lib


def status_name(status: int) -> str:
    return lib().oxz_status_name(status).decode()


def check(status: int) -> None:
    if status != OK:
        raise OxzError(status, lib().oxz_last_error().decode())
