"""oxidizr_b200: a B200-native data-parallel optimizer step for oxidizr, behind a C ABI.

The product is ``liboxz_dpstep.so`` (hand-written sm_100a CUDA + NCCL, declared in ``include/oxz_dpstep.h``).
This package binds it with ctypes and mirrors the reference's host-side interface for the path.
"""
from ._ffi import BF16, F16, F32, SYNC_COPY, SYNC_NCCL, SYNC_P2P, SYNC_REPLICATED, SYNC_SINGLE, OxzError, lib  # noqa: F401
from . import _ffi as ffi  # noqa: F401
from .dpstep import (CheckpointMeta, MixtureRecord, check_mixture_resume, Communicator, DataPosition, DecayPlan, DpOptimizer, GradScalerState, LitDataLoader, LitTrainerStep,  # noqa: F401
                     LossScaleConfig, LossScaler, LrPlan, RowLayout, SpikeGuard, SpikeGuardConfig, SpikeGuardState, StepConfig,
                     TensorInfo, TrainerConfig, WeightDecaySpec, check_resume_world, compute_grad_norm, mixture_quotas,
                     compute_grad_norm_static, diagnose_bad_gradients, read_loss_scale_state, run_ranks, selftest_bounded_wait,
                     step_weighting)
