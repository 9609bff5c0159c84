"""ctypes binding of the CPU checker in ``dpstep_oracle.c``.

Test infrastructure only: imported by ``tests/``, by ``__graft_entry__.smoke`` and by
``bench.py``'s CPU-baseline and reference arms. The product package never imports it.

PARITY UNPINNED for the AdamW arithmetic (no reference test fixes a number); pinned for
everything the reference's own tests hold known answers for. See ``dpstep_oracle.c``.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboxz_oracle.so")

F32, BF16, F16 = 0, 1, 2
NAN = float("nan")


def build(force: bool = False) -> str:
    """Compile the checker with the Makefile beside it; returns the path of the library."""
    src = os.path.join(_HERE, "dpstep_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return _SO


class AdamScalars(C.Structure):
    _fields_ = [
        ("beta1", C.c_float), ("one_minus_beta1", C.c_float),
        ("beta2", C.c_float), ("one_minus_beta2", C.c_float),
        ("eps", C.c_float), ("bias2_sqrt", C.c_float),
        ("step_size", C.c_float), ("decay_mul", C.c_float),
        ("decay_after", C.c_int32), ("eps_mode", C.c_int32),
    ]


class Hyper(C.Structure):
    _fields_ = [
        ("lr", C.c_double), ("beta1", C.c_double), ("beta2", C.c_double), ("eps", C.c_double),
        ("weight_decay", C.c_double), ("max_grad_norm", C.c_double), ("max_grad_value", C.c_double),
        ("target_grad_norm", C.c_double), ("loss_scale", C.c_double), ("clip_eps", C.c_double),
        ("decay_after", C.c_int32), ("eps_mode", C.c_int32), ("spike_skip", C.c_int32),
        ("absent_mode", C.c_int32),
    ]


class Result(C.Structure):
    _fields_ = [
        ("grad_norm", C.c_double), ("reported_norm", C.c_double), ("clip_coef", C.c_double),
        ("overflow", C.c_int32), ("applied", C.c_int32), ("timestep", C.c_uint64),
    ]


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        vp, sz = C.c_void_p, C.c_size_t
        L.orc_f32_to_bf16.argtypes = [vp, vp, sz]
        L.orc_f32_to_f16.argtypes = [vp, vp, sz]
        L.orc_widen.argtypes = [vp, C.c_int, vp, sz]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        L.orc_sum_ranks.argtypes = [C.POINTER(vp), C.c_int, C.c_int, sz, vp]
        L.orc_unscale.argtypes = [vp, C.c_int, sz, C.c_double, vp]
        L.orc_sumsq.argtypes = [vp, sz]
        L.orc_sumsq.restype = C.c_double
        L.orc_clamp.argtypes = [vp, sz, C.c_double]
        L.orc_scale.argtypes = [vp, sz, C.c_float]
        L.orc_clip_gradients.argtypes = [sz, C.POINTER(sz), C.POINTER(vp), vp, C.c_double, C.c_double, C.c_double,
                                         C.POINTER(C.c_double)]
        L.orc_clip_gradients.restype = C.c_double
        L.orc_adam_prepare.argtypes = [C.c_double] * 6 + [C.c_uint64, C.c_int32, C.c_int32, C.POINTER(AdamScalars)]
        L.orc_adamw.argtypes = [vp, vp, vp, vp, sz, C.POINTER(AdamScalars), vp, C.c_int]
        L.orc_step.argtypes = [sz, C.POINTER(sz), C.POINTER(vp), C.c_int, C.c_int, C.POINTER(vp), C.POINTER(vp),
                               C.POINTER(vp), C.POINTER(vp), C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double),
                               C.c_uint64, C.POINTER(Hyper), vp, C.POINTER(Result)]
        _lib = L
    return _lib


def _ptr(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


def np_dtype(code: int):
    return {F32: np.float32, BF16: np.uint16, F16: np.uint16}[code]


def to_bf16(x: np.ndarray) -> np.ndarray:
    """f32 -> bf16 bit patterns (uint16), round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_bf16(_ptr(x), _ptr(out), x.size)
    return out


def to_f16(x: np.ndarray) -> np.ndarray:
    """f32 -> f16 bit patterns (uint16), round to nearest even."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().orc_f32_to_f16(_ptr(x), _ptr(out), x.size)
    return out


def narrow(x: np.ndarray, code: int) -> np.ndarray:
    if code == F32:
        return np.ascontiguousarray(x, dtype=np.float32)
    return to_bf16(x) if code == BF16 else to_f16(x)


def widen(x: np.ndarray, code: int) -> np.ndarray:
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, dtype=np.float32)
    lib().orc_widen(_ptr(x), code, _ptr(out), x.size)
    return out


def sum_ranks(rank_grads: list[np.ndarray], code: int) -> np.ndarray:
    n = rank_grads[0].size
    arr = (C.c_void_p * len(rank_grads))(*[_ptr(g) for g in rank_grads])
    out = np.empty(n, dtype=np.float32)
    lib().orc_sum_ranks(arr, len(rank_grads), code, n, _ptr(out))
    return out


def unscale(g: np.ndarray, code: int, scale: float) -> np.ndarray:
    out = np.empty(g.size, dtype=np.float32)
    lib().orc_unscale(_ptr(np.ascontiguousarray(g)), code, g.size, scale, _ptr(out))
    return out


def sumsq(g: np.ndarray) -> float:
    g = np.ascontiguousarray(g, dtype=np.float32)
    return float(lib().orc_sumsq(_ptr(g), g.size))


def clip_gradients(grads: list[np.ndarray], max_grad_value: float, max_grad_norm: float, clip_eps: float = 1e-6,
                   present: list[bool] | None = None) -> tuple[float, float]:
    """clip_gradients (src/grad_clip.rs:36-56) in place on f32 arrays, through the function the checker's step calls.
    Returns (the norm the norm clip measured, the coefficient applied)."""
    T = len(grads)
    for g in grads:
        assert g.dtype == np.float32 and g.flags["C_CONTIGUOUS"]
    numel = (C.c_size_t * T)(*[g.size for g in grads])
    ptrs = (C.c_void_p * T)(*[_ptr(g) for g in grads])
    pres = np.array([1 if (present is None or present[i]) else 0 for i in range(T)], dtype=np.uint8)
    coef = C.c_double(1.0)
    norm = lib().orc_clip_gradients(T, numel, ptrs, _ptr(pres), max_grad_value, max_grad_norm, clip_eps, C.byref(coef))
    return float(norm), float(coef.value)


def adam_prepare(lr, lr_scale, beta1, beta2, eps, weight_decay, t, decay_after=0, eps_mode=0) -> AdamScalars:
    s = AdamScalars()
    lib().orc_adam_prepare(lr, lr_scale, beta1, beta2, eps, weight_decay, t, decay_after, eps_mode, C.byref(s))
    return s


def adamw(p, m, v, g, s: AdamScalars, work=None, work_dtype=F32):
    """In-place AdamW on f32 arrays p, m, v with the f32 gradient g."""
    lib().orc_adamw(_ptr(p), _ptr(m), _ptr(v), _ptr(g), p.size, C.byref(s),
                    _ptr(work) if work is not None else None, work_dtype)


@dataclass
class StepConfig:
    """The trainer keys the step reads (src/config.rs:40-62 defaults)."""
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-6
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    max_grad_value: float = NAN
    target_grad_norm: float = NAN
    loss_scale: float = NAN
    clip_eps: float = 1e-6
    decay_after: int = 0
    eps_mode: int = 0
    spike_skip: bool = False

    def hyper(self) -> Hyper:
        return Hyper(self.lr, self.beta1, self.beta2, self.eps, self.weight_decay, self.max_grad_norm,
                     self.max_grad_value, self.target_grad_norm, self.loss_scale, self.clip_eps,
                     self.decay_after, self.eps_mode, int(self.spike_skip), 0)


@dataclass
class StepState:
    """Per-tensor optimizer state of the checker: f32 master, moments and the working weights."""
    master: list[np.ndarray]
    exp_avg: list[np.ndarray]
    exp_avg_sq: list[np.ndarray]
    work: list[np.ndarray] | None
    work_dtype: int = F32
    lr_scale: list[float] = field(default_factory=list)
    group_wd: list[float] = field(default_factory=list)  # NaN = base weight decay
    timestep: int = 0


def step(state: StepState, rank_grads: list[list[np.ndarray | None]], grad_dtype: int, cfg: StepConfig) -> Result:
    """One optimizer step (src/trainer.rs:515-695). rank_grads[r][i] is rank r's gradient of tensor i or None."""
    T = len(state.master)
    world = len(rank_grads)
    numel = (C.c_size_t * T)(*[a.size for a in state.master])
    gp = (C.c_void_p * (T * world))()
    keep = []
    for r in range(world):
        for i in range(T):
            g = rank_grads[r][i]
            if g is not None:
                g = np.ascontiguousarray(g)
                keep.append(g)
                gp[r * T + i] = _ptr(g)
            else:
                gp[r * T + i] = None
    arr = lambda xs: (C.c_void_p * T)(*[_ptr(x) for x in xs])
    lr_scale = (C.c_double * T)(*(state.lr_scale or [1.0] * T))
    group_wd = (C.c_double * T)(*(state.group_wd or [NAN] * T))
    scratch = np.empty(max(1, sum(a.size for a in state.master)), dtype=np.float32)
    res = Result()
    h = cfg.hyper()
    lib().orc_step(T, numel, gp, world, grad_dtype, arr(state.master), arr(state.exp_avg), arr(state.exp_avg_sq),
                   arr(state.work) if state.work is not None else None, state.work_dtype, lr_scale, group_wd,
                   state.timestep, C.byref(h), _ptr(scratch), C.byref(res))
    state.timestep = int(res.timestep)
    return res


def is_finite(x: float) -> bool:
    return math.isfinite(x)
