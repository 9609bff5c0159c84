"""Shared pieces of the parity tests: seeded inputs, the CUDA path and the CPU checker side by side."""
from __future__ import annotations

import numpy as np

import oxidizr_b200 as ox
from oxidizr_b200 import ffi
from oracle import dpstep as orc

NAN = float("nan")


def bits(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32}[a.dtype.itemsize])


def seeded_state(numel, seed=0, grad_std=1e-3, world=1, grad_dtype=ox.BF16):
    """master ~N(0,0.02), m ~N(0,1e-4), v = |N(0,1e-6)|, per-rank grads ~N(0,grad_std) from seed+rank."""
    rng = np.random.default_rng(seed)
    master = [(rng.standard_normal(n) * 0.02).astype(np.float32) for n in numel]
    m = [(rng.standard_normal(n) * 1e-4).astype(np.float32) for n in numel]
    v = [np.abs(rng.standard_normal(n) * 1e-6).astype(np.float32) for n in numel]
    grads = []
    for r in range(world):
        g = np.random.default_rng(seed + 1000 + r)
        grads.append([orc.narrow((g.standard_normal(n) * grad_std).astype(np.float32), grad_dtype) for n in numel])
    return master, m, v, grads


class Pair:
    """One optimizer on the GPU and the checker's state on the CPU, fed the same inputs."""

    def __init__(self, numel, no_decay=None, grad_dtype=ox.BF16, param_dtype=ox.BF16, seed=0, grad_std=1e-3,
                 timestep=0, bucket_bytes=0):
        self.numel = list(numel)
        T = len(numel)
        self.no_decay = list(no_decay) if no_decay is not None else [False] * T
        self.grad_dtype, self.param_dtype = grad_dtype, param_dtype
        master, m, v, grads = seeded_state(numel, seed, grad_std, 1, grad_dtype)
        self.grads = grads[0]
        self.opt = ox.DpOptimizer(numel, self.no_decay, grad_dtype, param_dtype, bucket_bytes=bucket_bytes)
        work = [orc.narrow(p, param_dtype) for p in master] if param_dtype != ox.F32 else None
        self.ref = orc.StepState([p.copy() for p in master], [x.copy() for x in m], [x.copy() for x in v], work,
                                 param_dtype, lr_scale=[1.0] * T, group_wd=[0.0 if nd else NAN for nd in self.no_decay],
                                 timestep=timestep)
        for i in range(T):
            self.opt.import_tensor(ffi.STATE_MASTER, i, master[i])
            self.opt.import_tensor(ffi.STATE_EXP_AVG, i, m[i])
            self.opt.import_tensor(ffi.STATE_EXP_AVG_SQ, i, v[i])
            if work is not None:
                self.opt.import_tensor(ffi.STATE_WORK, i, work[i])
        self.opt.timestep = timestep
        self.set_grads(self.grads)

    def set_grads(self, grads):
        self.grads = grads
        for i, g in enumerate(grads):
            if g is not None:
                self.opt.import_tensor(ffi.STATE_GRADS, i, g)

    def step(self, cfg: ox.StepConfig, present=None):
        res = self.opt.step(cfg, present)
        rg = [g if (present is None or present[i]) else None for i, g in enumerate(self.grads)]
        ocfg = orc.StepConfig(**{k: getattr(cfg, k) for k in orc.StepConfig.__dataclass_fields__})
        ref = orc.step(self.ref, [rg], self.grad_dtype, ocfg)
        return res, ref

    def gpu_state(self):
        T = len(self.numel)
        out = {}
        for key, kind in (("master", ffi.STATE_MASTER), ("exp_avg", ffi.STATE_EXP_AVG), ("exp_avg_sq", ffi.STATE_EXP_AVG_SQ),
                          ("work", ffi.STATE_WORK)):
            out[key] = [self.opt.export_tensor(kind, i) for i in range(T)]
        return out

    def ref_state(self):
        work = self.ref.work if self.ref.work is not None else self.ref.master
        return dict(master=self.ref.master, exp_avg=self.ref.exp_avg, exp_avg_sq=self.ref.exp_avg_sq, work=work)

    def assert_bit_equal(self):
        g, r = self.gpu_state(), self.ref_state()
        for key in g:
            for i, (a, b) in enumerate(zip(g[key], r[key])):
                assert np.array_equal(bits(a), bits(b)), f"{key}[{i}] differs: {np.sum(bits(a) != bits(b))} of {a.size} elements"

    def assert_close(self, rel=1e-6):
        """|gpu - ref| <= rel * (|ref| + rms(ref)) for master and moments.

        The rms term keeps the bound meaningful where a moment passes through zero: its relative error is
        unbounded there although the absolute error is one rounding of a typical element. The reference's own
        cross-run bound has the same shape (1e-6 + 1e-5*|w|, tests/data_parallel.rs:258-262).
        """
        g, r = self.gpu_state(), self.ref_state()
        for key in ("master", "exp_avg", "exp_avg_sq"):
            for i, (a, b) in enumerate(zip(g[key], r[key])):
                if b.size == 0:
                    continue
                b64 = b.astype(np.float64)
                err = np.abs(a.astype(np.float64) - b64)
                bound = rel * (np.abs(b64) + np.sqrt(np.mean(b64 ** 2))) + 1e-30
                assert np.all(err <= bound), f"{key}[{i}]: max err/bound {np.max(err / bound):.3e}"

    def close(self):
        self.opt.destroy()
