"""Generates tests/golden/step_vectors.npz with the CPU checker (oracle/).

The reference itself cannot run here (Rust, un-vendored arithmetic crates), so these vectors do not come from it:
they freeze the checker's outputs on small seeded cases, so that a later change to the checker or to the kernels
shows up as a diff against committed numbers. Run from the repository root: python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import dpstep as orc  # noqa: E402

NAN = float("nan")
NUMEL = [37, 256, 1000, 5]
NO_DECAY = [True, False, False, True]

CASES = {
    # name: (grad dtype, param dtype, world, grad std, config overrides, steps)
    "bf16_clip": (orc.BF16, orc.BF16, 1, 1.0, dict(max_grad_norm=1.0), 2),
    "bf16_noclip_w2": (orc.BF16, orc.BF16, 2, 1e-3, dict(max_grad_norm=1e9, eps=1e-8), 2),
    "f16_scaled": (orc.F16, orc.F16, 1, 1e-3 * 1024.0, dict(loss_scale=1024.0, max_grad_norm=1e9), 1),
    "f32_value_target": (orc.F32, orc.F32, 1, 1.0, dict(max_grad_value=0.5, max_grad_norm=2.0, target_grad_norm=0.5), 1),
    # both norm clips fire on gradients so small that the epsilon of the first coefficient shows in the second
    "f32_both_clips_small": (orc.F32, orc.F32, 1, 4e-5, dict(max_grad_norm=1e-3, target_grad_norm=5e-4), 1),
}


def inputs(case):
    gd, pd, world, std, _, _ = CASES[case]
    rng = np.random.default_rng(sum(map(ord, case)))
    master = [(rng.standard_normal(n) * 0.02).astype(np.float32) for n in NUMEL]
    m = [(rng.standard_normal(n) * 1e-4).astype(np.float32) for n in NUMEL]
    v = [np.abs(rng.standard_normal(n) * 1e-6).astype(np.float32) for n in NUMEL]
    grads = [[orc.narrow((rng.standard_normal(n) * std).astype(np.float32), gd) for n in NUMEL] for _ in range(world)]
    return master, m, v, grads


def run(case):
    gd, pd, world, std, kw, steps = CASES[case]
    master, m, v, grads = inputs(case)
    work = [orc.narrow(p, pd) for p in master] if pd != orc.F32 else None
    st = orc.StepState([p.copy() for p in master], [x.copy() for x in m], [x.copy() for x in v], work, pd,
                       lr_scale=[1.0] * len(NUMEL), group_wd=[0.0 if nd else NAN for nd in NO_DECAY])
    norms = []
    for _ in range(steps):
        res = orc.step(st, grads, gd, orc.StepConfig(**kw))
        norms.append((res.grad_norm, res.reported_norm, res.clip_coef, res.overflow, res.applied, res.timestep))
    return st, np.array(norms, dtype=np.float64)


def main():
    out = {}
    for case in CASES:
        st, norms = run(case)
        out[f"{case}/results"] = norms
        for i in range(len(NUMEL)):
            out[f"{case}/master{i}"] = st.master[i]
            out[f"{case}/exp_avg{i}"] = st.exp_avg[i]
            out[f"{case}/exp_avg_sq{i}"] = st.exp_avg_sq[i]
            if st.work is not None:
                out[f"{case}/work{i}"] = st.work[i]
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "step_vectors.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
