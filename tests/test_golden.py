"""The committed golden vectors (tests/golden/step_vectors.npz, made by tests/golden/make_golden.py with the CPU
checker): the checker must still reproduce them bit for bit (CPU), and the CUDA path must match them (GPU)."""
import os

import numpy as np
import pytest

import oxidizr_b200 as ox
from oxidizr_b200 import ffi
from oracle import dpstep as orc
from tests.golden import make_golden as mg
from tests.helpers import bits

GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "step_vectors.npz"))


@pytest.mark.parametrize("case", list(mg.CASES))
def test_checker_reproduces_the_golden_vectors(case):
    st, results = mg.run(case)
    assert np.array_equal(results, GOLD[f"{case}/results"], equal_nan=True)
    for i in range(len(mg.NUMEL)):
        for key, arr in (("master", st.master), ("exp_avg", st.exp_avg), ("exp_avg_sq", st.exp_avg_sq)):
            assert np.array_equal(bits(arr[i]), bits(GOLD[f"{case}/{key}{i}"])), (key, i)
        if st.work is not None:
            assert np.array_equal(st.work[i], GOLD[f"{case}/work{i}"])


@pytest.mark.gpu
@pytest.mark.parametrize("case", list(mg.CASES))
def test_cuda_path_matches_the_golden_vectors(case):
    gd, pd, world, std, kw, steps = mg.CASES[case]
    master, m, v, grads = mg.inputs(case)
    from concurrent.futures import ThreadPoolExecutor
    comms = ox.Communicator.local_group(world, [0] * world, timeout=60.0) if world > 1 else [None]
    pool = ThreadPoolExecutor(world)

    def make(r):
        opt = ox.DpOptimizer(mg.NUMEL, mg.NO_DECAY, gd, pd, world=world, rank=r, comm=comms[r], bucket_bytes=2048)
        for i in range(len(mg.NUMEL)):
            opt.import_tensor(ffi.STATE_MASTER, i, master[i])
            opt.import_tensor(ffi.STATE_EXP_AVG, i, m[i])
            opt.import_tensor(ffi.STATE_EXP_AVG_SQ, i, v[i])
            opt.import_tensor(ffi.STATE_WORK, i, orc.narrow(master[i], pd))
            opt.import_tensor(ffi.STATE_GRADS, i, grads[r][i])
        return opt
    opts = list(pool.map(make, range(world)))
    want = GOLD[f"{case}/results"]
    for s in range(steps):
        results = list(pool.map(lambda r: opts[r].step(ox.StepConfig(**kw)), range(world)))
        for res in results:
            assert (res.overflow, res.applied, res.timestep) == tuple(int(x) for x in want[s][3:6])
            assert abs(res.grad_norm - want[s][0]) <= 1e-5 * want[s][0]
            assert abs(res.reported_norm - want[s][1]) <= 1e-5 * want[s][1]
            assert abs(res.clip_coef - want[s][2]) <= 1e-6 * want[s][2]
    exact = want[-1][2] == 1.0  # unclipped: bit for bit
    for i, n in enumerate(mg.NUMEL):
        for key, kind in (("master", ffi.STATE_MASTER), ("exp_avg", ffi.STATE_EXP_AVG), ("exp_avg_sq", ffi.STATE_EXP_AVG_SQ)):
            got = np.full(n, np.nan, np.float32)
            for opt in opts:
                opt.export_tensor(kind, i, got)
            ref = GOLD[f"{case}/{key}{i}"]
            if exact:
                assert np.array_equal(bits(got), bits(ref)), (key, i)
            else:
                r64 = ref.astype(np.float64)
                assert np.all(np.abs(got - r64) <= 1e-6 * (np.abs(r64) + np.sqrt(np.mean(r64 ** 2)))), (key, i)
    for opt in opts:
        opt.destroy()
    for c in comms:
        if c is not None:
            c.destroy()
