"""The allocation-free norm entry point against the allocating one, through the C ABI.

oxz_grad_norm_static is for hosts whose device memory is already spoken for, or whose step loop must not run into
the device-wide synchronisation of cudaMalloc/cudaFree; its scratch is a static device array inside the library.
This file is collected last, so a run that stops at the first failure has already run every other test; it passes
alone in a fresh process (its first call does the per-device set-up) and after the others.
"""
import math

import numpy as np
import pytest

import oxidizr_b200 as ox
from oracle import dpstep as orc

pytestmark = pytest.mark.gpu

NORM_RTOL = 1e-5  # the bound the other norm tests use


def test_static_scratch_norm_matches_the_allocating_entry_point_on_two_calls_in_a_row():
    import torch
    rng = np.random.default_rng(77)
    # two calls in a row on different inputs; the second is smaller, so anything left in the shared scratch by the
    # first call would show if a stage read it
    cases = [(ox.BF16, 3_000_003, dict(loss_scale=float("nan"), max_grad_value=float("nan"))),
             (ox.F16, 4_099, dict(loss_scale=1024.0, max_grad_value=2e-6))]
    for dtype, n, kw in cases:
        g = orc.narrow((rng.standard_normal(n) * 1e-3).astype(np.float32), dtype)
        d = torch.from_numpy(g.view(np.int16)).cuda()
        want = ox.compute_grad_norm(d.data_ptr(), dtype, n, **kw)
        got = ox.compute_grad_norm_static(d.data_ptr(), dtype, n, **kw)
        assert math.isfinite(want) and want > 0.0
        assert abs(got - want) <= NORM_RTOL * want, (got, want)
        # and against the CPU checker: widen, unscale, clamp, f32 squares summed in f64 (src/grad_clip.rs:47-55)
        x = orc.widen(g, dtype)
        if not math.isnan(kw["loss_scale"]):
            x = orc.unscale(x, orc.F32, kw["loss_scale"])
        if not math.isnan(kw["max_grad_value"]):
            x = np.clip(x, np.float32(-kw["max_grad_value"]), np.float32(kw["max_grad_value"]))
        cpu = math.sqrt(orc.sumsq(x))
        assert abs(got - cpu) <= NORM_RTOL * cpu, (got, cpu)
        # a caller-chosen, smaller launch uses fewer partial-sum slots of the same array
        got_small = ox.compute_grad_norm_static(d.data_ptr(), dtype, n, clusters=7, **kw)
        assert abs(got_small - want) <= NORM_RTOL * want, (got_small, want)
    # a non-finite element still gives a non-finite norm
    bad = np.ones(1000, np.float32)
    bad[999] = np.inf
    d = torch.from_numpy(bad).cuda()
    assert not math.isfinite(ox.compute_grad_norm_static(d.data_ptr(), ox.F32, bad.size))
    # beyond the array's capacity: refused with the limit in the message, nothing launched
    with pytest.raises(ox.OxzError, match=f"at most {ox.dpstep.STATIC_NORM_MAX_CLUSTERS}"):
        ox.compute_grad_norm_static(d.data_ptr(), ox.F32, bad.size, clusters=ox.dpstep.STATIC_NORM_MAX_CLUSTERS + 1)
