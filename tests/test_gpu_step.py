"""Parity of the CUDA path with the CPU checker on the same seeded inputs, through the C ABI.

Bars: the skip/overflow decision bit-exact; the global norm within 1e-5 relative; parameters and moments within
1e-6 relative per step (bit-exact whenever the clip coefficient is 1), within 1e-4 after 100 steps.
"""
import math

import numpy as np
import pytest

import oxidizr_b200 as ox
from oxidizr_b200 import ffi
from oracle import dpstep as orc
from tests.helpers import NAN, Pair, bits, seeded_state

pytestmark = pytest.mark.gpu

NORM_RTOL = 1e-5
RAGGED = [1, 7, 8, 9, 255, 256, 257, 1023, 1025, 4096, 100003, 0, 33]
DTYPES = [(ox.BF16, ox.BF16), (ox.F16, ox.F16), (ox.F32, ox.F32), (ox.F32, ox.BF16)]


def torch_dev(arr: np.ndarray):
    import torch
    return torch.from_numpy(arr).cuda()


@pytest.mark.parametrize("dtype", [ox.F32, ox.BF16, ox.F16])
@pytest.mark.parametrize("n", [1, 7, 8, 9, 1023, 1025, 262144 + 5, 3_000_001])
def test_grad_norm_matches_checker(dtype, n):
    import torch
    rng = np.random.default_rng(n)
    g = orc.narrow((rng.standard_normal(n) * 1e-3).astype(np.float32), dtype)
    d = torch_dev(g)
    got = ox.compute_grad_norm(d.data_ptr(), dtype, n)
    want = math.sqrt(orc.sumsq(orc.widen(g, dtype)))
    assert abs(got - want) <= NORM_RTOL * want
    # with a loss scale and a value clamp
    got = ox.compute_grad_norm(d.data_ptr(), dtype, n, loss_scale=64.0, max_grad_value=1e-5)
    u = orc.unscale(g, dtype, 64.0)
    orc.lib().orc_clamp(u.ctypes.data, u.size, 1e-5)
    want = math.sqrt(orc.sumsq(u))
    assert abs(got - want) <= NORM_RTOL * want


def test_grad_norm_known_answers():
    # src/grad_clip.rs:118-128 and :82-96 on the GPU
    d = torch_dev(np.array([3.0, 4.0], np.float32))
    assert abs(ox.compute_grad_norm(d.data_ptr(), ox.F32, 2) - 5.0) < 1e-6
    d = torch_dev(np.array([1e15, -1e15, 0.25, -7e14, 3.0], np.float32))
    got = ox.compute_grad_norm(d.data_ptr(), ox.F32, 5, max_grad_value=0.5)
    assert abs(got - math.sqrt(4.0 * 0.25 + 0.0625)) < 1e-6
    # each square fits f32, their sum does not: the norm must stay finite (no false overflow)
    d = torch_dev(np.full(64, 1.5e19, np.float32))
    got = ox.compute_grad_norm(d.data_ptr(), ox.F32, 64)
    assert math.isfinite(got) and abs(got - 1.5e19 * 8.0) <= 1e-5 * got


@pytest.mark.parametrize("bad", [float("nan"), float("inf"), float("-inf")])
@pytest.mark.parametrize("clamp", [NAN, 0.5])
@pytest.mark.parametrize("pos", [0, 1000, 4095])
def test_non_finite_gradient_gives_non_finite_norm(bad, clamp, pos):
    # src/grad_clip.rs:130-143: the clamp must not hide it
    g = np.ones(4096, np.float32)
    g[pos] = bad
    d = torch_dev(g)
    got = ox.compute_grad_norm(d.data_ptr(), ox.F32, g.size, max_grad_value=clamp)
    assert not math.isfinite(got)
    assert math.isnan(got) == math.isnan(bad)


@pytest.mark.parametrize("gd,pd", DTYPES)
def test_step_is_bit_exact_without_clipping(gd, pd):
    no_decay = [n < 300 for n in RAGGED]
    pair = Pair(RAGGED, no_decay, gd, pd, seed=3, timestep=0)
    cfg = ox.StepConfig(lr=3e-4, eps=1e-8, max_grad_norm=1e9)
    for _ in range(3):
        res, ref = pair.step(cfg)
        assert (res.overflow, res.applied, res.timestep) == (ref.overflow, ref.applied, ref.timestep) == (0, 1, res.timestep)
        assert abs(res.grad_norm - ref.grad_norm) <= NORM_RTOL * ref.grad_norm
        assert res.clip_coef == 1.0 == ref.clip_coef
        pair.assert_bit_equal()
    assert pair.opt.timestep == 3
    pair.close()


@pytest.mark.parametrize("gd,pd", DTYPES)
def test_step_with_norm_clip_matches(gd, pd):
    pair = Pair(RAGGED, None, gd, pd, seed=4, grad_std=1.0)
    res, ref = pair.step(ox.StepConfig(max_grad_norm=1.0))
    assert ref.clip_coef < 1.0 and abs(res.clip_coef - ref.clip_coef) <= 1e-6 * ref.clip_coef
    assert abs(res.grad_norm - ref.grad_norm) <= NORM_RTOL * ref.grad_norm
    assert res.reported_norm == 1.0 == ref.reported_norm
    pair.assert_close(1e-6)
    pair.close()


def test_value_clamp_then_norm_clip_then_target():
    pair = Pair([5000, 77], [False, True], ox.F32, ox.F32, seed=5, grad_std=1.0)
    cfg = ox.StepConfig(max_grad_value=0.5, max_grad_norm=2.0, target_grad_norm=0.5)
    res, ref = pair.step(cfg)
    assert abs(res.grad_norm - ref.grad_norm) <= NORM_RTOL * ref.grad_norm
    assert abs(res.clip_coef - ref.clip_coef) <= 1e-6 * ref.clip_coef
    assert res.reported_norm == ref.reported_norm == 0.5
    pair.assert_close(1e-6)
    pair.close()


def test_both_clips_fire_on_small_gradients_the_second_measures_again():
    # src/trainer.rs:635-645: the second norm clip measures the gradients the first one scaled. With a norm near 1e-3
    # the epsilon of the first coefficient leaves them 5e-4 under max_grad_norm, which target / (max + eps) would miss
    # by 500 times the tolerance; the checker measures again, the GPU forms c1 * norm.
    pair = Pair([5000, 77], [False, True], ox.F32, ox.F32, seed=15, grad_std=2e-5)
    cfg = ox.StepConfig(max_grad_norm=1e-3, target_grad_norm=5e-4)
    res, ref = pair.step(cfg)
    assert 1.2e-3 < ref.grad_norm < 1.7e-3
    closed_form = float(np.float32(1e-3 / (ref.grad_norm + 1e-6))) * float(np.float32(5e-4 / (1e-3 + 1e-6)))
    assert abs(closed_form - ref.clip_coef) > 1e-4 * ref.clip_coef  # the case does tell the two forms apart
    assert abs(res.clip_coef - ref.clip_coef) <= 1e-6 * ref.clip_coef
    assert abs(res.grad_norm - ref.grad_norm) <= NORM_RTOL * ref.grad_norm
    assert res.reported_norm == ref.reported_norm == 5e-4
    pair.assert_close(1e-6)
    pair.close()


@pytest.mark.parametrize("gd,pd", DTYPES)
@pytest.mark.parametrize("variant", ["1", "2", "3", "4", "5"])
def test_every_form_of_the_update_kernel_gives_the_same_bits(monkeypatch, variant, gd, pd):
    # OXZ_ADAM_VARIANT: other launch shapes (1, 2), 256-bit stores of the 16-bit weights (3), inputs staged through
    # shared memory by bulk asynchronous copies (4). Same arithmetic: the state must come out bit for bit the same.
    sizes = RAGGED + [8 * 256 * 5 + 77]  # more than a few whole 8-tile chunks for the staged form
    base = Pair(sizes, [n < 300 for n in sizes], gd, pd, seed=17, grad_std=1.0)
    base.step(ox.StepConfig(max_grad_norm=1.0, loss_scale=4.0, max_grad_value=3.0))
    want = base.gpu_state()
    base.close()
    monkeypatch.setenv("OXZ_ADAM_VARIANT", variant)
    other = Pair(sizes, [n < 300 for n in sizes], gd, pd, seed=17, grad_std=1.0)
    other.step(ox.StepConfig(max_grad_norm=1.0, loss_scale=4.0, max_grad_value=3.0))
    got = other.gpu_state()
    other.close()
    for key in want:
        for i, (a, b) in enumerate(zip(got[key], want[key])):
            assert np.array_equal(bits(a), bits(b)), (key, i)


@pytest.mark.parametrize("gd", [ox.BF16, ox.F16, ox.F32])
def test_per_tensor_norms_name_the_offending_tensors(gd):
    # grad_norm_for_tensor for every parameter (src/trainer.rs:933-937), as diagnose_bad_gradients reads it after a
    # non-finite norm (src/trainer.rs:990-1020)
    pair = Pair(RAGGED, None, gd, gd if gd != ox.F32 else ox.F32, seed=16)
    g = [x.copy() for x in pair.grads]
    inf_bits = {ox.BF16: 0x7f80, ox.F16: 0x7c00}
    if gd == ox.F32:
        g[9][17], g[10][99999] = np.float32(np.inf), np.float32(np.nan)
    else:
        g[9][17] = inf_bits[gd]
        g[10][99999] = inf_bits[gd] | 0x0040 | 1  # a NaN pattern of either 16-bit type
    pair.set_grads(g)
    present = [True] * len(RAGGED)
    present[4] = False
    res, ref = pair.step(ox.StepConfig(loss_scale=8.0), present)
    assert res.overflow == 1 and res.applied == 0 and ref.overflow == 1
    norms = pair.opt.grad_norms_per_tensor(loss_scale=8.0)
    assert norms[4] == -1.0 and norms[11] == 0.0
    assert math.isinf(norms[9]) and math.isnan(norms[10])
    for i in (0, 1, 2, 3, 5, 6, 7, 8, 12):
        want = math.sqrt(orc.sumsq(orc.unscale(g[i], gd, 8.0)))
        assert abs(norms[i] - want) <= NORM_RTOL * want, (i, norms[i], want)
    names = [f"model.t{i}.weight" for i in range(len(RAGGED))]
    assert [n for n, _ in ox.diagnose_bad_gradients(names, norms)] == ["model.t9.weight", "model.t10.weight"] or \
        [n for n, _ in ox.diagnose_bad_gradients(names, norms)] == ["model.t10.weight", "model.t9.weight"]
    pair.close()


@pytest.mark.parametrize("switch", [dict(decay_after=1), dict(eps_mode=1), dict(clip_eps=0.0)])
def test_unpinned_forms_follow_their_switches(switch):
    pair = Pair([3000, 10], [False, True], ox.BF16, ox.BF16, seed=6)
    res, ref = pair.step(ox.StepConfig(max_grad_norm=1e9, **switch))
    pair.assert_bit_equal()
    pair.close()


@pytest.mark.parametrize("bad", [float("inf"), float("nan")])
def test_overflow_step_changes_nothing(bad):
    # tests/loss_scale.rs:118-176: parameters, moments and the timestep keep their bits; the norm is not finite
    pair = Pair([2000, 300], None, ox.F16, ox.F16, seed=7, timestep=5)
    before = pair.gpu_state()
    g = [x.copy() for x in pair.grads]
    g[1][123] = np.array([bad], np.float16).view(np.uint16)[0]
    pair.set_grads(g)
    res, ref = pair.step(ox.StepConfig(loss_scale=65536.0))
    assert (res.overflow, res.applied, res.timestep) == (1, 0, 5) == (ref.overflow, ref.applied, ref.timestep)
    assert not math.isfinite(res.grad_norm) and not math.isfinite(res.reported_norm)
    after = pair.gpu_state()
    for key in before:
        for a, b in zip(before[key], after[key]):
            assert np.array_equal(bits(a), bits(b)), key
    # the next clean step applies and counts
    pair.set_grads(seeded_state([2000, 300], 7, 1e-3, 1, ox.F16)[3][0])
    res, ref = pair.step(ox.StepConfig(loss_scale=32768.0, max_grad_norm=1e9))
    assert (res.applied, res.timestep) == (1, 6)
    pair.assert_bit_equal()
    pair.close()


def test_spike_veto_skips_and_reports_the_measured_norm():
    # src/trainer.rs:629-632
    pair = Pair([1000], None, ox.BF16, ox.BF16, seed=8, grad_std=1.0)
    before = pair.gpu_state()
    res, ref = pair.step(ox.StepConfig(spike_skip=True))
    assert (res.overflow, res.applied) == (0, 0) == (ref.overflow, ref.applied)
    assert abs(res.reported_norm - ref.reported_norm) <= NORM_RTOL * ref.reported_norm and res.reported_norm > 1.0
    after = pair.gpu_state()
    for key in before:
        assert np.array_equal(bits(before[key][0]), bits(after[key][0]))
    pair.close()


def test_absent_gradients_leave_their_tensors_untouched():
    # src/dp/reduce.rs:20: an unrouted expert has no gradient; it must not decay nor move
    pair = Pair([700, 900, 50], [False, False, True], ox.BF16, ox.BF16, seed=9)
    before = pair.gpu_state()
    present = [True, False, True]
    res, ref = pair.step(ox.StepConfig(max_grad_norm=1e9), present)
    assert abs(res.grad_norm - ref.grad_norm) <= NORM_RTOL * ref.grad_norm
    pair.assert_bit_equal()
    after = pair.gpu_state()
    assert np.array_equal(bits(before["master"][1]), bits(after["master"][1]))
    assert not np.array_equal(bits(before["master"][0]), bits(after["master"][0]))
    # all present again next step
    res, ref = pair.step(ox.StepConfig(max_grad_norm=1e9))
    pair.assert_bit_equal()
    pair.close()


def test_zero_gradient_step_moves_only_the_decay_group():
    # tests/weight_decay.rs:102-147
    pair = Pair([640, 80], [False, True], ox.F32, ox.F32, seed=10)
    zero = [np.zeros(640, np.float32), np.zeros(80, np.float32)]
    for i in range(2):
        pair.opt.import_tensor(ffi.STATE_EXP_AVG, i, zero[i])
        pair.opt.import_tensor(ffi.STATE_EXP_AVG_SQ, i, zero[i])
    pair.set_grads(zero)
    before = pair.gpu_state()
    res = pair.opt.step(ox.StepConfig(lr=3e-3))
    assert res.applied == 1
    after = pair.gpu_state()
    assert np.array_equal(bits(before["master"][1]), bits(after["master"][1]))
    assert np.all(np.abs(after["master"][0]) < np.abs(before["master"][0]))
    pair.close()


def test_skip_all_equals_weight_decay_zero():
    # tests/weight_decay.rs:165-187
    a = Pair([1000, 10], [True, True], ox.BF16, ox.BF16, seed=11)
    b = Pair([1000, 10], [False, False], ox.BF16, ox.BF16, seed=11)
    a.opt.step(ox.StepConfig(weight_decay=0.1))
    b.opt.step(ox.StepConfig(weight_decay=0.0))
    sa, sb = a.gpu_state(), b.gpu_state()
    for key in sa:
        for x, y in zip(sa[key], sb[key]):
            assert np.array_equal(bits(x), bits(y))
    a.close(); b.close()


def test_hundred_steps_stay_within_drift_bound():
    numel = [3000, 64, 5000, 7]
    pair = Pair(numel, [False, True, False, True], ox.BF16, ox.BF16, seed=12, grad_std=5e-2)
    cfg = ox.StepConfig(lr=1e-3, max_grad_norm=1.0)
    for s in range(100):
        g = np.random.default_rng(500 + s)
        pair.set_grads([orc.narrow((g.standard_normal(n) * 5e-2).astype(np.float32), ox.BF16) for n in numel])
        res, ref = pair.step(cfg)
        assert res.applied == ref.applied == 1
        assert abs(res.grad_norm - ref.grad_norm) <= NORM_RTOL * ref.grad_norm
    pair.assert_close(1e-4)
    pair.close()


def test_loss_scaler_drives_the_skip_and_backoff_path():
    # f16 gradients pre-multiplied by the scale, an inf injected on one step: the step is skipped, the scale halves,
    # the clean-step counter restarts (tests/loss_scale.rs:118-214)
    numel = [4096, 128]
    pair = Pair(numel, [False, True], ox.F16, ox.F16, seed=13)
    opt = pair.opt
    trainer = ox.LitTrainerStep(ox.TrainerConfig(loss_scale=ox.LossScaleConfig(initial=65536.0, growth_interval=2),
                                                 max_grad_norm=1e9), opt)
    states = []
    for s in range(5):
        rng = np.random.default_rng(900 + s)
        scale = trainer.loss_scaler.scale()
        g = [orc.narrow((rng.standard_normal(n) * 1e-3 * scale).astype(np.float32), ox.F16) for n in numel]
        if s == 1:
            g[0][77] = np.array([np.inf], np.float16).view(np.uint16)[0]
        pair.set_grads(g)
        loss, norm = trainer.training_step(1.0)
        st = trainer.loss_scale_state()
        states.append((st.scale, st.consecutive_ok, trainer.optimizer_timestep(), math.isfinite(norm)))
    assert states == [(65536.0, 1, 1, True), (32768.0, 0, 1, False), (32768.0, 1, 2, True), (65536.0, 0, 3, True),
                      (65536.0, 1, 4, True)]
    pair.close()


def test_flatten_packs_per_tensor_gradients():
    import torch
    numel = [5, 256, 1000, 0, 77]
    opt = ox.DpOptimizer(numel, None, ox.BF16, ox.BF16)
    rng = np.random.default_rng(14)
    host = [orc.to_bf16(rng.standard_normal(n).astype(np.float32)) for n in numel]
    # 16-byte aligned sources of their own
    dev = [torch.from_numpy(h.view(np.int16)).cuda() if h.size else None for h in host]
    ptrs = [d.data_ptr() if d is not None else None for d in dev]
    ptrs[2] = None  # this rank has no gradient for tensor 2: zero-filled
    opt.flatten_grads(ptrs)
    for i, n in enumerate(numel):
        got = opt.export_tensor(ffi.STATE_GRADS, i)
        want = host[i] if i != 2 else np.zeros(n, np.uint16)
        assert np.array_equal(got, want), i
    # accumulate: the micro-batch sum of src/trainer.rs:1087-1107
    ptrs[2] = dev[2].data_ptr()
    opt.flatten_grads(ptrs, accumulate=True)
    for i, n in enumerate(numel):
        got = orc.widen(opt.export_tensor(ffi.STATE_GRADS, i), ox.BF16)
        base = orc.widen(host[i], ox.BF16)
        want = base + base if i != 2 else base
        assert np.array_equal(orc.to_bf16(want), orc.to_bf16(got)), i
    opt.destroy()


def test_param_groups_with_their_own_lr_scale_and_decay():
    # boostr ParamGroup{ids, lr_scale, weight_decay} (src/weight_decay/plan.rs:113-122): five distinct groups at once
    numel = [1000, 300, 777, 64, 2048]
    lr_scale = [1.0, 0.5, 0.5, 1.0, 0.25]
    no_decay = [False, False, True, True, False]
    master, m, v, grads = seeded_state(numel, 16, 1e-3, 1, ox.BF16)
    opt = ox.DpOptimizer(numel, no_decay, ox.BF16, ox.BF16, lr_scale=lr_scale)
    assert opt.info.n_groups == 5
    ref = orc.StepState([p.copy() for p in master], [x.copy() for x in m], [x.copy() for x in v],
                        [orc.to_bf16(p) for p in master], orc.BF16, lr_scale=lr_scale,
                        group_wd=[0.0 if nd else NAN for nd in no_decay])
    for i in range(len(numel)):
        opt.import_tensor(ffi.STATE_MASTER, i, master[i])
        opt.import_tensor(ffi.STATE_EXP_AVG, i, m[i])
        opt.import_tensor(ffi.STATE_EXP_AVG_SQ, i, v[i])
        opt.import_tensor(ffi.STATE_GRADS, i, grads[0][i])
    cfg = dict(lr=1e-3, max_grad_norm=1e9, eps=1e-8)
    for _ in range(2):
        opt.step(ox.StepConfig(**cfg))
        orc.step(ref, [grads[0]], orc.BF16, orc.StepConfig(**cfg))
    for kind, arrs in ((ffi.STATE_MASTER, ref.master), (ffi.STATE_EXP_AVG, ref.exp_avg), (ffi.STATE_EXP_AVG_SQ, ref.exp_avg_sq), (ffi.STATE_WORK, ref.work)):
        for i in range(len(numel)):
            assert np.array_equal(bits(opt.export_tensor(kind, i)), bits(arrs[i])), (kind, i)
    opt.destroy()


def test_f32_gradients_need_only_16_byte_alignment():
    # caller-owned f32 memory is promised 16-byte aligned, not 32: the norm and the flatten must accept it
    import torch
    rng = np.random.default_rng(15)
    host = rng.standard_normal(4 + 5000).astype(np.float32)
    dev = torch.from_numpy(host).cuda()
    ptr = dev.data_ptr() + 16  # 16-byte aligned, not 32
    assert ptr % 32 == 16
    want = math.sqrt(orc.sumsq(host[4:]))
    assert abs(ox.compute_grad_norm(ptr, ox.F32, 5000) - want) <= NORM_RTOL * want
    opt = ox.DpOptimizer([5000], None, ox.F32, ox.F32)
    opt.flatten_grads([ptr])
    assert np.array_equal(opt.export_tensor(ffi.STATE_GRADS, 0), host[4:])
    with pytest.raises(ox.OxzError, match="16-byte aligned"):
        opt.flatten_grads([ptr + 4])
    opt.destroy()


def test_call_order_errors_are_reported_not_fatal():
    opt = ox.DpOptimizer([100], None, ox.BF16, ox.BF16)
    with pytest.raises(ox.OxzError, match="no step is in flight"):
        opt.step_wait()
    opt.step_async(ox.StepConfig())
    with pytest.raises(ox.OxzError, match="still in flight"):
        opt.step_async(ox.StepConfig())
    opt.step_wait()
    with pytest.raises(ox.OxzError, match="max_grad_value"):
        opt.step(ox.StepConfig(max_grad_value=-1.0))
    opt.destroy()
