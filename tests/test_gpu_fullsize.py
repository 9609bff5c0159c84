"""The step at the full sizes of the named parameter sets, on one GPU.

The two small sets (hybrid-384, 41 M; nano_dense, 134 M, all f32 as in the CPU-runnable configuration) are compared
with the CPU checker element for element. The large ones (Llama-3.2-1B, Qwen3-1.7B, the MoE set) are held to
size-independent properties plus an exact comparison on sampled tensors:
  - the norm against an independent float64 evaluation (torch) and against the sum of per-tensor norms;
  - sampled tensors updated by the checker with the coefficient the GPU reports: bit for bit;
  - every working weight equals the narrowed master;
  - an inf anywhere skips the step and every checksum of the state is unchanged;
  - a zero-gradient step multiplies exactly the decay group by (1 - lr*wd) and leaves the rest bit-identical;
  - halving the loss scale doubles the norm exactly.
Seeded synthetic inputs stand in for real gradients: bf16/f16 ~N(0,1e-3) (times the loss scale for f16),
master ~N(0,0.02), m ~N(0,1e-4), v = |N(0,1e-6)|.
"""
import math

import numpy as np
import pytest

import oxidizr_b200 as ox
from oxidizr_b200 import ffi, inventory
from oracle import dpstep as orc
from tests.helpers import NAN, bits

pytestmark = pytest.mark.gpu

NORM_RTOL = 1e-5


def build(name, gd, pd, seed=5, scale=1.0):
    import torch
    from oxidizr_b200.interop import state_views
    tensors = inventory.PARAM_SETS[name]()
    plan = ox.DecayPlan(ox.WeightDecaySpec("skip_1d"), tensors)
    numel = [t.elements for t in tensors]
    opt = ox.DpOptimizer(numel, plan.no_decay, gd, pd)
    v = state_views(opt)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    chunk = 1 << 26
    n = opt.info.local_elems
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        v["master"][lo:hi].normal_(0.0, 0.02, generator=gen)
        v["exp_avg"][lo:hi].normal_(0.0, 1e-4, generator=gen)
        v["exp_avg_sq"][lo:hi].normal_(0.0, 1e-6, generator=gen).abs_()
    for off, k in zip(opt.offsets, numel):  # padding between tensors stays zero
        for lo in range(0, k, chunk):
            hi = min(k, lo + chunk)
            v["grads"][off + lo:off + hi] = (torch.empty(hi - lo, device="cuda").normal_(0.0, 1e-3, generator=gen) * scale).to(v["grads"].dtype)
    # zero the state in the padding too, as a freshly allocated optimizer has it
    pos = 0
    for off, k in zip(opt.offsets, numel):
        if off > pos:
            for key in ("master", "exp_avg", "exp_avg_sq"):
                v[key][pos:off] = 0
        pos = off + k
    for key in ("master", "exp_avg", "exp_avg_sq"):
        v[key][pos:] = 0
    if pd != ox.F32:
        for lo in range(0, n, chunk):
            hi = min(n, lo + chunk)
            v["work"][lo:hi] = v["master"][lo:hi].to(v["work"].dtype)
    opt.timestep = 3
    torch.cuda.synchronize()
    return tensors, plan, numel, opt, v


def grads_host(v, off, n, gd):
    import torch
    t = v["grads"][off:off + n]
    return t.cpu().numpy().copy() if gd == ox.F32 else t.view(torch.int16).cpu().numpy().view(np.uint16).copy()


def checksums(v):
    import torch
    out = {}
    for key in ("master", "exp_avg", "exp_avg_sq", "work"):
        t = v[key]
        raw = t.view(torch.int32) if t.element_size() == 4 else t.view(torch.int16)
        out[key] = int(raw.to(torch.int64).sum().item()) if raw.numel() < (1 << 28) else \
            sum(int(raw[i:i + (1 << 28)].to(torch.int64).sum().item()) for i in range(0, raw.numel(), 1 << 28))
    return out


def torch_norm(v, opt, numel, inv_scale):
    import torch
    total, per_tensor = 0.0, []
    for off, k in zip(opt.offsets, numel):
        s = 0.0
        for lo in range(0, k, 1 << 26):
            hi = min(k, lo + (1 << 26))
            x = v["grads"][off + lo:off + hi].float() * inv_scale
            s += float((x * x).double().sum().item())
        per_tensor.append(s)
        total += s
    return math.sqrt(total), per_tensor


@pytest.mark.parametrize("name,gd,pd,kw", [
    ("hybrid-384", ox.BF16, ox.BF16, dict(max_grad_norm=1.0, eps=1e-6)),
    ("nano_dense", ox.F32, ox.F32, dict(lr=3e-4, eps=1e-8, weight_decay=0.1, max_grad_norm=1.0)),
])
def test_small_sets_match_the_checker_element_for_element(name, gd, pd, kw):
    tensors, plan, numel, opt, v = build(name, gd, pd)
    T = len(numel)
    host = {k: [v[k][off:off + n].cpu().numpy().copy() for off, n in zip(opt.offsets, numel)] for k in ("master", "exp_avg", "exp_avg_sq")}
    grads = [grads_host(v, off, n, gd) for off, n in zip(opt.offsets, numel)]
    work = [orc.narrow(p, pd) for p in host["master"]] if pd != ox.F32 else None
    ref = orc.StepState(host["master"], host["exp_avg"], host["exp_avg_sq"], work, pd, lr_scale=[1.0] * T,
                        group_wd=[0.0 if nd else NAN for nd in plan.no_decay], timestep=3)
    for unclipped in (True, False):
        cfg = dict(kw, max_grad_norm=1e9) if unclipped else kw
        res = opt.step(ox.StepConfig(**cfg))
        want = orc.step(ref, [grads], gd, orc.StepConfig(**cfg))
        assert (res.overflow, res.applied, res.timestep) == (want.overflow, want.applied, want.timestep)
        assert abs(res.grad_norm - want.grad_norm) <= NORM_RTOL * want.grad_norm
        assert abs(res.clip_coef - want.clip_coef) <= 1e-6 * want.clip_coef
        for key, arrs in (("master", ref.master), ("exp_avg", ref.exp_avg), ("exp_avg_sq", ref.exp_avg_sq)):
            for i, (off, n) in enumerate(zip(opt.offsets, numel)):
                got = v[key][off:off + n].cpu().numpy()
                if unclipped:
                    assert np.array_equal(bits(got), bits(arrs[i])), (key, tensors[i].name)
                else:
                    b64 = arrs[i].astype(np.float64)
                    tol = 1e-6 * (np.abs(b64) + math.sqrt(float(np.mean(b64 ** 2))))
                    assert np.all(np.abs(got - b64) <= tol + 1e-30), (key, tensors[i].name)
    opt.destroy()


@pytest.mark.parametrize("name,gd,pd,scale", [
    ("llama-3.2-1b", ox.BF16, ox.BF16, NAN),
    ("qwen3-1.7b", ox.F16, ox.F16, 65536.0),
    ("moe-1b", ox.BF16, ox.BF16, NAN),
])
def test_large_sets_hold_the_size_independent_properties(name, gd, pd, scale):
    import torch
    scaled = scale == scale
    tensors, plan, numel, opt, v = build(name, gd, pd, scale=scale if scaled else 1.0)
    T = len(numel)
    cfg = ox.StepConfig(lr=3e-4, eps=1e-8, max_grad_norm=1.0, loss_scale=scale)
    present = None
    if name == "moe-1b":
        # 2 of 8 routed experts per layer got no token: all-zero gradients; half of those are reported absent
        rng = np.random.default_rng(9)
        present = [True] * T
        for layer in range(12):
            for j, e in enumerate(rng.choice(8, 2, replace=False)):
                for i, t in enumerate(tensors):
                    if f"layers.{layer}.moe.experts.{e}." in t.name:
                        v["grads"][opt.offsets[i]:opt.offsets[i] + numel[i]] = 0
                        if j == 0:
                            present[i] = False
    torch.cuda.synchronize()
    inv = 1.0 / scale if scaled else 1.0
    want_norm, per_tensor = torch_norm(v, opt, numel, inv)

    # sampled tensors for the exact comparison: the smallest, a mid-sized matrix, the largest-but-embedding, an expert
    order = sorted(range(T), key=lambda i: numel[i])
    sample = sorted({order[0], order[T // 2], order[-2], T - 1})
    if present is not None:
        sample = sorted(set(sample) | {next(i for i in range(T) if not present[i]), next(i for i in range(T) if present[i] and "experts" in tensors[i].name)})
    snap = {}
    for i in sample:
        off, n = opt.offsets[i], numel[i]
        snap[i] = {k: v[k][off:off + n].cpu().numpy().copy() for k in ("master", "exp_avg", "exp_avg_sq")}
        snap[i]["grads"] = grads_host(v, off, n, gd)

    res = opt.step(cfg, present)
    assert (res.overflow, res.applied, res.timestep) == (0, 1, 4)
    assert abs(res.grad_norm - want_norm) <= NORM_RTOL * want_norm
    assert abs(math.sqrt(sum(per_tensor)) - res.grad_norm) <= NORM_RTOL * res.grad_norm
    c = np.float32(res.clip_coef)
    if want_norm > 1.0:
        assert abs(res.clip_coef - 1.0 / (want_norm + 1e-6)) <= 1e-6 * res.clip_coef and res.reported_norm == 1.0

    for i in sample:
        off, n = opt.offsets[i], numel[i]
        got = {k: v[k][off:off + n].cpu().numpy() for k in ("master", "exp_avg", "exp_avg_sq")}
        if present is not None and not present[i]:
            for k in got:
                assert np.array_equal(bits(got[k]), bits(snap[i][k])), (tensors[i].name, k)  # an absent tensor is untouched
            continue
        g = orc.unscale(snap[i]["grads"], gd, scale) if scaled else orc.widen(snap[i]["grads"], gd)
        if c != 1.0:
            orc.lib().orc_scale(g.ctypes.data, g.size, c)
        s = orc.adam_prepare(cfg.lr, 1.0, cfg.beta1, cfg.beta2, cfg.eps, 0.0 if plan.no_decay[i] else cfg.weight_decay, 4)
        p, m, vv = snap[i]["master"], snap[i]["exp_avg"], snap[i]["exp_avg_sq"]
        w = np.zeros(n, np.uint16)
        orc.adamw(p, m, vv, g, s, w, pd)
        for k, ref in (("master", p), ("exp_avg", m), ("exp_avg_sq", vv)):
            assert np.array_equal(bits(got[k]), bits(ref)), (tensors[i].name, k)
        assert np.array_equal(v["work"][off:off + n].view(torch.int16).cpu().numpy().view(np.uint16), w), tensors[i].name

    # every working weight is the narrowed master
    n_local = opt.info.local_elems
    for lo in range(0, n_local, 1 << 27):
        hi = min(n_local, lo + (1 << 27))
        assert torch.equal(v["master"][lo:hi].to(v["work"].dtype).view(torch.int16), v["work"][lo:hi].view(torch.int16))

    # halving the loss scale doubles the norm exactly; an unscaled run takes scale 0.5 against 1.0
    a = ox.compute_grad_norm(opt.pointers()["grads"], gd, opt.info.padded_total, loss_scale=scale if scaled else 1.0)
    b = ox.compute_grad_norm(opt.pointers()["grads"], gd, opt.info.padded_total, loss_scale=(scale if scaled else 1.0) / 2)
    assert b == 2.0 * a

    # an inf anywhere skips the step: every checksum of the state is unchanged and the timestep stays
    before = checksums(v)
    pos = opt.offsets[T // 3] + numel[T // 3] // 2
    saved = v["grads"][pos].clone()
    v["grads"][pos] = float("inf")
    torch.cuda.synchronize()  # the views are written on torch's stream, the step runs on the plan's own
    res = opt.step(cfg, None)
    assert (res.overflow, res.applied, res.timestep) == (1, 0, 4) and math.isinf(res.grad_norm)
    assert checksums(v) == before
    v["grads"][pos] = saved

    # a zero-gradient step from zero moments: the decay group shrinks by exactly (1 - lr*wd), the rest keeps its bits
    v["grads"].zero_()
    v["exp_avg"].zero_()
    v["exp_avg_sq"].zero_()
    old = {i: v["master"][opt.offsets[i]:opt.offsets[i] + numel[i]].clone() for i in sample}
    torch.cuda.synchronize()
    res = opt.step(ox.StepConfig(lr=3e-3, weight_decay=0.1, eps=1e-8, loss_scale=scale), None)
    assert res.applied == 1 and res.grad_norm == 0.0
    decay = torch.tensor(np.float32(1.0 - 3e-3 * 0.1), device="cuda")
    for i in sample:
        new = v["master"][opt.offsets[i]:opt.offsets[i] + numel[i]]
        want = old[i] if plan.no_decay[i] else old[i] * decay
        assert torch.equal(new.view(torch.int32), want.view(torch.int32)), tensors[i].name
    opt.destroy()
