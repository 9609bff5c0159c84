"""The sharded multi-rank step against the CPU checker's replicated step.

Ranks run as threads of this process, one optimizer each (the reference's one-thread-per-rank model,
src/dp/launch.rs:207-240). With a local group every rank may share cuda:0, so the pull-reduce and push kernels are
exercised on a single GPU; with two or more GPUs the same tests also run over NCCL and real peer memory.
The checker sums the ranks' gradients in rank order in f32 (src/dp/reduce.rs:11-29); the P2P kernels do the same,
so without clipping the result is bit-identical.
"""
import math
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

import oxidizr_b200 as ox
from oxidizr_b200 import ffi
from oracle import dpstep as orc
from tests.helpers import NAN, bits, seeded_state

pytestmark = pytest.mark.gpu

NUMEL = [1, 300, 4096, 70001, 0, 513, 9000]
NO_DECAY = [True, True, False, False, False, True, False]


def gpu_count():
    import torch
    return torch.cuda.device_count()


class Group:
    def __init__(self, world, devices, kind, mode=ox.SYNC_P2P, gd=ox.BF16, pd=ox.BF16, seed=0, grad_std=1e-3,
                 bucket_bytes=16384, numel=NUMEL, no_decay=NO_DECAY):
        self.world, self.numel, self.gd, self.pd = world, numel, gd, pd
        self.pool = ThreadPoolExecutor(world)
        if kind == "local":
            self.comms = ox.Communicator.local_group(world, devices, timeout=60.0)
        else:
            self.comms = ox.Communicator.init_all(devices)
        master, m, v, grads = seeded_state(numel, seed, grad_std, world, gd)
        self.grads = grads
        work = [orc.narrow(p, pd) for p in master]
        self.ref = orc.StepState([p.copy() for p in master], [x.copy() for x in m], [x.copy() for x in v],
                                 [w.copy() for w in work], pd, lr_scale=[1.0] * len(numel),
                                 group_wd=[0.0 if nd else NAN for nd in no_decay])

        def make(r):
            opt = ox.DpOptimizer(numel, no_decay, gd, pd, world=world, rank=r, sync_mode=mode, device=devices[r],
                                 bucket_bytes=bucket_bytes, comm=self.comms[r])
            for i in range(len(numel)):
                opt.import_tensor(ffi.STATE_MASTER, i, master[i])
                opt.import_tensor(ffi.STATE_EXP_AVG, i, m[i])
                opt.import_tensor(ffi.STATE_EXP_AVG_SQ, i, v[i])
                opt.import_tensor(ffi.STATE_WORK, i, work[i])
                opt.import_tensor(ffi.STATE_GRADS, i, grads[r][i])
            return opt
        self.opts = list(self.pool.map(make, range(world)))

    def set_grads(self, grads):
        self.grads = grads
        def put(r):
            for i, g in enumerate(grads[r]):
                self.opts[r].import_tensor(ffi.STATE_GRADS, i, g)
        list(self.pool.map(put, range(self.world)))

    def step(self, cfg, extras=None, present=None):
        """present: one list of flags for every rank, or one list per rank (the ranks' flags may differ)."""
        per_rank = present is not None and len(present) > 0 and isinstance(present[0], (list, tuple))
        flags = [present[r] if per_rank else present for r in range(self.world)]

        def run(r):
            res = self.opts[r].step(cfg, flags[r], [extras[r]] if extras else None)
            return res, (self.opts[r].last_extras if extras else None)
        out = list(self.pool.map(run, range(self.world)))
        rg = [[g if (flags[r] is None or flags[r][i]) else None for i, g in enumerate(self.grads[r])] for r in range(self.world)]
        ocfg = orc.StepConfig(**{k: getattr(cfg, k) for k in orc.StepConfig.__dataclass_fields__})
        ref = orc.step(self.ref, rg, self.gd, ocfg)
        return out, ref

    def merged(self, kind):
        """Each rank exports the elements it owns; together they must cover every tensor."""
        out = []
        for i, n in enumerate(self.numel):
            acc = np.full(n, np.nan, np.float32)
            for opt in self.opts:
                opt.export_tensor(kind, i, acc)
            out.append(acc)
        return out

    def assert_state(self, exact=True, rel=1e-6):
        for kind, ref in ((ffi.STATE_MASTER, self.ref.master), (ffi.STATE_EXP_AVG, self.ref.exp_avg),
                          (ffi.STATE_EXP_AVG_SQ, self.ref.exp_avg_sq)):
            for i, (a, b) in enumerate(zip(self.merged(kind), ref)):
                assert not np.isnan(a).any(), f"tensor {i}: some element has no owner"
                if exact:
                    assert np.array_equal(bits(a), bits(b)), (kind, i, int(np.sum(bits(a) != bits(b))))
                else:
                    tol = rel * (np.abs(b.astype(np.float64)) + math.sqrt(float(np.mean(b.astype(np.float64) ** 2)) if b.size else 0.0))
                    assert np.all(np.abs(a.astype(np.float64) - b) <= tol + 1e-30), (kind, i)
        # every rank holds the full, identical working weights after the push / all-gather
        for r, opt in enumerate(self.opts):
            for i in range(len(self.numel)):
                w = opt.export_tensor(ffi.STATE_WORK, i)
                if exact:
                    assert np.array_equal(bits(w), bits(self.ref.work[i])), (r, i)
                else:
                    assert np.array_equal(bits(w), bits(self.opts[0].export_tensor(ffi.STATE_WORK, i))), (r, i)

    def close(self):
        list(self.pool.map(lambda r: self.opts[r].destroy(), range(self.world)))
        for c in self.comms:
            c.destroy()
        self.pool.shutdown()


def layouts():
    out = [("local", 2, [0, 0]), ("local", 3, [0, 0, 0]), ("local", 4, [0, 0, 0, 0])]
    n = gpu_count()
    if n >= 2:
        out += [("nccl", 2, [0, 1]), ("local", 2, [0, 1])]
    if n >= 4:
        out += [("nccl", 4, [0, 1, 2, 3])]
    if n >= 8:
        out += [("nccl", 8, list(range(8)))]
    return out


@pytest.mark.parametrize("mode", [ox.SYNC_P2P, ox.SYNC_COPY])
@pytest.mark.parametrize("kind,world,devices", layouts())
@pytest.mark.parametrize("gd,pd", [(ox.BF16, ox.BF16), (ox.F16, ox.F16), (ox.F32, ox.F32)])
def test_sharded_p2p_step_is_bit_identical_to_the_replicated_step(kind, world, devices, gd, pd, mode):
    g = Group(world, devices, kind, mode=mode, gd=gd, pd=pd, seed=21)
    cfg = ox.StepConfig(max_grad_norm=1e9, eps=1e-8)
    for s in range(2):
        out, ref = g.step(cfg, extras=[0.25 * (r + 1) for r in range(world)])
        for res, extras in out:
            assert (res.overflow, res.applied, res.timestep) == (ref.overflow, ref.applied, ref.timestep)
            assert abs(res.grad_norm - ref.grad_norm) <= 1e-5 * ref.grad_norm
            assert extras == [sum(0.25 * (r + 1) for r in range(world))]  # the loss summed over ranks
        norms = {res.grad_norm for res, _ in out}
        assert len(norms) == 1, "every rank must see the same norm bits"
        g.assert_state(exact=True)
    g.close()


@pytest.mark.parametrize("bulk", [True, False])
@pytest.mark.parametrize("world,bucket_bytes", [(2, 16384), (4, 16384), (8, 32768), (2, 8192 + 4096)])
@pytest.mark.parametrize("gd", [ox.BF16, ox.F16])
def test_bulk_copy_pull_gives_the_same_bits_as_the_per_lane_pull(world, bucket_bytes, gd, bulk, monkeypatch):
    """The pull has two kernels: bulk asynchronous copies into shared memory where a bucket's shard is a multiple of
    8 tiles, per-lane loads otherwise. Both must reproduce the replicated step bit for bit, ragged last shard included."""
    monkeypatch.setenv("OXZ_PULL_BULK", "1" if bulk else "0")
    g = Group(world, [0] * world, "local", gd=gd, pd=gd, seed=31, bucket_bytes=bucket_bytes)
    shard_tiles = bucket_bytes // 2 // 256 // world
    expect = 2 if (bulk and shard_tiles % 8 == 0) else 1
    for _ in range(2):
        out, ref = g.step(ox.StepConfig(max_grad_norm=1e9, loss_scale=8.0 if gd == ox.F16 else float("nan")))
        assert {opt.last_pull_kernel() for opt in g.opts} == {expect}
        for res, _ in out:
            assert (res.overflow, res.applied, res.timestep) == (ref.overflow, ref.applied, ref.timestep)
            assert abs(res.grad_norm - ref.grad_norm) <= 1e-5 * ref.grad_norm
        g.assert_state(exact=True)
    # an absent tensor: its tiles (and padding) stay out of the sum and the norm in either kernel
    present = [True, True, False, True, True, True, True]
    g.step(ox.StepConfig(max_grad_norm=1e9, loss_scale=8.0 if gd == ox.F16 else float("nan")), present=present)
    assert {opt.last_pull_kernel() for opt in g.opts} == {expect}
    g.assert_state(exact=True)
    g.close()


@pytest.mark.parametrize("kind,world,devices", layouts())
@pytest.mark.parametrize("gd,pd", [(ox.BF16, ox.BF16), (ox.F32, ox.F32)])
def test_full_replicas_step_like_the_reference_and_agree_with_the_sharded_step(kind, world, devices, gd, pd):
    """OXZ_SYNC_REPLICATED is the reference's own arrangement (every rank sums all gradients and updates a full copy,
    src/dp/reduce.rs:30-60): each rank alone must hold the oracle's state, bit for bit, and so must the sharded run."""
    rep = Group(world, devices, kind, mode=ox.SYNC_REPLICATED, gd=gd, pd=pd, seed=41)
    shd = Group(world, devices, kind, mode=ox.SYNC_P2P, gd=gd, pd=pd, seed=41)
    cfg = ox.StepConfig(max_grad_norm=1e9)
    for s in range(2):
        out, ref = rep.step(cfg, extras=[1.0 + r for r in range(world)])
        out2, _ = shd.step(cfg, extras=[1.0 + r for r in range(world)])
        for (res, extras), (res2, extras2) in zip(out, out2):
            assert (res.overflow, res.applied, res.timestep) == (ref.overflow, ref.applied, ref.timestep)
            assert abs(res.grad_norm - ref.grad_norm) <= 1e-5 * ref.grad_norm
            assert extras == extras2 == [sum(1.0 + r for r in range(world))]
        assert len({res.grad_norm for res, _ in out}) == 1
    for opt in rep.opts:  # every rank by itself, not a merge over ranks
        assert opt.info.local_elems == opt.info.padded_total
        for kind_, refs in ((ffi.STATE_MASTER, rep.ref.master), (ffi.STATE_EXP_AVG, rep.ref.exp_avg),
                            (ffi.STATE_EXP_AVG_SQ, rep.ref.exp_avg_sq)):
            for i, b in enumerate(refs):
                assert np.array_equal(bits(opt.export_tensor(kind_, i)), bits(b)), (kind_, i)
        for i in range(len(rep.numel)):
            assert np.array_equal(bits(opt.export_tensor(ffi.STATE_WORK, i)), bits(rep.ref.work[i]))
    shd.assert_state(exact=True)
    # an overflow on one rank is seen by every replica
    grads = [[x.copy() for x in rg] for rg in rep.grads]
    grads[world - 1][1][7] = np.inf if gd == ox.F32 else 0x7F80  # +inf in f32, and its bf16 pattern
    rep.set_grads(grads)
    out, ref = rep.step(cfg)
    for res, _ in out:
        assert (res.overflow, res.applied) == (1, 0) == (ref.overflow, ref.applied)
    rep.close()
    shd.close()


@pytest.mark.parametrize("world,mode", [(1, ox.SYNC_SINGLE), (2, ox.SYNC_P2P), (4, ox.SYNC_P2P), (2, ox.SYNC_REPLICATED)])
def test_gradients_uploaded_into_the_second_buffer_while_a_step_runs_give_the_same_steps(world, mode):
    """Host-fed steps over the two gradient buffers: the copy of step i+1 is issued while step i is in flight, every
    rank swaps between the same two steps, and the state after four such steps with four different gradients is, bit
    for bit, that of four plain steps (import, then step) and of the checker."""
    steps = 4
    if world == 1:
        comms = [None]
    else:
        comms = ox.Communicator.local_group(world, [0] * world, timeout=60.0)
    pool = ThreadPoolExecutor(world)
    master, m, v, _ = seeded_state(NUMEL, 61, 1e-3, world, ox.BF16)
    per_step = [seeded_state(NUMEL, 70 + k, 1e-3, world, ox.BF16)[3] for k in range(steps)]
    work = [orc.narrow(p, ox.BF16) for p in master]
    ref = orc.StepState([p.copy() for p in master], [x.copy() for x in m], [x.copy() for x in v], [w.copy() for w in work],
                        ox.BF16, lr_scale=[1.0] * len(NUMEL), group_wd=[0.0 if nd else NAN for nd in NO_DECAY])

    def make(r):
        opt = ox.DpOptimizer(NUMEL, NO_DECAY, ox.BF16, ox.BF16, world=world, rank=r, sync_mode=mode, device=0,
                             bucket_bytes=16384, comm=comms[r])
        for i in range(len(NUMEL)):
            opt.import_tensor(ffi.STATE_MASTER, i, master[i])
            opt.import_tensor(ffi.STATE_EXP_AVG, i, m[i])
            opt.import_tensor(ffi.STATE_EXP_AVG_SQ, i, v[i])
            opt.import_tensor(ffi.STATE_WORK, i, work[i])
        return opt
    cfg = ox.StepConfig(max_grad_norm=1e9)

    def pipelined(r):
        opt = opts[r]
        opt.double_buffer_grads()
        keep = [[np.ascontiguousarray(g) for g in per_step[k][r]] for k in range(steps)]  # stay alive during the copies
        def upload(k):
            for i, g in enumerate(keep[k]):
                if g.size:
                    opt.upload_next_grads(i, g.ctypes.data)
        out = []
        upload(0)
        for k in range(steps):
            opt.swap_grads()
            opt.step_async(cfg)
            if k + 1 < steps:
                upload(k + 1)
            out.append(opt.step_wait())
        return out
    opts = list(pool.map(make, range(world)))
    results = list(pool.map(pipelined, range(world)))
    for k in range(steps):
        want = orc.step(ref, [per_step[k][r] for r in range(world)], ox.BF16, orc.StepConfig(max_grad_norm=1e9))
        for r in range(world):
            res = results[r][k]
            assert (res.overflow, res.applied, res.timestep) == (want.overflow, want.applied, want.timestep)
            assert abs(res.grad_norm - want.grad_norm) <= 1e-5 * want.grad_norm
    for kind, refs in ((ffi.STATE_MASTER, ref.master), (ffi.STATE_EXP_AVG, ref.exp_avg), (ffi.STATE_EXP_AVG_SQ, ref.exp_avg_sq)):
        for i, b in enumerate(refs):
            acc = np.full(NUMEL[i], np.nan, np.float32)
            for opt in opts:
                opt.export_tensor(kind, i, acc)
            assert np.array_equal(bits(acc), bits(b)), (kind, i)
    for opt in opts:
        for i in range(len(NUMEL)):
            assert np.array_equal(bits(opt.export_tensor(ffi.STATE_WORK, i)), bits(ref.work[i]))
    # the current buffer is what the state calls see: the last step's gradients
    for r, opt in enumerate(opts):
        assert np.array_equal(bits(opt.export_tensor(ffi.STATE_GRADS, 3)), bits(per_step[steps - 1][r][3]))
    list(pool.map(lambda r: opts[r].destroy(), range(world)))
    for c in comms:
        if c is not None:
            c.destroy()
    pool.shutdown()


def test_a_pull_wait_that_runs_out_is_reported_and_changes_nothing(monkeypatch):
    """The bulk-copy pull bounds every wait on its own copies. Here the bound of the main-loop waits is lowered to zero,
    so the first wait gives up at once while the copies are in fact on their way: the kernel records the run-out,
    collects its copies in flight and ends normally; every rank's step comes back as OXZ_ERR_TIMEOUT with optimizer
    state and weights untouched (the norm is poisoned, so the update is skipped everywhere); the context stays usable
    and the next step, with the bound restored, is the checker's step. No fault, trap or hang is involved."""
    world = 2
    g = Group(world, [0] * world, "local", seed=51)
    before = [g.merged(k) for k in (ffi.STATE_MASTER, ffi.STATE_EXP_AVG, ffi.STATE_EXP_AVG_SQ)]
    work_before = [g.opts[1].export_tensor(ffi.STATE_WORK, i) for i in range(len(g.numel))]
    monkeypatch.setenv("OXZ_PULL_WAIT_LIMIT", "0")

    def failing(r):
        try:
            g.opts[r].step(ox.StepConfig(max_grad_norm=1e9))
            return None
        except ox.OxzError as e:
            return e
    errors = list(g.pool.map(failing, range(world)))
    assert all(e is not None and e.status == ffi.ERR_TIMEOUT and "bounded wait" in str(e) for e in errors), errors
    assert {opt.last_pull_kernel() for opt in g.opts} == {2}
    assert all(opt.timestep == 0 for opt in g.opts)
    after = [g.merged(k) for k in (ffi.STATE_MASTER, ffi.STATE_EXP_AVG, ffi.STATE_EXP_AVG_SQ)]
    for b, a in zip(before, after):
        for x, y in zip(b, a):
            assert np.array_equal(bits(x), bits(y))
    for i, w in enumerate(work_before):
        assert np.array_equal(bits(w), bits(g.opts[1].export_tensor(ffi.STATE_WORK, i)))
    monkeypatch.delenv("OXZ_PULL_WAIT_LIMIT")
    out, ref = g.step(ox.StepConfig(max_grad_norm=1e9))
    for res, _ in out:
        assert (res.overflow, res.applied, res.timestep) == (0, 1, 1) == (ref.overflow, ref.applied, ref.timestep)
    g.assert_state(exact=True)
    g.close()


def test_a_run_out_on_one_rank_alone_is_reported_by_every_rank(monkeypatch):
    """Only rank 1's pull gives up (its bound alone is lowered). Its flag rides on the step's exchange, so rank 0 does
    not take the poisoned norm for an overflow: both ranks return OXZ_ERR_TIMEOUT, nothing changes anywhere, and no
    rank would back its loss scale off and walk into the next collective alone."""
    world = 2
    g = Group(world, [0] * world, "local", seed=52)
    before = [g.merged(k) for k in (ffi.STATE_MASTER, ffi.STATE_EXP_AVG, ffi.STATE_EXP_AVG_SQ)]
    monkeypatch.setenv("OXZ_PULL_WAIT_LIMIT", "0@1")

    def failing(r):
        try:
            return g.opts[r].step(ox.StepConfig(max_grad_norm=1e9))
        except ox.OxzError as e:
            return e
    got = list(g.pool.map(failing, range(world)))
    assert all(isinstance(e, ox.OxzError) and e.status == ffi.ERR_TIMEOUT for e in got), got
    assert all(opt.timestep == 0 for opt in g.opts)
    after = [g.merged(k) for k in (ffi.STATE_MASTER, ffi.STATE_EXP_AVG, ffi.STATE_EXP_AVG_SQ)]
    for b, a in zip(before, after):
        for x, y in zip(b, a):
            assert np.array_equal(bits(x), bits(y))
    monkeypatch.delenv("OXZ_PULL_WAIT_LIMIT")
    out, ref = g.step(ox.StepConfig(max_grad_norm=1e9))
    for res, _ in out:
        assert (res.overflow, res.applied, res.timestep) == (0, 1, 1)
    g.assert_state(exact=True)
    g.close()


def test_a_wait_for_a_rank_that_never_arrives_runs_out_and_leaves_the_context_usable():
    # the gate kernel of the peer-memory exchanges, as rank 0 of two ranks whose other rank does not exist: its wait is
    # bounded, the kernel records the run-out and returns; nothing faults, traps or hangs
    assert ox.selftest_bounded_wait(0, limit_ms=30) == 1


@pytest.mark.parametrize("mode", [ox.SYNC_P2P, ox.SYNC_COPY, ox.SYNC_REPLICATED])
@pytest.mark.parametrize("kind,world,devices", layouts())
def test_ranks_with_different_gradient_flags_update_the_union(kind, world, devices, mode):
    """src/dp/reduce.rs:20: a tensor is left alone only when NO rank has a gradient for it. Tensor 2 has one on rank 0
    only, tensor 5 on the last rank only, tensor 3 on no rank, the others on every rank. The ranks hand in different
    flags; the library forms their union, the ranks without a gradient contribute the zeros their buffers hold."""
    g = Group(world, devices, kind, mode=mode, seed=24)
    T = len(g.numel)
    flags = [[True] * T for _ in range(world)]
    grads = [[x.copy() for x in rg] for rg in g.grads]
    for r in range(world):
        flags[r][3] = False
        if r != 0:
            flags[r][2] = False
            grads[r][2] = np.zeros_like(grads[r][2])
        if r != world - 1:
            flags[r][5] = False
            grads[r][5] = np.zeros_like(grads[r][5])
    g.set_grads(grads)
    before3 = g.merged(ffi.STATE_MASTER)[3].copy()
    out, ref = g.step(ox.StepConfig(max_grad_norm=1e9), present=flags)
    for res, _ in out:
        assert (res.overflow, res.applied) == (0, 1) and abs(res.grad_norm - ref.grad_norm) <= 1e-5 * ref.grad_norm
    if mode == ox.SYNC_REPLICATED:
        for opt in g.opts:  # every replica holds everything
            for kind_, refs in ((ffi.STATE_MASTER, g.ref.master), (ffi.STATE_EXP_AVG, g.ref.exp_avg), (ffi.STATE_EXP_AVG_SQ, g.ref.exp_avg_sq)):
                for i in range(T):
                    assert np.array_equal(bits(opt.export_tensor(kind_, i)), bits(refs[i])), (kind_, i)
    else:
        g.assert_state(exact=True)
        assert np.array_equal(bits(g.merged(ffi.STATE_MASTER)[3]), bits(before3))
    # the per-tensor norms name the tensor no rank had a gradient for
    per = list(g.pool.map(lambda r: g.opts[r].grad_norms_per_tensor(), range(world)))
    for norms in per:
        assert norms[3] == -1.0 and norms[4] == 0.0  # tensor 4 is empty
        for i in (0, 1, 2, 5, 6):
            rank_sum = orc.sum_ranks([orc.widen(grads[r][i], g.gd) for r in range(world)], orc.F32)
            want = math.sqrt(orc.sumsq(rank_sum))
            assert abs(norms[i] - want) <= 1e-5 * want, (i, norms[i], want)
    g.close()


@pytest.mark.parametrize("kind,world,devices", layouts())
@pytest.mark.parametrize("gd,pd", [(ox.BF16, ox.BF16), (ox.F32, ox.F16)])
def test_the_wide_push_lands_the_same_weights_on_every_rank(monkeypatch, kind, world, devices, gd, pd):
    # OXZ_ADAM_VARIANT=3: the 16-bit working weights leave as one 256-bit store per lane and rank for two tiles
    monkeypatch.setenv("OXZ_ADAM_VARIANT", "3")
    g = Group(world, devices, kind, gd=gd, pd=pd, seed=26)
    out, ref = g.step(ox.StepConfig(max_grad_norm=1e9, eps=1e-8))
    for res, _ in out:
        assert (res.overflow, res.applied, res.timestep) == (0, 1, 1)
    g.assert_state(exact=True)
    present = [True, True, False, True, True, True, False]
    out, ref = g.step(ox.StepConfig(max_grad_norm=1e9, eps=1e-8), present=present)
    g.assert_state(exact=True)
    g.close()


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs: real peer memory")
def test_pull_and_push_over_real_peer_memory_beyond_l2():
    """Two rank threads of one process, one GPU each, meeting on the host: the bulk-copy pull reads the other GPU's
    gradients over NVLink and the update stores the weights into the other GPU's buffer, on tensors larger than the
    L2 cache (100 M parameters: 200 MB of gradients per rank), bit for bit against the checker. One process and no
    kernel that waits on another: this is the case a profiler capture of the two peer kernels runs on."""
    numel = [60_000_000, 2048, 40_000_000 + 77]
    g = Group(2, [0, 1], "local", seed=27, bucket_bytes=0, numel=numel, no_decay=[False, True, False])
    out, ref = g.step(ox.StepConfig(max_grad_norm=1e9, eps=1e-8))
    for res, _ in out:
        assert (res.overflow, res.applied, res.timestep) == (0, 1, 1)
        assert abs(res.grad_norm - ref.grad_norm) <= 1e-5 * ref.grad_norm
    assert {opt.last_pull_kernel() for opt in g.opts} == {2} and {opt.last_update_kernel() for opt in g.opts} == {2}
    g.assert_state(exact=True)
    g.close()


ABORT_CHILD = r"""
import threading, time
import oxidizr_b200 as ox
from oxidizr_b200 import ffi
comms = ox.Communicator.init_all([0, 1])
opts = [None, None]
def make(r):
    opts[r] = ox.DpOptimizer([70001, 300], None, ox.BF16, ox.BF16, world=2, rank=r, device=r, comm=comms[r], bucket_bytes=16384)
threads = [threading.Thread(target=make, args=(r,)) for r in range(2)]
[t.start() for t in threads]
[t.join() for t in threads]
assert opts[0].exchange_kind() == ffi.EXCHANGE_MAILBOX
opts[0].step_async(ox.StepConfig())   # rank 1 never joins: rank 0's gate kernel waits for its arrival
time.sleep(0.3)
t0 = time.time()
for c in comms:
    c.abort()
try:
    opts[0].step_wait()
    print("NO ERROR")
except ox.OxzError as e:
    print("STATUS", e.status, "AFTER", round(time.time() - t0, 2), "TIMESTEP", opts[0].timestep)
"""


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs: the peer-memory exchanges run one GPU per rank")
def test_an_abort_ends_the_wait_for_a_rank_that_never_joins():
    """src/dp/launch.rs:97-103, 142-150: the first failure aborts the group so that peers blocked in a collective
    return. Here the collective is the step's opening gate, a kernel polling its mailbox: rank 1 never makes the step
    (a failure made on the host), rank 0 waits, and oxz_comm_abort from another thread ends the wait at once - well
    inside the 20 s the wait itself would allow - with OXZ_ERR_ABORTED and nothing applied. A child process with NVLS
    off, as every test that leaves a rank behind should run; no kernel faults, traps or spins without a bound."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OXZ_MAIL_TIMEOUT_MS="20000", PYTHONPATH=root)
    out = subprocess.run([sys.executable, "-c", ABORT_CHILD], capture_output=True, text=True, timeout=180, env=env, cwd=root)
    line = [l for l in out.stdout.splitlines() if l.startswith(("STATUS", "NO ERROR"))]
    assert line, out.stdout + out.stderr
    words = line[-1].split()
    assert words[0] == "STATUS" and int(words[1]) == ffi.ERR_ABORTED, line
    assert float(words[3]) < 5.0 and int(words[5]) == 0, line


@pytest.mark.parametrize("kind,world,devices", layouts())
def test_exchange_kind_follows_the_communicator(kind, world, devices):
    g = Group(world, devices, kind, seed=25)
    # mailboxes by default up to four ranks on distinct GPUs; the communicator's collectives otherwise
    want = ffi.EXCHANGE_MAILBOX if (kind == "nccl" and world <= 4) else ffi.EXCHANGE_COMM
    assert {opt.exchange_kind() for opt in g.opts} == {want}
    g.close()


@pytest.mark.parametrize("mode", [ox.SYNC_P2P, ox.SYNC_COPY])
@pytest.mark.parametrize("kind,world,devices", layouts())
def test_sharded_step_with_clipping_and_absent_tensors(kind, world, devices, mode):
    g = Group(world, devices, kind, mode=mode, seed=22, grad_std=1.0)
    present = [True, True, False, True, True, True, True]
    out, ref = g.step(ox.StepConfig(max_grad_norm=1.0), present=present)
    for res, _ in out:
        assert abs(res.grad_norm - ref.grad_norm) <= 1e-5 * ref.grad_norm
        assert abs(res.clip_coef - ref.clip_coef) <= 1e-6 * ref.clip_coef and res.reported_norm == 1.0
    g.assert_state(exact=False)
    g.close()


@pytest.mark.parametrize("mode", [ox.SYNC_P2P, ox.SYNC_COPY])
@pytest.mark.parametrize("kind,world,devices", layouts())
def test_overflow_on_one_rank_skips_on_every_rank(kind, world, devices, mode):
    # tests/data_parallel.rs:353-392
    g = Group(world, devices, kind, mode=mode, gd=ox.F16, pd=ox.F16, seed=23)
    before = [g.merged(k) for k in (ffi.STATE_MASTER, ffi.STATE_EXP_AVG, ffi.STATE_EXP_AVG_SQ)]
    grads = [[x.copy() for x in rg] for rg in g.grads]
    grads[world - 1][3][4242] = np.array([np.inf], np.float16).view(np.uint16)[0]
    g.set_grads(grads)
    out, ref = g.step(ox.StepConfig(loss_scale=1024.0))
    for res, _ in out:
        assert (res.overflow, res.applied, res.timestep) == (1, 0, 0) == (ref.overflow, ref.applied, ref.timestep)
        assert not math.isfinite(res.grad_norm)
    after = [g.merged(k) for k in (ffi.STATE_MASTER, ffi.STATE_EXP_AVG, ffi.STATE_EXP_AVG_SQ)]
    for b, a in zip(before, after):
        for x, y in zip(b, a):
            assert np.array_equal(bits(x), bits(y))
    g.close()


@pytest.mark.skipif(gpu_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("gd", [ox.F32, ox.BF16])
def test_nccl_mode_matches_within_its_wire_precision(gd):
    # reduce-scatter in the gradient's dtype: f32 sums differ from the rank-order sum only by rounding order;
    # bf16 sums are rounded to bf16 by the collective, so only the looser bound holds
    g = Group(2, [0, 1], "nccl", mode=ox.SYNC_NCCL, gd=gd, pd=ox.BF16, seed=24)
    out, ref = g.step(ox.StepConfig(max_grad_norm=1e9))
    rel = 1e-6 if gd == ox.F32 else 2e-2
    for res, _ in out:
        assert res.applied == 1 and abs(res.grad_norm - ref.grad_norm) <= max(rel, 1e-5) * ref.grad_norm
    g.assert_state(exact=False, rel=rel)
    g.close()


def test_f16_loss_scale_run_with_seeded_overflows_over_eight_ranks():
    """fp16 gradients pre-multiplied by a dynamic loss scale of 65536, eight ranks, and a seeded 1-in-50 step that
    writes an inf into a random rank's bucket: the skip/backoff decisions must equal the checker's on every step and
    the state must stay within the 100-step bound (the growth interval is shortened so growth is exercised too)."""
    world, steps = 8, 100
    numel = [3000, 64, 5000, 7, 1200]
    no_decay = [False, True, False, True, False]
    g = Group(world, [0] * world, "local", gd=ox.F16, pd=ox.F16, seed=50, numel=numel, no_decay=no_decay, bucket_bytes=4096)
    cfg_scaler = dict(initial=65536.0, growth_interval=20)
    gpu_scaler = ox.LossScaler(ox.LossScaleConfig(**cfg_scaler))
    from oracle import host_logic as hl
    ref_scaler = hl.LossScaler(hl.LossScaleConfig(**cfg_scaler))
    pick = np.random.default_rng(51)
    skipped = 0
    for s in range(steps):
        scale = gpu_scaler.scale()
        assert scale == ref_scaler.scale()
        grads = []
        for r in range(world):
            rng = np.random.default_rng(10_000 + 97 * s + r)
            grads.append([orc.narrow((rng.standard_normal(n) * 1e-3 * scale).astype(np.float32), ox.F16) for n in numel])
        inject = pick.integers(0, 50) == 0 or s == 7
        if inject:
            r, t = int(pick.integers(0, world)), int(pick.choice([0, 2, 4]))
            grads[r][t][int(pick.integers(0, numel[t]))] = np.array([np.inf], np.float16).view(np.uint16)[0]
        g.set_grads(grads)
        out, ref = g.step(ox.StepConfig(lr=1e-3, max_grad_norm=1.0, loss_scale=scale))
        for res, _ in out:
            assert (res.overflow, res.applied, res.timestep) == (ref.overflow, ref.applied, ref.timestep), s
            if not ref.overflow:
                assert abs(res.grad_norm - ref.grad_norm) <= 1e-5 * ref.grad_norm
        assert bool(ref.overflow) == bool(inject)
        skipped += ref.overflow
        gpu_scaler.record_step(bool(out[0][0].overflow))
        hl.record_after_step(ref_scaler, bool(ref.overflow), False)
        assert (gpu_scaler.state().scale, gpu_scaler.state().consecutive_ok) == (ref_scaler.state().scale, ref_scaler.state().consecutive_ok)
    assert skipped >= 1 and g.opts[0].timestep == steps - skipped
    g.assert_state(exact=False, rel=1e-4)
    g.close()


@pytest.mark.parametrize("world", [1, 2, 4])
def test_buckets_reduced_during_backward_give_the_same_step(world):
    """oxz_grads_ready_async hands finished buckets in early (last buckets first, as backward produces them); the step
    then reduces the rest. The state must equal the checker's bit for bit, exactly as a plain step's does."""
    numel = [5000, 300, 70001, 513, 9000, 40000]
    no_decay = [False, True, False, True, False, False]
    if world == 1:
        from tests.helpers import Pair
        pair = Pair(numel, no_decay, ox.BF16, ox.BF16, seed=61, bucket_bytes=16384)
        nb = pair.opt.info.n_buckets
        assert nb >= 6
        cfg = ox.StepConfig(max_grad_norm=1e9, eps=1e-8)
        for s in range(2):
            pair.opt.grads_ready(cfg, nb - 2, 2)
            pair.opt.grads_ready(cfg, nb - 5, 3)
            res, ref = pair.step(cfg)
            assert (res.applied, res.timestep) == (1, s + 1) and abs(res.grad_norm - ref.grad_norm) <= 1e-5 * ref.grad_norm
            pair.assert_bit_equal()
        # a plain step afterwards still works, and call-order mistakes are errors, not hangs
        res, ref = pair.step(cfg)
        pair.assert_bit_equal()
        pair.opt.grads_ready(cfg, 0, 1)
        with pytest.raises(ox.OxzError, match="already handed in"):
            pair.opt.grads_ready(cfg, 0, 1)
        with pytest.raises(ox.OxzError, match="differs from the one"):
            pair.opt.step(ox.StepConfig(max_grad_norm=1e9, eps=1e-8, loss_scale=2.0))
        res, ref = pair.step(cfg)
        pair.assert_bit_equal()
        pair.close()
        return
    g = Group(world, [0] * world, "local", seed=62, numel=numel, no_decay=no_decay, bucket_bytes=16384 * world)
    nb = g.opts[0].info.n_buckets
    assert nb >= 4
    cfg = ox.StepConfig(max_grad_norm=1e9, eps=1e-8)
    for s in range(2):
        list(g.pool.map(lambda r: g.opts[r].grads_ready(cfg, nb - 1, 1), range(world)))
        list(g.pool.map(lambda r: g.opts[r].grads_ready(cfg, 1, nb - 3), range(world)))
        out, ref = g.step(cfg, extras=[1.0] * world)
        for res, extras in out:
            assert (res.applied, res.timestep) == (1, s + 1) and abs(res.grad_norm - ref.grad_norm) <= 1e-5 * ref.grad_norm
            assert extras == [float(world)]
        g.assert_state(exact=True)
    g.close()


def test_two_ranks_equal_one_rank_fed_the_summed_gradients():
    """tests/data_parallel.rs:226-269 (2 ranks x batch 2 == 1 rank x batch 4): the gradients are summed, never averaged,
    so two ranks must end bit-identical to a single rank that is handed the f32 sum of their gradients."""
    numel = [4096, 300, 70001, 513]
    no_decay = [False, True, False, True]
    g = Group(2, [0, 0], "local", gd=ox.F32, pd=ox.BF16, seed=71, numel=numel, no_decay=no_decay, grad_std=1.0)
    summed = [orc.sum_ranks([g.grads[0][i], g.grads[1][i]], orc.F32) for i in range(len(numel))]
    single = ox.DpOptimizer(numel, no_decay, ox.F32, ox.BF16, bucket_bytes=16384)
    from tests.helpers import seeded_state
    master, m, v, _ = seeded_state(numel, 71, 1.0, 2, ox.F32)
    for i in range(len(numel)):
        single.import_tensor(ffi.STATE_MASTER, i, master[i])
        single.import_tensor(ffi.STATE_EXP_AVG, i, m[i])
        single.import_tensor(ffi.STATE_EXP_AVG_SQ, i, v[i])
        single.import_tensor(ffi.STATE_WORK, i, orc.narrow(master[i], ox.BF16))
        single.import_tensor(ffi.STATE_GRADS, i, summed[i])
    cfg = ox.StepConfig(max_grad_norm=1.0)
    for _ in range(2):
        out, ref = g.step(cfg)
        one = single.step(cfg)
        assert {res.grad_norm for res, _ in out} == {out[0][0].grad_norm}
        assert abs(one.grad_norm - out[0][0].grad_norm) <= 1e-9 * one.grad_norm and one.clip_coef < 1.0
    same_coef = one.clip_coef == out[0][0].clip_coef
    for kind in (ffi.STATE_MASTER, ffi.STATE_EXP_AVG, ffi.STATE_EXP_AVG_SQ):
        for i, merged in enumerate(g.merged(kind)):
            alone = single.export_tensor(kind, i)
            if same_coef:
                assert np.array_equal(bits(merged), bits(alone)), (kind, i)
            else:  # the norm's partial sums are grouped differently; the coefficient may differ in its last bit
                ref64 = alone.astype(np.float64)
                assert np.all(np.abs(merged - ref64) <= 1e-6 * (np.abs(ref64) + math.sqrt(float(np.mean(ref64 ** 2))))), (kind, i)
    single.destroy()
    g.close()


def test_spike_guard_vetoes_the_same_step_on_every_rank():
    """tests/spike_guard.rs with two ranks: the guard judges the loss summed over ranks, so every rank skips the same
    step (skip list [F,F,F,T,F]); a spike skip with finite gradients leaves the optimizer and the loss scale untouched."""
    world = 2
    numel = [3000, 64]
    g = Group(world, [0, 0], "local", gd=ox.F16, pd=ox.F16, seed=81, numel=numel, no_decay=[False, True])
    cfg = ox.TrainerConfig(max_grad_norm=1e9, loss_scale=ox.LossScaleConfig(initial=1024.0, growth_interval=100),
                           spike_guard=ox.SpikeGuardConfig(window=4, z_threshold=6.0, min_steps=2))
    trainers = [ox.LitTrainerStep(cfg, g.opts[r]) for r in range(world)]
    for t in trainers:
        t.loss_probe = lambda index, loss: 1e3 if index == 3 else loss  # the scripted spike of src/metrics/state.rs:122-152
    history = [[] for _ in range(world)]
    for step in range(5):
        before = g.merged(ffi.STATE_MASTER)
        out = list(g.pool.map(lambda r: trainers[r].training_step(0.5 + 0.05 * (step % 2)), range(world)))
        for r, (loss, norm) in enumerate(out):
            history[r].append((loss, math.isfinite(norm), trainers[r].optimizer_timestep(), trainers[r].loss_scale_state().consecutive_ok))
        after = g.merged(ffi.STATE_MASTER)
        changed = any(not np.array_equal(bits(a), bits(b)) for a, b in zip(before, after))
        assert changed == (step != 3)
    assert history[0] == history[1]
    assert [h[2] for h in history[0]] == [1, 2, 3, 3, 4]          # the vetoed step does not count
    assert [h[3] for h in history[0]] == [1, 2, 3, 3, 4]          # and leaves the scaler's clean-step count alone
    assert history[0][3][0] == 1e3 and abs(history[0][0][0] - 1.0) < 1e-12  # the loss is the sum over the ranks
    assert all(t.spike_guard.state["skipped"] == 1 and t.spike_guard.state["observed"] == 4 for t in trainers)
    g.close()
