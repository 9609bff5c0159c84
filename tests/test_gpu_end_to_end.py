"""One whole data-parallel step of the hybrid Mamba3/GDN/attention parameter set, end to end through the library:
rank-sliced loader (batch 8, seq 1024, uniform tokens, vocab 32000) -> a stand-in backward that turns each rank's
batch into per-tensor gradients -> flatten into the buckets -> the trainer's half of the step -> the CPU checker.

The forward/backward of Mamba3 and GDN is outside the path; the stand-in only has to produce, per rank, gradients
that depend on that rank's tokens, for the real inventory with its many tiny tensors (A_log, D, dt_bias, conv1d),
so that bucket packing, the no-decay mask, the rank sum and the update are exercised together."""
import math
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

import oxidizr_b200 as ox
from oxidizr_b200 import ffi, inventory
from oracle import dpstep as orc
from tests.helpers import NAN, bits

pytestmark = pytest.mark.gpu

BATCH, SEQ, VOCAB = 8, 1024, 32000


def stand_in_backward(tensors, inputs, targets, rank_seed):
    """Per-tensor bf16 gradients on the device, a deterministic function of the batch's tokens."""
    import torch
    key = int((inputs.sum() * 31 + targets.sum()).item()) % (2 ** 31)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(key + rank_seed)
    scale = 1e-3 * (1.0 + (key % 7) / 7.0)
    return [(torch.empty(t.elements, device="cuda").normal_(0.0, scale, generator=gen)).to(torch.bfloat16) for t in tensors]


@pytest.mark.parametrize("world", [1, 8])
def test_hybrid_set_steps_end_to_end(world, tmp_path):
    import torch
    from oxidizr_b200.interop import device_view
    tensors = inventory.hybrid()
    plan = ox.DecayPlan(ox.WeightDecaySpec("skip_1d"), tensors)
    numel = [t.elements for t in tensors]
    T = len(numel)
    assert sum(1 for n in numel if n <= 64) >= 20, "the set must hold many tiny tensors"
    rng = np.random.default_rng(3)
    tokens = rng.integers(0, VOCAB, size=(world * BATCH * 3 + 1) * (SEQ + 1) + 5, dtype=np.uint32)
    path = str(tmp_path / "tokens.bin")
    tokens.astype("<u4").tofile(path)

    master0 = [(rng.standard_normal(n) * 0.02).astype(np.float32) for n in numel]
    comms = ox.Communicator.local_group(world, [0] * world, timeout=120.0) if world > 1 else [None]
    pool = ThreadPoolExecutor(world)
    cfg = ox.TrainerConfig(learning_rate=3e-4, adamw_eps=1e-6, weight_decay=0.1, max_grad_norm=1.0, lr_schedule="cosine",
                           warmup_steps=2, total_steps=10, min_lr_ratio=0.1)

    def make(r):
        opt = ox.DpOptimizer(numel, plan.no_decay, ox.BF16, ox.BF16, world=world, rank=r, comm=comms[r], bucket_bytes=4 << 20)
        for i in range(T):
            opt.import_tensor(ffi.STATE_MASTER, i, master0[i])
            opt.import_tensor(ffi.STATE_WORK, i, orc.to_bf16(master0[i]))
        loader = ox.LitDataLoader(path, BATCH, SEQ, rank=r, world_size=world)
        return opt, loader, ox.LitTrainerStep(cfg, opt)
    ranks = list(pool.map(make, range(world)))

    ref = orc.StepState([p.copy() for p in master0], [np.zeros(n, np.float32) for n in numel],
                        [np.zeros(n, np.float32) for n in numel], [orc.to_bf16(p) for p in master0], orc.BF16,
                        lr_scale=[1.0] * T, group_wd=[0.0 if nd else NAN for nd in plan.no_decay])
    ref_lr = ox.LrPlan(3e-4, "cosine", 2, 10, 0.1)

    for step in range(3):
        def one(r):
            opt, loader, trainer = ranks[r]
            i_ptr, t_ptr, rows = loader.next_batch()
            torch.cuda.synchronize()
            inputs = device_view(i_ptr, BATCH * SEQ * 8, torch.int64)
            targets = device_view(t_ptr, BATCH * SEQ * 8, torch.int64)
            assert int(inputs.max()) < VOCAB and torch.equal(inputs.view(BATCH, SEQ)[:, 1:], targets.view(BATCH, SEQ)[:, :-1])
            grads = stand_in_backward(tensors, inputs, targets, r)
            opt.flatten_grads([g.data_ptr() for g in grads])
            torch.cuda.synchronize()
            loss, norm = trainer.training_step(2.0 + 0.1 * r)
            return rows, [g.view(torch.int16).cpu().numpy().view(np.uint16) for g in grads], loss, norm
        out = list(pool.map(one, range(world)))
        # the ranks' rows concatenate to the global batch of this step
        rows = [x for o in out for x in o[0]]
        assert rows == list(range(step * world * BATCH, (step + 1) * world * BATCH))
        want = orc.step(ref, [o[1] for o in out], orc.BF16,
                        orc.StepConfig(lr=ref_lr.lr_at(step), eps=1e-6, weight_decay=0.1, max_grad_norm=1.0))
        for _, _, loss, norm in out:
            assert abs(loss - sum(2.0 + 0.1 * r for r in range(world))) < 1e-12  # the loss is summed over ranks
            assert norm == want.reported_norm == 1.0 and want.applied == 1
    # state against the checker after three clipped steps
    for kind, arrs in ((ffi.STATE_MASTER, ref.master), (ffi.STATE_EXP_AVG, ref.exp_avg), (ffi.STATE_EXP_AVG_SQ, ref.exp_avg_sq)):
        for i, n in enumerate(numel):
            got = np.full(n, np.nan, np.float32)
            for opt, _, _ in ranks:
                opt.export_tensor(kind, i, got)
            b64 = arrs[i].astype(np.float64)
            tol = 3e-6 * (np.abs(b64) + math.sqrt(float(np.mean(b64 ** 2)))) + 1e-30
            assert np.all(np.abs(got - b64) <= tol), (kind, tensors[i].name)
    # every rank ends with the same working weights, and no-decay tensors of size <= 64 are among those updated
    w0 = [ranks[0][0].export_tensor(ffi.STATE_WORK, i) for i in range(T)]
    for opt, _, _ in ranks[1:]:
        for i in range(T):
            assert np.array_equal(opt.export_tensor(ffi.STATE_WORK, i), w0[i])
    assert ranks[0][2].optimizer_timestep() == 3
    for opt, loader, _ in ranks:
        loader.close()
        opt.destroy()
    for c in comms:
        if c is not None:
            c.destroy()
