"""World-size-2 checks on CPU over gloo: the host-side logic of the multi-rank path.

Two processes build their own rank's plan, agree on the shard layout through the process group, and run the
sharded form of the step with the CPU checker's passes as the per-shard arithmetic (reduce-scatter -> norm partials
-> one all-reduce of the partials -> update on the owned shard -> all-gather of the weights). The result must be
bit-identical to the checker's replicated step: this pins the ZeRO-1-style sharding (shard boundaries cutting
through tensors, padding, the ownership map) independently of any GPU.
"""
import math
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

NUMEL = [1, 300, 4096, 70001, 0, 513, 9000]
NO_DECAY = [True, True, False, False, False, True, False]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import oxidizr_b200 as ox
    from oracle import dpstep as orc
    from tests.helpers import seeded_state

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc.lib().orc_set_num_threads(2)
    plan = ox.DpOptimizer(NUMEL, NO_DECAY, ox.BF16, ox.BF16, world=world, rank=rank, sync_mode=ox.SYNC_P2P,
                          bucket_bytes=16384, allocate=False)
    info = plan.info
    padded, local = info.padded_total, info.local_elems

    # every rank must derive the same layout
    mine = torch.tensor([padded, local, info.n_buckets, info.bucket_elems] + plan.offsets, dtype=torch.int64)
    both = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(both, mine)
    assert all(torch.equal(b, mine) for b in both)

    # ownership: flat index -> local index on exactly one rank
    owner = np.full(padded, -1, np.int64)
    lidx = np.zeros(padded, np.int64)
    for b in range(info.n_buckets):
        for r in range(world):
            _, _, ss, sl = plan.bucket(b, r)
            li = plan.local_index(ss, r)
            assert li is not None and owner[ss:ss + sl].max(initial=-1) == -1
            owner[ss:ss + sl] = r
            lidx[ss:ss + sl] = li + np.arange(sl)
    assert owner.min() >= 0
    mine_mask = owner == rank
    assert mine_mask.sum() == local and sorted(lidx[mine_mask].tolist()) == list(range(local))

    master, m, v, grads = seeded_state(NUMEL, 31, 1.0, world, ox.BF16)  # grad_std 1: the norm clip is active

    def flat(arrs, dtype):
        out = np.zeros(padded, dtype)
        for off, a in zip(plan.offsets, arrs):
            out[off:off + a.size] = a
        return out
    g_flat = flat(grads[rank], np.uint16)

    # "reduce-scatter": each rank receives every rank's values of its own shard and adds them in rank order in f32
    all_g = [torch.zeros(padded * 2, dtype=torch.uint8) for _ in range(world)]  # gloo moves bytes
    dist.all_gather(all_g, torch.from_numpy(g_flat.view(np.uint8)))
    shard = [np.ascontiguousarray(t.numpy().view(np.uint16)[mine_mask]) for t in all_g]
    summed = orc.sum_ranks(shard, orc.BF16)

    # norm partial of the shard, then the one all-reduce of the step
    part = torch.tensor([orc.sumsq(summed)], dtype=torch.float64)
    parts = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(parts, part)
    norm = math.sqrt(sum(float(p) for p in parts))  # rank order: the same bits on every rank
    cfg = orc.StepConfig(max_grad_norm=1.0)
    coef = np.float32(cfg.max_grad_norm / (norm + cfg.clip_eps)) if norm > cfg.max_grad_norm else np.float32(1.0)
    if coef != 1.0:
        orc.lib().orc_scale(summed.ctypes.data, summed.size, coef)

    # the update on the owned shard, group by group
    p_l, m_l, v_l = (np.ascontiguousarray(flat(x, np.float32)[mine_mask]) for x in (master, m, v))
    w_l = np.zeros(local, np.uint16)
    group = np.zeros(padded, np.int8)
    for off, n, nd in zip(plan.offsets, NUMEL, NO_DECAY):
        group[off:off + n] = 1 if nd else 0
    g_l = group[mine_mask]
    for gid, wd in ((0, cfg.weight_decay), (1, 0.0)):
        sel = np.nonzero(g_l == gid)[0]
        s = orc.adam_prepare(cfg.lr, 1.0, cfg.beta1, cfg.beta2, cfg.eps, wd, 1)
        pp, mm, vv, gg = (np.ascontiguousarray(a[sel]) for a in (p_l, m_l, v_l, summed))
        ww = np.zeros(sel.size, np.uint16)
        orc.adamw(pp, mm, vv, gg, s, ww, orc.BF16)
        p_l[sel], m_l[sel], v_l[sel], w_l[sel] = pp, mm, vv, ww

    # "all-gather" of the working weights
    w_all = [torch.zeros(local * 2, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(w_all, torch.from_numpy(w_l.view(np.uint8)))
    w_flat = np.zeros(padded, np.uint16)
    for r in range(world):
        w_flat[owner == r] = w_all[r].numpy().view(np.uint16)

    # the replicated step of the checker on the same inputs
    ref = orc.StepState([x.copy() for x in master], [x.copy() for x in m], [x.copy() for x in v],
                        [orc.to_bf16(x) for x in master], orc.BF16, lr_scale=[1.0] * len(NUMEL),
                        group_wd=[0.0 if nd else float("nan") for nd in NO_DECAY])
    res = orc.step(ref, grads, orc.BF16, cfg)
    assert res.applied == 1 and abs(res.grad_norm - norm) <= 1e-12 * norm and res.clip_coef < 1.0
    ok = True
    for arrs, loc in ((ref.master, p_l), (ref.exp_avg, m_l), (ref.exp_avg_sq, v_l)):
        want = flat(arrs, np.float32)[mine_mask]
        ok &= np.array_equal(want.view(np.uint32), loc.view(np.uint32))
    for off, n, w in zip(plan.offsets, NUMEL, ref.work):
        ok &= np.array_equal(w_flat[off:off + n], w)
    with open(os.path.join(result_dir, f"rank{rank}.ok"), "w") as f:
        f.write("1" if ok else "0")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_sharded_step_equals_replicated_step_over_gloo(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.ok").read_text() == "1", f"rank {r}: the sharded step differs from the replicated one"


def test_reference_arm_prints_on_rank_zero_only(tmp_path):
    """bench.py --impl reference under a 2-rank launch: rank 0 prints the line, the other rank exits 0 silently."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "2",
                          "--steps", "1", "--warmup", "0"], env=env, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and out.stdout.strip() == ""
