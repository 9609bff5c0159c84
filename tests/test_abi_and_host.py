"""CPU-side checks: the library loads and exports every declared symbol, the planner's layout is consistent,
and the C++ host logic agrees with the Python checker on the reference's known answers and on random cases."""
import ctypes as C
import math
import os
import re
import threading

import numpy as np
import pytest

import oxidizr_b200 as ox
from oxidizr_b200 import ffi, inventory
from oracle import host_logic as hl

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAN = float("nan")


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "oxz_dpstep.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(oxz_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = ox.lib()
    names = declared_symbols()
    assert len(names) >= 40
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/oxz_dpstep.h but not exported"
        assert n in ffi.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(ffi.SIGNATURES) == names
    assert L.oxz_abi_version() == 1
    assert ffi.status_name(ffi.ERR_NCCL) == "OXZ_ERR_NCCL"


def test_no_gpu_call_fails_loudly_instead_of_falling_back():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(ox.OxzError, match="OXZ_ERR_CUDA"):
        ox.DpOptimizer([10])


def test_calls_that_need_device_state_say_so_before_it_exists():
    # a plan is host-only until oxz_state_alloc: the newer entry points refuse it with a status, not a crash
    opt = ox.DpOptimizer([10, 300], allocate=False)
    for call in (opt.grad_norms_per_tensor, opt.exchange_kind, opt.launch_geometry):
        with pytest.raises(ox.OxzError, match="OXZ_ERR_STATE"):
            call()
    assert opt.last_update_kernel() == 0 and opt.last_pull_kernel() == 0
    with pytest.raises(ox.OxzError, match="limit_ms 0 is outside"):
        ox.selftest_bounded_wait(0, limit_ms=0)
    opt.destroy()


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("bucket_bytes", [0, 4096, 1 << 20])
def test_plan_layout_covers_every_element_once(world, bucket_bytes):
    numel = [1, 0, 255, 256, 257, 5000, 33, 70000]
    mode = ox.SYNC_SINGLE if world == 1 else ox.SYNC_P2P
    plans = [ox.DpOptimizer(numel, None, ox.BF16, ox.BF16, world=world, rank=r, sync_mode=mode,
                            bucket_bytes=bucket_bytes, allocate=False) for r in range(world)]
    p0 = plans[0]
    info = p0.info
    assert info.numel_total == sum(numel) and info.tile_elems == 256
    assert all(o % 256 == 0 for o in p0.offsets)
    for a, b, n in zip(p0.offsets, p0.offsets[1:], numel):
        assert b - a == (n + 255) // 256 * 256
    assert info.padded_total % (256 * world) == 0 and info.local_elems * world == info.padded_total
    # buckets tile the flat space; shards tile each bucket in rank order
    pos = 0
    for b in range(info.n_buckets):
        start, length, _, _ = p0.bucket(b, 0)
        assert start == pos and length % (256 * world) == 0
        spos = start
        for r in range(world):
            s, l, ss, sl = plans[r].bucket(b, r)
            assert (s, l) == (start, length) and ss == spos and sl == length // world
            spos += sl
        pos += length
    assert pos == info.padded_total
    # every element has exactly one owner and local indices are a bijection onto [0, local_elems)
    rng = np.random.default_rng(0)
    probes = set(rng.integers(0, info.padded_total, 300).tolist()) | {0, info.padded_total - 1}
    for e in probes:
        owners = [(r, plans[r].local_index(e, r)) for r in range(world)]
        owned = [(r, li) for r, li in owners if li is not None]
        assert len(owned) == 1 and owned[0][1] < info.local_elems
    seen = set()
    for e in range(0, info.padded_total, 256):
        li = plans[world - 1].local_index(e, world - 1)
        if li is not None:
            assert li % 256 == 0 and li not in seen
            seen.add(li)
    assert len(seen) * 256 == info.local_elems
    for p in plans:
        p.destroy()


def test_plan_rejects_bad_descriptions():
    with pytest.raises(ox.OxzError, match="rank 2 is not below world size 2"):
        ox.DpOptimizer([10], world=2, rank=2, sync_mode=ox.SYNC_P2P, allocate=False)
    with pytest.raises(ox.OxzError, match="OXZ_SYNC_SINGLE"):
        ox.DpOptimizer([10], world=2, rank=0, sync_mode=ox.SYNC_SINGLE, allocate=False)
    with pytest.raises(ox.OxzError, match="dtype"):
        ox.DpOptimizer([10], grad_dtype=7, allocate=False)
    with pytest.raises(ox.OxzError, match="groups"):
        ox.DpOptimizer([1] * 9, lr_scale=[float(i + 1) for i in range(9)], allocate=False)
    with pytest.raises(ox.OxzError, match="no device state"):
        ox.DpOptimizer([10], allocate=False).step(ox.StepConfig())


def test_inventories_match_the_reference_models():
    want = {"nano_dense": (75, 134_188_544, 17), "llama-3.2-1b": (146, 1_235_814_400, 33),
            "qwen3-1.7b": (310, 1_720_574_976, 113), "moe-1b": (411, 1_031_398_400, 25)}
    for key, (T, P, nd) in want.items():
        tensors = inventory.PARAM_SETS[key]()
        plan = ox.DecayPlan(ox.WeightDecaySpec("skip_1d"), tensors)
        assert (len(tensors), sum(t.elements for t in tensors), sum(plan.no_decay)) == (T, P, nd), key
    llama = ox.DecayPlan(ox.WeightDecaySpec("skip_1d"), inventory.llama_3_2_1b())
    assert llama.no_decay_elements == 67_584
    hyb = inventory.hybrid()
    names = {t.name.rsplit(".", 1)[-1] for t, nd in zip(hyb, ox.DecayPlan(ox.WeightDecaySpec("skip_1d"), hyb).no_decay) if nd}
    assert {"A_log", "D", "dt_bias", "b_bias", "c_bias", "bias", "weight"} <= names
    assert "summary" and "do not" in llama.summary(0.1)


# ---- host logic of the library against the checker and the reference's known answers

def test_scaler_matches_checker_on_random_sequences():
    rng = np.random.default_rng(1)
    for trial in range(20):
        cfg = dict(initial=float(2 ** rng.integers(4, 20)), growth_interval=int(rng.integers(1, 6)))
        a, b = ox.LossScaler(ox.LossScaleConfig(**cfg)), hl.LossScaler(hl.LossScaleConfig(**cfg))
        for _ in range(60):
            overflow, spike = bool(rng.random() < 0.2), bool(rng.random() < 0.2)
            a.record_step(overflow, spike)
            hl.record_after_step(b, overflow, spike)
            assert (a.state().scale, a.state().consecutive_ok) == (b.state().scale, b.state().consecutive_ok)
    s = ox.LossScaler(ox.LossScaleConfig(initial=64.0, growth_interval=2))
    table = []
    for _ in range(4):
        s.record_step(False)
        table.append((s.state().scale, s.state().consecutive_ok))
    assert table == [(64.0, 1), (128.0, 0), (128.0, 1), (256.0, 0)]  # tests/loss_scale.rs:180-214
    for bad, key in [(dict(initial=0.0), "initial"), (dict(growth_factor=1.0), "growth_factor"),
                     (dict(backoff_factor=1.0), "backoff_factor"), (dict(growth_interval=0), "growth_interval")]:
        with pytest.raises(ox.OxzError, match=f"trainer.loss_scale.{key}"):
            ox.LossScaler(ox.LossScaleConfig(**bad))
    with pytest.raises(ox.OxzError):
        s.restore(ox.GradScalerState(NAN, 0))
    s.restore(ox.GradScalerState(512.0, 7))
    assert (s.state().scale, s.state().consecutive_ok) == (512.0, 7)


def test_decay_rule_matches_checker():
    from tests.test_oracle_pins import NAMES
    for rule in ("decay_all", "skip_1d", "skip_all"):
        for pats in ([], ["embed_tokens", "lora_"]):
            if pats and rule != "skip_1d":
                with pytest.raises(ox.OxzError, match="skip_1d"):
                    ox.WeightDecaySpec(rule, pats).check()
                continue
            a, b = ox.WeightDecaySpec(rule, pats), hl.WeightDecaySpec(rule, pats)
            for name, rank in NAMES + [("D", 3), ("x.D", 2), ("x.Dx", 2), ("model.a.bias_b", 2), ("bias", 5)]:
                assert a.excludes(name, rank) == b.excludes(name, rank), (rule, name)
    with pytest.raises(ox.OxzError, match=r"no_decay_patterns\[0\] is empty"):
        ox.WeightDecaySpec("skip_1d", [""]).check()
    plan = ox.DecayPlan(ox.WeightDecaySpec("skip_1d"), [ox.TensorInfo("model.embed_tokens.weight", (2, 3), id=7),
                                                         ox.TensorInfo("lm_head.weight", (2, 3), id=7),
                                                         ox.TensorInfo("model.norm.weight", (3,), id=9)])
    assert plan.no_decay == [False, True] and (plan.decay_tensors, plan.decay_elements, plan.no_decay_elements) == (1, 6, 3)


def test_spike_guard_matches_checker():
    rng = np.random.default_rng(2)
    for trial in range(10):
        cfg = dict(window=int(rng.integers(1, 20)), z_threshold=float(rng.uniform(0.5, 6)), min_steps=int(rng.integers(0, 8)),
                   action="skip" if trial % 2 == 0 else "warn")
        a, b = ox.SpikeGuard(ox.SpikeGuardConfig(**cfg)), hl.SpikeGuard(hl.SpikeGuardConfig(**cfg))
        for i in range(80):
            loss = float(rng.normal(2.0, 0.1)) if rng.random() > 0.1 else float(rng.choice([50.0, NAN, math.inf]))
            assert a.judge(i, loss) == b.judge(i, loss)
            sa, sb = a.state, b.state
            assert (sa["mean"], sa["variance"], sa["observed"], sa["detected"], sa["skipped"]) == \
                   (sb.mean, sb.variance, sb.observed, sb.detected, sb.skipped)
    g = ox.SpikeGuard(ox.SpikeGuardConfig(window=4, z_threshold=6.0, min_steps=2))
    losses = [1e3 if i == 3 else 1.0 + 0.1 * (i % 2) for i in range(5)]
    assert [g.judge(i, l) for i, l in enumerate(losses)] == [False, False, False, True, False]  # src/metrics/state.rs:122-152
    with pytest.raises(ox.OxzError, match="window"):
        ox.SpikeGuard(ox.SpikeGuardConfig(window=0))
    with pytest.raises(ox.OxzError, match="z_threshold"):
        ox.SpikeGuard(ox.SpikeGuardConfig(z_threshold=0.0))


def test_lr_plan_is_bitwise_equal_to_the_closed_form():
    # src/schedule.rs:323-351
    base, total = 3e-4, 110
    for schedule in ("constant", "cosine", "linear"):
        for warmup in (0, 10, 120):
            for min_ratio in (0.0, 0.1, 0.37):
                plan = ox.LrPlan(base, schedule, warmup, total, min_ratio)
                for step in range(total + 25):
                    assert plan.lr_at(step) == hl.lr_at(step, base, schedule, warmup, total, min_ratio)
    for shape in ("linear", "cosine", "sqrt"):
        plan = ox.LrPlan(base, "wsd", 10, total, 0.1, decay_steps=20, decay_shape=shape)
        for step in range(total + 25):
            assert plan.lr_at(step) == hl.lr_at(step, base, "wsd", 10, total, 0.1, decay_steps=20, decay_shape=shape)
        assert plan.lr_at(90) == base and plan.lr_at(total) == base * 0.1
    assert ox.LrPlan(base, "wsd", 10, total, 0.1).lr_at(99) == base  # ceil(110 * 0.1) = 11 decay steps
    with pytest.raises(ox.OxzError, match="decay_steps"):
        ox.LrPlan(base, "wsd", 10, total, 0.1, decay_steps=101)
    with pytest.raises(ox.OxzError, match="min_lr_ratio"):
        ox.LrPlan(base, "cosine", 0, 10, 1.5)


def test_row_arithmetic_matches_checker_bit_for_bit():
    for rows, bs, world in [(10, 3, 1), (9, 3, 1), (7, 1, 1), (5, 5, 1), (11, 4, 1), (23, 3, 2), (22, 3, 2), (11, 1, 3)]:
        a, b = ox.RowLayout(rows, bs, world), hl.RowLayout(rows, bs, world)
        for start_row in range(rows + 1):
            for n in range(3 * a.batches_per_epoch() + 3):
                got = a.advance(ox.DataPosition(2, start_row), n)
                want = b.advance(hl.DataPosition(2, start_row), n)
                assert (got.epoch, got.row) == (want.epoch, want.row)
    # rank windows concatenate to the global window and the token indices are exact (tests/data_ranks.rs:94-122)
    seq, rows = 3, 23
    tokens = np.arange(rows * (seq + 1) + 2, dtype=np.uint32) * 7 % 100003
    glob, ranks = ox.RowLayout(rows, 6, 1), ox.RowLayout(rows, 3, 2)
    gpos, rpos = ox.DataPosition(), [ox.DataPosition(), ox.DataPosition()]
    cpos = hl.DataPosition()
    for _ in range(10):
        grows, gin, gtg, gpos = glob.next_window(gpos, 0, seq, tokens)
        parts = []
        for k in range(2):
            r, i, t, rpos[k] = ranks.next_window(rpos[k], k, seq, tokens)
            crow, cin, ctg, cnext = hl.rank_window(hl.RowLayout(rows, 3, 2), cpos, k, seq)
            assert r.tolist() == crow
            assert np.array_equal(i, tokens[np.array(cin)].astype(np.int64))
            assert np.array_equal(t, tokens[np.array(ctg)].astype(np.int64))
            parts.append((r, i, t))
        cpos = cnext
        assert np.array_equal(np.concatenate([p[0] for p in parts]), grows)
        assert np.array_equal(np.concatenate([p[1] for p in parts]), gin)
        assert np.array_equal(np.concatenate([p[2] for p in parts]), gtg)
        assert rpos[0] == rpos[1] == gpos and (gpos.epoch, gpos.row) == (cpos.epoch, cpos.row)
    for args, msg in [((5, 3, 2), "one global batch of 6 rows"), ((3, 4, 1), "fewer than batch_size 4"),
                      ((5, 3, 0), "world size is 0"), ((3, 0, 1), "batch_size is 0")]:
        with pytest.raises(ox.OxzError, match=msg):
            ox.RowLayout(*args)
    with pytest.raises(ox.OxzError, match="rank 2 is not below world size 2"):
        ranks.next_window(ox.DataPosition(), 2, seq)


def test_shuffled_row_order_with_the_callers_permutations_matches_the_checker():
    # EpochOrder::row (src/data/rows.rs:240-256): the row at `slot` of `epoch` is that epoch's permutation at `slot`;
    # the permutation is the caller's (here any seeded one from NumPy: the library never makes it)
    seq, rows, bs, world = 3, 23, 3, 2
    tokens = (np.arange(rows * (seq + 1) + 1, dtype=np.uint64) * 2654435761 % 100003).astype(np.uint32)
    perm_of = lambda epoch: np.random.default_rng(1000 + epoch).permutation(rows).astype(np.uint32)  # noqa: E731
    layout, cl = ox.RowLayout(rows, bs, world), hl.RowLayout(rows, bs, world)
    pos, cpos = [ox.DataPosition(), ox.DataPosition()], hl.DataPosition()
    seen_epochs = set()
    for step in range(11):  # crosses three epoch boundaries (3 global batches per epoch)
        union = []
        for k in range(world):
            epoch = layout.batch_epoch(pos[k])
            assert epoch == cl.batch_start(cpos).epoch
            seen_epochs.add(epoch)
            r, i, t, pos[k] = layout.next_window(pos[k], k, seq, tokens, row_order=(epoch, perm_of(epoch)))
            crow, cin, ctg, cnext = hl.rank_window(cl, cpos, k, seq, order=perm_of)
            assert r.tolist() == crow
            assert np.array_equal(i, tokens[np.array(cin)].astype(np.int64))
            assert np.array_equal(t, tokens[np.array(ctg)].astype(np.int64))
            union += crow
        assert len(set(union)) == bs * world  # every row of the global batch once
        cpos = cnext
        assert (pos[0].epoch, pos[0].row) == (pos[1].epoch, pos[1].row) == (cpos.epoch, cpos.row)
    assert seen_epochs == {0, 1, 2, 3}
    # within an epoch the batches visit distinct rows (src/data/rows.rs:376-411: an epoch reads every row once)
    p, rows_seen = ox.DataPosition(), []
    for _ in range(3):
        for k in range(world):
            r, _, _, nxt = layout.next_window(p, k, seq, row_order=(0, perm_of(0)))
            rows_seen += r.tolist()
        p = nxt
    assert len(set(rows_seen)) == 18
    # the wrong epoch's order, a wrong length and a non-permutation are refused
    with pytest.raises(ox.OxzError, match="reads epoch 0 and the row order given is epoch 1"):
        layout.next_window(ox.DataPosition(), 0, seq, row_order=(1, perm_of(1)))
    with pytest.raises(ox.OxzError, match="holds 22 rows and the layout 23"):
        layout.next_window(ox.DataPosition(), 0, seq, row_order=(0, perm_of(0)[:22]))
    bad = perm_of(0).copy()
    bad[1] = bad[0]
    with pytest.raises(ox.OxzError, match="twice"):
        ffi.check(ox.lib().oxz_rows_check_permutation(bad.ctypes.data_as(C.POINTER(C.c_uint32)), bad.size))
    bad[1] = 99
    with pytest.raises(ox.OxzError, match="past its 23 rows"):
        ffi.check(ox.lib().oxz_rows_check_permutation(bad.ctypes.data_as(C.POINTER(C.c_uint32)), bad.size))


def test_step_weighting_matches_checker():
    assert ox.step_weighting(2, 2, 0, 0) == (4, None)
    assert ox.step_weighting(1, 2, 12, 2) == (2, 12)
    with pytest.raises(ox.OxzError, match="1 of 2 data-parallel ranks carry a loss mask"):
        ox.step_weighting(1, 2, 5, 1)
