#!/usr/bin/env python
"""Benchmark of the data-parallel optimizer step (gradient sync + unscale/inf check + global-norm clip + fused AdamW
+ weight write-back) on the Llama-3.2-1B parameter set, with a self-check of the result at every rank count.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU restatement of the reference's path on the host cores
    ... --workload qwen3-1.7b --dtype f16 --loss-scale 65536 --inject-inf     # f16 gradients, overflow scenario
    ... --workload moe-1b --absent skip|zero                                   # experts no rank routed to

One JSON line on stdout (rank 0). A step is one pass of the whole path over one set of synthetic gradients:
16-bit gradients ~N(0,1e-3) (times the loss scale) from seed+rank, f32 master ~N(0,0.02), m ~N(0,1e-4),
v = |N(0,1e-6)|. `value` is params/s with the gradients already resident in HBM; `e2e` is the same call fed from
pinned host memory. After the timed steps an untimed leg checks the result (`check`): every rank's weights equal,
the norm against a float64 sum over the ranks' gradients, and sampled tensors bit for bit against the CPU checker.
A failed check makes the process exit non-zero after printing the line.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "dp_sync_clip_adamw_step_params_per_s"
UNIT = "params/s"
WORKLOAD = "llama-3.2-1b"
SEED = 1234
HYPER = dict(lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, max_grad_norm=1.0)
# Algorithmic HBM bytes per parameter: the norm pass reads the gradient (2 or 4); the update reads gradient +
# master 4 + m 4 + v 4 and writes master 4 + m 4 + v 4 + the working weight: 28 for 16-bit and for all-f32 alike.
BYTES_UPDATE = 28
# DRAM bytes over algorithmic bytes of k_adamw from one ncu capture of a smaller case of the same kernel
# (nano_dense, 134 M parameters): 3.7015 GB read+write for 3.7573 GB algorithmic.
ADAMW_TRAFFIC_RATIO = 3.7015 / 3.7573
# The same for the update kernel with peers (k_adamw_wide reading the f32 sum, 30 B per owned parameter) from a capture
# on two GPUs with 50 M owned parameters: 800.84 MB read + 641.82 MB written for 1500.03 MB algorithmic (the part of
# the write-back still in L2 at the kernel's end weighs more on that small case).
ADAMW_PEER_TRAFFIC_RATIO = (800.84 + 641.82) / 1500.03
# NVLink 5 per direction and GPU: nominal, and the peer-copy figure measured on this pool's B200s.
NVLINK_NOMINAL_GBS, NVLINK_MEASURED_GBS = 900.0, 770.0
NVLINK_MEASURED_SOURCE = "peer copy per direction measured on this pool (770 GB/s; nominal 900)"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU through NVML while the timed region runs.
    Read-only: it queries, it never sets anything."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index: int):
        self.index, self.sm, self.bits, self.stop_flag, self.thread, self.max_mhz = index, [], 0, False, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()

    def stop(self) -> dict:
        if self.nv is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["nvml unavailable"]}
        self.stop_flag = True
        self.thread.join(2.0)
        reasons = sorted(k for k, b in self.REASONS.items() if self.bits & b)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "samples": len(self.sm), "reasons": reasons}


def tiled_normal(n: int, std: float, seed: int, absolute: bool = False) -> np.ndarray:
    """n seeded N(0, std) values; a 4M-value block repeated, which keeps host generation short."""
    block = np.random.default_rng(seed).standard_normal(min(n, 1 << 22)).astype(np.float32) * np.float32(std)
    if absolute:
        block = np.abs(block)
    return np.resize(block, n)


def absent_tensors(tensors, seed: int = SEED) -> list[int]:
    """The mixture-of-experts case: per layer, 2 of the 8 routed experts (a seeded choice) were routed to by no rank;
    their three projections have no gradient this step. Empty for a set without routed experts."""
    rng = np.random.default_rng(seed + 77)
    layers: dict[str, dict[int, list[int]]] = {}
    for i, t in enumerate(tensors):
        if ".moe.experts." in t.name:
            layer, rest = t.name.split(".moe.experts.")
            layers.setdefault(layer, {}).setdefault(int(rest.split(".")[0]), []).append(i)
    out = []
    for layer in sorted(layers):
        experts = sorted(layers[layer])
        for e in sorted(rng.choice(len(experts), size=min(2, len(experts)), replace=False).tolist()):
            out += layers[layer][experts[e]]
    return sorted(out)


# ------------------------------------------------------------------ the CPU arm
def product_library_mapped() -> bool:
    with open("/proc/self/maps") as f:
        return "liboxz_dpstep" in f.read()


def cpu_arm(args, steps: int, warmup: int, threads: int | None = None, world: int = 1):
    """The reference's CPU optimizer path, restated (the reference is Rust over un-vendored crates and cannot be built
    here), on the WHOLE parameter set of the workload with every host core the process may use. With world > 1 the
    step first sums that many gradient buffers in f32, as the reference's in-process communicator does
    (src/dp/reduce.rs:30-60). Nothing of the product library is loaded: the parameter inventory is plain data and the
    decay groups come from the checker's own restatement of the rule."""
    from oracle import dpstep as orc
    from oracle import host_logic as hl
    from oxidizr_b200 import inventory  # names and shapes only; no entry point of the library is touched

    tensors = inventory.PARAM_SETS[args.workload]()
    no_decay, _, _, _ = hl.decay_plan(hl.WeightDecaySpec("skip_1d"), [(i, t.name, len(t.shape), t.elements) for i, t in enumerate(tensors)])
    numel = [t.elements for t in tensors]
    P = sum(numel)
    # the thread count is set here: a launcher may have exported OMP_NUM_THREADS=1 for its workers
    want = threads or len(os.sched_getaffinity(0))
    orc.lib().orc_set_num_threads(want)
    cores = orc.lib().orc_num_threads()
    code = {"bf16": orc.BF16, "f16": orc.F16, "f32": orc.F32}[args.dtype]
    scale = args.loss_scale if args.loss_scale else 1.0
    master = [tiled_normal(n, 0.02, SEED + i) for i, n in enumerate(numel)]
    work = [orc.narrow(p, code) for p in master] if code != orc.F32 else None
    state = orc.StepState(master, [tiled_normal(n, 1e-4, SEED + 100 + i) for i, n in enumerate(numel)],
                          [tiled_normal(n, 1e-6, SEED + 200 + i, True) for i, n in enumerate(numel)],
                          work, code, lr_scale=[1.0] * len(numel),
                          group_wd=[0.0 if i in no_decay else float("nan") for i in range(len(numel))], timestep=1)
    gone = set(absent_tensors(tensors)) if args.absent != "none" else set()
    grads = []
    for i, n in enumerate(numel):
        if i in gone:
            grads.append(None if args.absent == "skip" else orc.narrow(np.zeros(n, np.float32), code))
        else:
            grads.append(orc.narrow(tiled_normal(n, 1e-3 * scale, SEED + 300 + i), code))
    cfg = orc.StepConfig(**HYPER, loss_scale=args.loss_scale if args.loss_scale else float("nan"))
    ranks = [grads] * max(world, 1)  # every rank's buffer holds the same values: only the work of the sum matters here
    for _ in range(warmup):
        orc.step(state, ranks, code, cfg)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.step(state, ranks, code, cfg)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    sample = (f"the whole set: {len(numel)} tensors, {P} params, {steps} steps after {warmup} warm-up, "
              f"{max(world, 1)} rank buffer(s) summed, {cores} OpenMP threads")
    return P / dt, dt * 1e3, cores, sample, P


def workload_config(args, P: int, T: int, world: int, sync: str) -> dict:
    return {"workload": args.workload, "params": P, "tensors": T, "grad_dtype": args.dtype, "param_dtype": args.dtype,
            "world": world, "sync": sync, "loss_scale": args.loss_scale or None, "absent": args.absent, "hyper": HYPER}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, ms, cores, sample, P = cpu_arm(args, args.steps, args.warmup, world=args.gpus)
    from oxidizr_b200 import inventory
    cfg = workload_config(args, P, len(inventory.PARAM_SETS[args.workload]()), args.gpus, args.sync if args.gpus > 1 else "single")
    cfg["note"] = "CPU restatement of the reference's unfused per-tensor path over the whole parameter set"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "product_library_mapped": product_library_mapped(),
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ checks of the GPU arm's result
class Checker:
    """The untimed leg after the timed steps: is what the ranks hold right? Uses torch.distributed only to move the
    evidence between the bench's own processes; the step under test is the library's."""

    def __init__(self, torch, dist, ox, opt, cfg, tensors, numel, no_decay, present, gone, views, world, rank, local_rank, code, scale):
        self.torch, self.dist, self.ox, self.opt, self.cfg = torch, dist, ox, opt, cfg
        self.tensors, self.numel, self.no_decay, self.present, self.gone = tensors, numel, no_decay, present, gone
        self.v, self.world, self.rank, self.dev, self.code, self.scale = views, world, rank, local_rank, code, scale
        self.problems: list[str] = []
        # The NCCL mode's reduce-scatter sums in the gradients' own 16-bit type and rounds the sum to it: that mode (a
        # baseline for comparison, not the product) is checked to a tolerance, every other mode bit for bit.
        self.exact = True

    # -- evidence helpers
    def checksum(self, t) -> tuple[int, int]:
        """Two 64-bit sums over a device array's 32-bit words: plain, and weighted by position (period 2^20)."""
        torch = self.torch
        w = t.view(torch.int32) if t.element_size() == 4 else t.view(torch.int16)
        n = w.numel()
        period = 1 << 20
        weights = (torch.arange(period, device=w.device, dtype=torch.int64) % 65521) + 1
        s1 = s2 = 0
        chunk = 1 << 26
        for lo in range(0, n, chunk):
            c = w[lo:min(n, lo + chunk)].to(torch.int64)
            s1 += int(c.sum().item())
            full = (c.numel() // period) * period
            if full:
                s2 += int((c[:full].view(-1, period) * weights).sum().item())
            if full < c.numel():
                s2 += int((c[full:] * weights[:c.numel() - full]).sum().item())
        mask = (1 << 64) - 1
        return s1 & mask, s2 & mask

    def state_checksums(self) -> list[tuple[int, int]]:
        return [self.checksum(self.v[k]) for k in ("master", "exp_avg", "exp_avg_sq", "work")]

    def all_equal_over_ranks(self, value) -> bool:
        if self.dist is None:
            return True
        got = [None] * self.world
        self.dist.all_gather_object(got, value)
        return all(g == got[0] for g in got)

    def agree(self, ok: bool) -> bool:
        """True only if every rank says so."""
        if self.dist is None:
            return ok
        t = self.torch.tensor([1 if ok else 0], device="cuda", dtype=self.torch.int32)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return bool(t.item())

    def rank_grads(self, i: int) -> list[np.ndarray]:
        """Tensor i's gradient on every rank, as bit patterns, in rank order."""
        torch = self.torch
        off, n = self.opt.offsets[i], self.numel[i]
        mine = self.v["grads"][off:off + n].contiguous()
        if self.dist is None:
            parts = [mine]
        else:
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            self.dist.all_gather(parts, mine)
        bits = torch.int32 if mine.element_size() == 4 else torch.int16
        out = [p.view(bits).cpu().numpy() for p in parts]
        return [a.view(np.float32) if a.dtype == np.int32 else a.view(np.uint16) for a in out]

    def norm_float64(self) -> float:
        """sqrt of the sum over every present tensor of (sum over ranks of the unscaled gradient)^2, in float64."""
        torch = self.torch
        inv = np.float32(1.0 / self.scale) if self.scale else np.float32(1.0)
        acc = torch.zeros((), device="cuda", dtype=torch.float64)
        for i, n in enumerate(self.numel):
            if n == 0 or (self.present is not None and not self.present[i]):
                continue
            off = self.opt.offsets[i]
            s = self.v["grads"][off:off + n].to(torch.float32)
            if self.dist is not None:
                self.dist.all_reduce(s)
            acc += ((s * float(inv)).to(torch.float64) ** 2).sum()
        return math.sqrt(float(acc.item()))

    def sample_tensors(self) -> list[int]:
        """The smallest tensor, a matrix in the middle, the largest (the embedding: it crosses shard and bucket
        boundaries), one that straddles a bucket boundary, and, with absent tensors, one of those."""
        opt, numel = self.opt, self.numel
        live = [i for i, n in enumerate(numel) if n > 0]
        picks = [min(live, key=lambda i: numel[i]), max(live, key=lambda i: numel[i])]
        mats = [i for i in live if len(self.tensors[i].shape) == 2 and i not in picks]
        if mats:
            picks.append(mats[len(mats) // 2])
        be = opt.info.bucket_elems
        for i in live:
            if i not in picks and opt.offsets[i] // be != (opt.offsets[i] + numel[i] - 1) // be:
                picks.append(i)
                break
        if self.gone:  # a tensor no rank routed to: untouched when flagged absent, decayed on zero gradients
            picks.append(self.gone[len(self.gone) // 2])
        return picks

    # -- the checks
    def one_step_against_the_checker(self) -> dict:
        """Snapshot sampled tensors, run ONE more step, and compare what each rank owns of them bit for bit with the
        CPU checker's AdamW fed the f32 rank-order sum of the ranks' gradients and the coefficient the step reported."""
        from oracle import dpstep as orc
        ox, opt, ffi = self.ox, self.opt, self.ox.ffi
        picks = self.sample_tensors()
        kinds = (("master", ffi.STATE_MASTER), ("exp_avg", ffi.STATE_EXP_AVG), ("exp_avg_sq", ffi.STATE_EXP_AVG_SQ))
        before = {i: {k: opt.export_tensor(kind, i, np.full(self.numel[i], np.nan, np.float32)) for k, kind in kinds} for i in picks}
        grads = {i: self.rank_grads(i) for i in picks}
        t0 = opt.timestep
        want_norm = self.norm_float64()
        res = opt.step(self.cfg, self.present)
        out = {"norm": res.grad_norm, "norm_float64": want_norm, "norm_rel_err": abs(res.grad_norm - want_norm) / want_norm,
               "applied": res.applied, "sampled": []}
        if not (out["norm_rel_err"] <= 1e-5):
            self.problems.append(f"norm {res.grad_norm} differs from the float64 sum {want_norm} by {out['norm_rel_err']:.3e} relative")
        if not self.all_equal_over_ranks((res.grad_norm, res.clip_coef, res.applied, res.timestep)):
            self.problems.append("the ranks report different norms, coefficients or decisions for one step")
        if not res.applied:
            self.problems.append("the check step was not applied")
            return out
        c = np.float32(res.clip_coef)  # no target clip here: the product of the coefficients is the first one
        inv = np.float32(1.0 / self.scale) if self.scale else np.float32(1.0)
        for i in picks:
            after = {k: opt.export_tensor(kind, i, np.full(self.numel[i], np.nan, np.float32)) for k, kind in kinds}
            own = ~np.isnan(before[i]["master"])
            entry = {"tensor": self.tensors[i].name, "elements": self.numel[i], "owned_by_this_rank": int(own.sum())}
            if self.present is not None and not self.present[i]:
                same = all(np.array_equal(before[i][k][own].view(np.uint32), after[k][own].view(np.uint32)) for k, _ in kinds)
                entry["untouched"] = bool(same)
                if not same:
                    self.problems.append(f"{self.tensors[i].name} has no gradient on any rank but its state changed")
            else:
                g = orc.sum_ranks([np.ascontiguousarray(x) for x in grads[i]], self.code)[own]
                g = ((g * inv) * c) * np.float32(1.0)
                p, m, v = (np.ascontiguousarray(before[i][k][own]) for k, _ in kinds)
                wd = 0.0 if self.no_decay[i] else self.cfg.weight_decay
                s = orc.adam_prepare(self.cfg.lr, 1.0, self.cfg.beta1, self.cfg.beta2, self.cfg.eps, wd, t0 + 1)
                orc.adamw(p, m, v, np.ascontiguousarray(g.astype(np.float32)), s)
                if self.exact:
                    eq = {k: bool(np.array_equal(x.view(np.uint32), after[k][own].view(np.uint32))) for (k, _), x in zip(kinds, (p, m, v))}
                    if self.code != orc.F32:
                        w = opt.export_tensor(ffi.STATE_WORK, i)
                        eq["work"] = bool(np.array_equal(orc.narrow(p, self.code), w[own]))
                    entry["bit_equal"] = eq
                else:
                    def close(x, y):
                        x64, y64 = x.astype(np.float64), y.astype(np.float64)
                        return bool(x.size == 0 or np.all(np.abs(x64 - y64) <= 2e-2 * (np.abs(x64) + np.sqrt(np.mean(x64 ** 2)))))
                    eq = {k: close(x, after[k][own]) for (k, _), x in zip(kinds, (p, m, v))}
                    entry["within_2e-2_of_the_f32_sum"] = eq
                if not all(eq.values()):
                    bad = np.flatnonzero(p.view(np.uint32) != after["master"][own].view(np.uint32))
                    where = {"differing_master_elements": int(bad.size)}
                    if bad.size:
                        k = int(bad[0])
                        where.update(first=k, last=int(bad[-1]), want=float(p[k]), got=float(after["master"][own][k]))
                    entry["mismatch"] = where
                    self.problems.append(f"{self.tensors[i].name}: not bit-equal to the checker: {eq} {where}")
            out["sampled"].append(entry)
        return out

    def weights_equal_on_every_rank(self) -> bool:
        same = self.all_equal_over_ranks(self.checksum(self.v["work"]))
        if not same:
            self.problems.append("the ranks hold different working weights after the step")
        return same

    def overflow_scenario(self, steps: int = 60, interval: int = 8) -> dict:
        """f16 gradients under a loss scale: a seeded 1-in-50 of the steps (and step 3) has an inf written into a random
        rank's gradient buffer at a random element. That step must be skipped on every rank with every state byte
        unchanged, the scale must halve and the clean-step count restart; after `interval` clean steps it doubles."""
        torch, ox, opt = self.torch, self.ox, self.opt
        rng = np.random.default_rng(SEED + 5)
        hits = sorted({3} | {s for s in range(steps) if rng.random() < 1.0 / 50.0})
        scaler = ox.LossScaler(ox.LossScaleConfig(initial=self.scale, growth_factor=2.0, backoff_factor=0.5, growth_interval=interval))
        inf16 = torch.tensor([float("inf")], dtype=self.v["grads"].dtype, device="cuda")
        log = {"steps": steps, "injected_at": hits, "growth_interval": interval, "skipped": 0, "grown": 0}
        live = [i for i, n in enumerate(self.numel) if n > 0 and (self.present is None or self.present[i])]
        for s in range(steps):
            cfg = self.ox.StepConfig(**{**HYPER, "loss_scale": scaler.scale()})
            hit = s in hits
            if hit:
                who, i = int(rng.integers(self.world)), live[int(rng.integers(len(live)))]
                at = self.opt.offsets[i] + int(rng.integers(self.numel[i]))
                sums = self.state_checksums()
                t_before = opt.timestep
                if who == self.rank:
                    keep = self.v["grads"][at:at + 1].clone()
                    self.v["grads"][at:at + 1] = inf16
                torch.cuda.synchronize()
            before_scale = scaler.scale()
            res = opt.step(cfg, self.present)
            scaler.record_step(bool(res.overflow))
            if hit:
                ok = (res.overflow == 1 and res.applied == 0 and opt.timestep == t_before and not math.isfinite(res.grad_norm)
                      and self.state_checksums() == sums and scaler.scale() == before_scale * 0.5
                      and scaler.state().consecutive_ok == 0)
                if not self.agree(ok):
                    self.problems.append(f"overflow step {s}: not skipped cleanly on every rank")
                log["skipped"] += 1
                if who == self.rank:
                    self.v["grads"][at:at + 1] = keep
                torch.cuda.synchronize()
            else:
                if not self.agree(res.overflow == 0 and res.applied == 1):
                    self.problems.append(f"clean step {s} was not applied on every rank")
                if scaler.scale() == before_scale * 2.0:
                    log["grown"] += 1
        log["final_scale"] = scaler.scale()
        if log["grown"] == 0:
            self.problems.append("the loss scale never grew although clean runs reached the growth interval")
        return log


# ------------------------------------------------------------------ the GPU arm
def run_gpu(args):
    import torch
    import oxidizr_b200 as ox
    from oxidizr_b200 import inventory
    from oxidizr_b200.interop import state_views

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the optimizer step has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    dist = None
    comm = None
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # keep stdout for the one JSON line
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        uid = [ox.Communicator.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        comm = ox.Communicator.init_rank(local_rank, rank, world, uid[0])

    tensors = inventory.PARAM_SETS[args.workload]()
    plan = ox.DecayPlan(ox.WeightDecaySpec("skip_1d"), tensors)
    numel = [t.elements for t in tensors]
    T, P = len(numel), sum(numel)
    mode = {"p2p": ox.SYNC_P2P, "nccl": ox.SYNC_NCCL, "copy": ox.SYNC_COPY, "replicated": ox.SYNC_REPLICATED}[args.sync] if world > 1 else ox.SYNC_SINGLE
    es = 4 if args.dtype == "f32" else 2  # bytes per gradient and per working weight
    ox_dt = {"bf16": ox.BF16, "f16": ox.F16, "f32": ox.F32}[args.dtype]
    t_dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[args.dtype]
    bytes_norm = es  # the norm pass reads every gradient once; the update moves 28 B/param in either width
    scale = float(args.loss_scale) if args.loss_scale else 0.0
    opt = ox.DpOptimizer(numel, plan.no_decay, ox_dt, ox_dt, world=world, rank=rank, sync_mode=mode,
                         device=local_rank, comm=comm)
    info = opt.info
    stream = torch.cuda.Stream()
    opt.set_stream(stream.cuda_stream)
    opt.set_profile(True)
    v = state_views(opt)
    separate_work = opt.pointers()["work"] != opt.pointers()["master"]  # f32 parameters at one rank keep no narrow copy

    # tensors no rank has a gradient for (mixture-of-experts sets): all-zero gradients, or flagged absent
    gone = absent_tensors(tensors) if args.absent != "none" else []
    present = None
    if args.absent == "skip" and gone:
        present = [i not in set(gone) for i in range(T)]

    # seeded synthetic state, generated on the device straight into the library's buffers
    gen = torch.Generator(device="cuda")
    gen.manual_seed(SEED)
    chunk = 1 << 26
    for lo in range(0, info.local_elems, chunk):
        hi = min(info.local_elems, lo + chunk)
        v["master"][lo:hi].normal_(0.0, 0.02, generator=gen)
        v["exp_avg"][lo:hi].normal_(0.0, 1e-4, generator=gen)
        v["exp_avg_sq"][lo:hi].normal_(0.0, 1e-6, generator=gen).abs_()
    gen.manual_seed(SEED + 1 + rank)
    gstd = 1e-3 * (scale if scale else 1.0)
    gone_set = set(gone)
    for i, (off, n) in enumerate(zip(opt.offsets, numel)):
        if i in gone_set:
            # flagged absent: the span may hold anything, so it holds something; all-zero gradients otherwise
            v["grads"][off:off + n] = 7.0 if args.absent == "skip" else 0.0
        else:
            v["grads"][off:off + n] = torch.empty(n, device="cuda", dtype=torch.float32).normal_(0.0, gstd, generator=gen).to(t_dt)
    if separate_work and (world == 1 or mode == ox.SYNC_REPLICATED):
        v["work"].copy_(v["master"].to(t_dt))
    opt.timestep = 1
    torch.cuda.synchronize()

    cfg = ox.StepConfig(**HYPER, loss_scale=scale if scale else float("nan"))

    def barrier():
        torch.cuda.synchronize()
        if comm is not None:
            comm.barrier()

    def max_over_ranks(sec: float) -> float:
        if dist is None:
            return sec
        t = torch.tensor([sec], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(n_steps: int, before_step=None):
        """n_steps steps bracketed by barrier + synchronize; device time by CUDA events; returns seconds."""
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        profs = []
        with torch.cuda.stream(stream):
            t0.record(stream)
            for _ in range(n_steps):
                if before_step is not None:
                    before_step()
                res = opt.step(cfg, present)
                profs.append(opt.profile())
            t1.record(stream)
        barrier()
        return max_over_ranks(t0.elapsed_time(t1) / 1e3), profs, res

    for _ in range(max(args.warmup, 3)):
        opt.step(cfg, present)
    sampler = ClockSampler(local_rank)
    sampler.start()
    sec, profs, res = timed(args.steps)
    clocks = sampler.stop()
    ms_per_step = sec * 1e3 / args.steps
    value = P * args.steps / sec
    exchange = {0: "none", 1: "communicator collectives", 2: "peer-memory mailboxes"}[opt.exchange_kind()]
    pull_kernel = {0: None, 1: "k_pull_sumsq", 2: "k_pull_bulk"}[opt.last_pull_kernel()]
    update_kernel = {0: None, 1: "k_adamw", 2: "k_adamw_wide", 3: "k_adamw_staged"}[opt.last_update_kernel()]

    # ---- the check leg (untimed): before anything else touches the gradient buffer
    check = None
    if not args.skip_check:
        ck = Checker(torch, dist, ox, opt, cfg, tensors, numel, plan.no_decay, present, gone, v, world, rank, local_rank, ox_dt, scale)
        ck.exact = mode != ox.SYNC_NCCL
        check = {"step": ck.one_step_against_the_checker()}
        check["exact"] = ck.exact
        check["work_equal_on_every_rank"] = ck.weights_equal_on_every_rank()
        if args.inject_inf:
            check["overflow_scenario"] = ck.overflow_scenario()
        if gone:
            check["absent"] = {"mode": args.absent, "tensors": len(gone), "elements": int(sum(numel[i] for i in gone)),
                               "share_of_params": sum(numel[i] for i in gone) / P}
        check["problems"] = ck.problems
        check["ok"] = ck.agree(not ck.problems)

    # ---- end to end: every step copies that step's gradients from pinned host memory, then reads the result back
    host_off, base = [], 0
    if not args.skip_e2e:
        host = torch.empty(P, dtype=t_dt).pin_memory()
        pos = 0
        for off, n in zip(opt.offsets, numel):
            host[pos:pos + n].copy_(v["grads"][off:off + n])
            host_off.append(pos)
            pos += n
        torch.cuda.synchronize()
        base = host.data_ptr()

    def upload():
        for i, n in enumerate(numel):
            opt.upload_grads(i, base + host_off[i] * es)

    def upload_next():
        for i, n in enumerate(numel):
            opt.upload_next_grads(i, base + host_off[i] * es)

    def timed_host_fed(n_steps: int):
        """Every step's gradients come from pinned host memory and its result is read back. The library's second
        gradient buffer lets the copy of step i+1 run while step i still computes; each copy is inside the timed region."""
        barrier()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            t0.record(stream)
            upload_next()
            for i in range(n_steps):
                opt.swap_grads()
                opt.step_async(cfg, present)
                if i + 1 < n_steps:
                    upload_next()
                opt.step_wait()
            t1.record(stream)
        barrier()
        return max_over_ranks(t0.elapsed_time(t1) / 1e3)

    e2e_steps = max(2, min(args.steps, 5))
    pipelined = mode in (ox.SYNC_SINGLE, ox.SYNC_P2P, ox.SYNC_REPLICATED, ox.SYNC_NCCL)
    if pipelined and not args.skip_e2e:
        # every rank must take the same leg: if the second buffer cannot be set up on some rank, all fall back
        ok = 1
        try:
            opt.double_buffer_grads()
        except ox.OxzError as e:
            print(f"rank {rank}: no second gradient buffer ({e}); the host-fed leg copies, then steps", file=sys.stderr)
            ok = 0
        if dist is not None:
            t = torch.tensor([ok], device="cuda", dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            ok = int(t.item())
        pipelined = bool(ok)
    if args.skip_e2e:
        e2e_sec, e2e_value = float("nan"), None
    elif pipelined:
        timed_host_fed(2)
        e2e_sec = timed_host_fed(e2e_steps)
        e2e_value = P * e2e_steps / e2e_sec
    else:
        timed(1, upload)
        e2e_sec, _, _ = timed(e2e_steps, upload)
        e2e_value = P * e2e_steps / e2e_sec

    # Overlap with backward: three quarters of the buckets are handed in while "backward" would still be running
    # (untimed here); the timed part is what is left exposed after backward ends. A separate figure, not `value`.
    overlap = None
    if mode in (ox.SYNC_SINGLE, ox.SYNC_P2P) and not args.skip_e2e:
        nb = info.n_buckets
        early = max(1, (3 * nb) // 4)
        exposed = []
        for _ in range(5):
            opt.grads_ready(cfg, nb - early, early, present, producer_stream=stream.cuda_stream)
            sec1, _, _ = timed(1)
            exposed.append(sec1 * 1e3)
        overlap = {"buckets": nb, "buckets_reduced_during_backward": early, "exposed_ms_per_step": statistics.median(exposed)}

    aux = None
    if world == 1 and not args.skip_aux:
        aux = aux_measurements(ox, torch, opt, numel, stream, local_rank, t_dt, es)

    peak, peak_kind = measured_peaks()
    totals = sorted(p.total_ms for p in profs)
    pct = lambda q: totals[min(len(totals) - 1, int(q * len(totals)))]  # noqa: E731
    upd = statistics.mean(p.update_ms for p in profs)
    nrm = statistics.mean(p.norm_ms for p in profs)
    replicated = mode == ox.SYNC_REPLICATED
    live = P - (sum(numel[i] for i in gone) if present is not None else 0)  # parameters the kernels touch
    local_params = live if replicated else live / world  # ... of which one rank's update kernel covers these
    roof = kernel_rooflines(live, world, replicated, es, nrm, upd, peak, pull_kernel, update_kernel, mode == ox.SYNC_SINGLE, args.dtype)
    roof["peak_kind"] = peak_kind
    sync_name = args.sync if world > 1 else "single"
    config = workload_config(args, P, T, world, sync_name)
    config["exchange"] = exchange
    config["l2"] = "inputs larger than L2: %d B/param x %d params per rank per step" % (bytes_norm + BYTES_UPDATE, int(local_params))
    # kernels of this library per step: norm (or pull), the decision (one fused kernel with the mailboxes, else two), the
    # update, and with the mailboxes the two gate kernels; the copy mode runs pull and update once per pipeline group
    per_step = {"none": 4, "communicator collectives": 4, "peer-memory mailboxes": 5}[exchange]
    if mode == ox.SYNC_COPY:
        per_step = 10
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": config,
        "roofline": roof,
        "phases_ms": {k: statistics.mean(getattr(p, k) for p in profs) for k in
                      ("collect_ms", "norm_ms", "decide_ms", "update_ms", "publish_ms", "total_ms")},
        # device time of each timed step on this rank (CUDA events inside the library), for the spread
        "step_ms_device": {"median": statistics.median(totals), "p10": pct(0.10), "p90": pct(0.90)},
        "step_roofline": step_roofline(live, world, ms_per_step, peak, es),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": P * es * world, "d2h_bytes_per_step": 32 * world,
                "ms_per_step": e2e_sec * 1e3 / e2e_steps, "steps": e2e_steps,
                "copy_overlaps_previous_step": bool(pipelined and not args.skip_e2e)},
        "gpu_launches": per_step * args.steps * world,
        "launch_geometry": opt.launch_geometry(),
        "overlap_with_backward": overlap,
        "aux": aux,
        "clocks": clocks,
        "result": {"grad_norm": res.grad_norm, "applied": res.applied, "timestep": res.timestep},
        "check": check,
    }
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            cv, ms, cores, sample, _ = cpu_arm(args, 3, 1)
            cv1, _, _, _, _ = cpu_arm(args, 1, 0, threads=1)
            line["cpu_baseline"] = {"value": cv, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                    "single_thread_value": cv1}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    opt.destroy()
    if comm is not None:
        comm.barrier()
        comm.destroy()
    if dist is not None:
        dist.destroy_process_group()
    if check is not None and not check["ok"]:
        print(f"rank {rank}: the result check failed: {check['problems']}", file=sys.stderr)
        sys.exit(1)


def kernel_rooflines(live: float, world: int, replicated: bool, es: int, norm_ms: float, update_ms: float, hbm_peak: float,
                     pull_kernel, update_kernel, single: bool, dtype: str) -> dict:
    """The roofline of the two kernels that carry the step, each against the resource that binds it.

    One rank: both are HBM streams (norm es B/param, update 28 B/param). More ranks (sharded): the norm kernel is the
    fused reduce-scatter - it pulls (W-1)/W * es B/param over NVLink - and the update kernel is the fused all-gather -
    it pushes (W-1)/W * es B/param - while their HBM traffic shrinks with 1/W. For each kernel both fractions are
    given and the larger names the bound; the line's own fields describe the kernel that takes longer."""
    W = world
    own = live if replicated else live / W
    norm_name = ("k_sumsq_stream16" if es == 2 else "k_sumsq") if single else pull_kernel
    kernels = []
    # HBM bytes one launch moves on its own GPU (algorithmic for one rank; with peers the bytes served to them count)
    if W == 1:
        norm_hbm, upd_hbm, wire_in, wire_out = es * own, BYTES_UPDATE * own, 0.0, 0.0
    elif replicated:
        norm_hbm, upd_hbm = es * live * W + 4 * live, (4 + 24 + es) * live  # reads every rank's copy once each, writes the f32 sum
        wire_in, wire_out = (W - 1) * es * live, 0.0
    else:
        norm_hbm = es * own + (W - 1) * es * own + 4 * own   # own tiles, tiles served to the peers, the f32 sum out
        upd_hbm = (4 + 24 + es) * own + (W - 1) * es * own   # f32 sum in, state, own weights out, the peers' weights landing
        wire_in = wire_out = (W - 1) * es * own
    for name, ms, hbm, wire, what in ((norm_name, norm_ms, norm_hbm, wire_in, "pull (reduce-scatter) + unscale + norm"),
                                      (update_kernel, update_ms, upd_hbm, wire_out, "AdamW + push (all-gather)")):
        hbm_gbs = hbm / (ms * 1e-3) / 1e9
        wire_gbs = wire / (ms * 1e-3) / 1e9
        f_hbm, f_wire = hbm_gbs / hbm_peak, wire_gbs / NVLINK_MEASURED_GBS
        bound = "nvlink" if f_wire > f_hbm else "hbm"
        kernels.append({"kernel": name, "work": what, "kernel_ms": ms, "bound": bound,
                        "hbm_bytes_per_launch": hbm, "hbm_gbs": hbm_gbs, "hbm_frac_of_measured_peak": f_hbm,
                        "nvlink_bytes_per_launch_per_direction": wire, "nvlink_gbs": wire_gbs,
                        "nvlink_frac_of_measured": f_wire, "nvlink_frac_of_nominal": wire_gbs / NVLINK_NOMINAL_GBS})
    top = max(kernels, key=lambda k: k["kernel_ms"])
    if top["bound"] == "hbm":
        is_update = top["work"].startswith("AdamW")
        algorithmic = BYTES_UPDATE * own if is_update else es * own
        out = {"bound": "hbm", "kernel": top["kernel"], "achieved": top["hbm_gbs"], "peak": hbm_peak, "unit": "GB/s",
               "frac": top["hbm_frac_of_measured_peak"],
               "traffic": None, "traffic_source": "not captured",
               "algorithmic_bytes_per_launch": algorithmic if W == 1 else top["hbm_bytes_per_launch"], "kernel_ms": top["kernel_ms"]}
        if dtype == "bf16" and is_update and W == 1:
            out["traffic"] = ADAMW_TRAFFIC_RATIO * top["hbm_bytes_per_launch"]
            out["traffic_source"] = "ncu capture of nano_dense (one rank) scaled by bytes per launch"
        elif dtype == "bf16" and is_update and not replicated:
            # the kernel's own 30 B per owned parameter by the two-GPU capture, plus the peers' weights landing here
            out["traffic"] = ADAMW_PEER_TRAFFIC_RATIO * (4 + 24 + es) * own + (W - 1) * es * own
            out["traffic_source"] = ("ncu capture of the update kernel on two GPUs (50 M owned parameters) scaled by bytes per "
                                     "launch, plus the algorithmic bytes of the peers' weights landing in this GPU's memory")
    else:
        out = {"bound": "nvlink", "kernel": top["kernel"], "achieved": top["nvlink_gbs"], "peak": NVLINK_MEASURED_GBS,
               "peak_source": NVLINK_MEASURED_SOURCE, "peak_nominal": NVLINK_NOMINAL_GBS, "unit": "GB/s",
               "frac": top["nvlink_frac_of_measured"], "frac_of_nominal": top["nvlink_frac_of_nominal"],
               "traffic": None, "traffic_source": "wire bytes are algorithmic: (W-1)/W x bytes per value x parameters, per direction",
               "algorithmic_bytes_per_launch": top["nvlink_bytes_per_launch_per_direction"], "kernel_ms": top["kernel_ms"]}
    out["kernels"] = kernels
    return out


def aux_measurements(ox, torch, opt, numel, stream, local_rank: int, t_dt, es: int) -> dict:
    """The callers either side of the step, timed apart from `value`: per-tensor gradients into the flat buffer
    (overwrite and accumulate), and the rank-sliced loader with and without its masks."""
    import tempfile
    P = sum(numel)
    pos, offs = 0, []
    for n in numel:
        offs.append(pos)
        pos += (n + 7) // 8 * 8  # 16-byte aligned starts
    src = torch.empty(pos, dtype=t_dt, device="cuda").normal_(0.0, 1e-3)
    ptrs = [src.data_ptr() + o * es for o in offs]
    out = {"flatten": {}}
    for name, acc, bytes_per in (("overwrite", False, 2 * es), ("accumulate", True, 3 * es)):
        opt.flatten_grads(ptrs, acc)
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        with torch.cuda.stream(stream):
            t0.record(stream)
            for _ in range(reps):
                opt.flatten_grads(ptrs, acc)
            t1.record(stream)
        torch.cuda.synchronize()
        ms = t0.elapsed_time(t1) / reps
        out["flatten"][name] = {"ms": ms, "gbs": bytes_per * P / (ms * 1e-3) / 1e9, "bytes_per_param": bytes_per}
    del src
    batch, seq, rows = 8, 2048, 2048
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tokens.bin")
        rng = np.random.default_rng(SEED)
        toks = rng.integers(1, 32000, size=rows * (seq + 1), dtype=np.uint32)
        toks[rng.integers(0, toks.size, size=toks.size // 400)] = 0  # document separators
        toks.tofile(path)
        out["loader"] = {"batch": batch, "seq_len": seq}
        for name, masked in (("plain", False), ("masked", True)):
            l = ox.LitDataLoader(path, batch, seq, device=local_rank)
            if masked:
                l.with_target_mask(16000, [2]).with_document_mask(0)
            for _ in range(5):
                l.next_batch(stream.cuda_stream)
            torch.cuda.synchronize()
            n = 200
            t = time.perf_counter()
            for _ in range(n):
                l.next_batch(stream.cuda_stream)
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t) / n
            out["loader"][name] = {"us_per_batch": dt * 1e6, "tokens_per_s": batch * seq / dt}
            l.close()
    return out


def step_roofline(P: float, world: int, ms: float, hbm_gbs: float, es: int = 2) -> dict:
    """Whole-step roofline: the slower of the HBM term (es + 28 B/param on each rank's 1/world: 30 for 16-bit, 32 for
    f32) and, with more ranks, the NVLink term (reduce-scatter in + all-gather out in the gradients' and weights' own
    width, (world-1)/world * es B/param each)."""
    hbm_ms_nominal = (es + BYTES_UPDATE) * P / world / 8.0e12 * 1e3
    hbm_ms_measured = (es + BYTES_UPDATE) * P / world / (hbm_gbs * 1e9) * 1e3
    wire = 2 * (world - 1) / world * es * P
    wire_ms_nominal = wire / (NVLINK_NOMINAL_GBS * 1e9) * 1e3
    wire_ms_measured = wire / (NVLINK_MEASURED_GBS * 1e9) * 1e3
    nominal = max(hbm_ms_nominal, wire_ms_nominal)
    measured = max(hbm_ms_measured, wire_ms_measured)
    return {"roofline_ms_nominal": nominal, "frac_of_nominal": nominal / ms, "roofline_ms_measured_peaks": measured,
            "frac_of_measured_peaks": measured / ms, "bound": "nvlink" if wire_ms_nominal > hbm_ms_nominal else "hbm"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--sync", choices=["p2p", "copy", "nccl", "replicated"], default="p2p", help="how ranks meet at --gpus > 1")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: leave the host-fed and overlap legs out")
    ap.add_argument("--skip-aux", action="store_true", help="leave out the flatten and loader timings (1 GPU only)")
    ap.add_argument("--skip-check", action="store_true", help="profiling runs: leave the untimed result check out")
    ap.add_argument("--dtype", choices=["bf16", "f16", "f32"], default="bf16",
                    help="width of gradients and working weights: bf16 is the headline; f16 goes with --loss-scale")
    ap.add_argument("--loss-scale", type=float, default=0.0, help="gradients arrive multiplied by this scale (f16 runs); 0 = no scaler")
    ap.add_argument("--inject-inf", action="store_true",
                    help="check leg: a seeded 1-in-50 of 60 more steps has an inf in one rank's gradients; needs --loss-scale")
    ap.add_argument("--absent", choices=["none", "zero", "skip"], default="none",
                    help="mixture-of-experts sets: 2 of 8 routed experts per layer have all-zero gradients (zero) or none at all (skip)")
    ap.add_argument("--workload", default=WORKLOAD, help="parameter set; the headline is llama-3.2-1b, smaller sets serve profiler captures")
    args = ap.parse_args()
    if args.inject_inf and not args.loss_scale:
        ap.error("--inject-inf goes with --loss-scale (the overflow signal of a scaled f16 run)")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
