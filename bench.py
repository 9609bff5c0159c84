#!/usr/bin/env python
"""Benchmark of the data-parallel optimizer step (gradient sync + unscale/inf check + global-norm clip + fused AdamW
+ weight write-back) on the Llama-3.2-1B parameter set.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the CPU restatement of the reference's path on the host cores

One JSON line on stdout (rank 0). A step is one pass of the whole path over one set of synthetic gradients:
bf16 gradients ~N(0,1e-3) from seed+rank, f32 master ~N(0,0.02), m ~N(0,1e-4), v = |N(0,1e-6)|.
`value` is params/s with the gradients already resident in HBM; `e2e` is the same call fed from pinned host memory.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
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
# Algorithmic HBM bytes per parameter: the norm pass reads the bf16 gradient (2); the update reads gradient 2 +
# master 4 + m 4 + v 4 and writes master 4 + m 4 + v 4 + bf16 weight 2 (28).
BYTES_NORM, BYTES_UPDATE = 2, 28
# DRAM bytes over algorithmic bytes of k_adamw from one ncu capture of a smaller case of the same kernel
# (nano_dense, 134 M parameters): 3.7015 GB read+write for 3.7573 GB algorithmic.
ADAMW_TRAFFIC_RATIO = 3.7015 / 3.7573


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


# ------------------------------------------------------------------ the CPU arm
def cpu_arm(steps: int, warmup: int, threads: int | None = None, world: int = 1):
    """The reference's CPU optimizer path, restated (the reference is Rust over un-vendored crates and cannot be
    built here), on a bounded sample of the workload: the first 4 of 16 decoder layers. With world > 1 the step first
    sums that many gradient buffers in f32, as the reference's in-process communicator does (src/dp/reduce.rs:30-60)."""
    from oracle import dpstep as orc
    from oxidizr_b200 import DecayPlan, WeightDecaySpec, inventory

    tensors = inventory.llama_3_2_1b()
    plan = DecayPlan(WeightDecaySpec("skip_1d"), tensors)
    pick = list(range(1, 1 + 9 * 4))  # 4 layers x (2 norms + 4 attention + 3 MLP tensors); the embedding is skipped
    numel = [tensors[i].elements for i in pick]
    P = sum(numel)
    all_threads = orc.lib().orc_num_threads()
    if threads:
        orc.lib().orc_set_num_threads(threads)
    cores = orc.lib().orc_num_threads()
    master = [tiled_normal(n, 0.02, SEED + i) for i, n in enumerate(numel)]
    state = orc.StepState(master, [tiled_normal(n, 1e-4, SEED + 100 + i) for i, n in enumerate(numel)],
                          [tiled_normal(n, 1e-6, SEED + 200 + i, True) for i, n in enumerate(numel)],
                          [orc.to_bf16(p) for p in master], orc.BF16, lr_scale=[1.0] * len(numel),
                          group_wd=[0.0 if plan.no_decay[i] else float("nan") for i in pick], timestep=1)
    grads = [orc.to_bf16(tiled_normal(n, 1e-3, SEED + 300 + i)) for i, n in enumerate(numel)]
    cfg = orc.StepConfig(**HYPER)
    ranks = [grads] * max(world, 1)  # every rank's buffer holds the same values: only the work of the sum matters here
    for _ in range(warmup):
        orc.step(state, ranks, orc.BF16, cfg)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.step(state, ranks, orc.BF16, cfg)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    orc.lib().orc_set_num_threads(all_threads)
    sample = f"{len(pick)} tensors = 4 of 16 decoder layers, {P} of 1235814400 params, {steps} steps, {max(world, 1)} rank buffer(s) summed"
    return P / dt, dt * 1e3, cores, sample


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, ms, cores, sample = cpu_arm(args.steps, args.warmup, world=args.gpus)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "params": 1235814400, "grad_dtype": "bf16", "param_dtype": "bf16",
                   "world": args.gpus, "note": "CPU restatement of the reference's unfused per-tensor path; "
                                               "ms_per_step is for the sample, value is sample params / time"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ the GPU arm
def run_gpu(args):
    import torch
    import oxidizr_b200 as ox
    from oxidizr_b200 import inventory
    from oxidizr_b200.interop import device_view

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
    P = sum(numel)
    mode = {"p2p": ox.SYNC_P2P, "nccl": ox.SYNC_NCCL, "copy": ox.SYNC_COPY, "replicated": ox.SYNC_REPLICATED}[args.sync] if world > 1 else ox.SYNC_SINGLE
    es = 4 if args.dtype == "f32" else 2  # bytes per gradient and per working weight
    ox_dt = ox.F32 if args.dtype == "f32" else ox.BF16
    t_dt = torch.float32 if args.dtype == "f32" else torch.bfloat16
    bytes_norm = es  # the norm pass reads every gradient once; the update moves 28 B/param in either dtype
    opt = ox.DpOptimizer(numel, plan.no_decay, ox_dt, ox_dt, world=world, rank=rank, sync_mode=mode,
                         device=local_rank, comm=comm)
    ptr, info = opt.pointers(), opt.info
    stream = torch.cuda.Stream()
    opt.set_stream(stream.cuda_stream)
    opt.set_profile(True)

    # seeded synthetic state, generated on the device straight into the library's buffers
    gen = torch.Generator(device="cuda")
    grads = device_view(ptr["grads"], info.padded_total * es, t_dt, local_rank)
    separate_work = ptr["work"] != ptr["master"]  # f32 parameters at one rank keep no narrow copy
    work = device_view(ptr["work"], info.padded_total * es, t_dt, local_rank) if separate_work else None
    master = device_view(ptr["master"], info.local_elems * 4, torch.float32, local_rank)
    m = device_view(ptr["exp_avg"], info.local_elems * 4, torch.float32, local_rank)
    v = device_view(ptr["exp_avg_sq"], info.local_elems * 4, torch.float32, local_rank)
    gen.manual_seed(SEED)
    chunk = 1 << 26
    for lo in range(0, info.local_elems, chunk):
        hi = min(info.local_elems, lo + chunk)
        master[lo:hi].normal_(0.0, 0.02, generator=gen)
        m[lo:hi].normal_(0.0, 1e-4, generator=gen)
        v[lo:hi].normal_(0.0, 1e-6, generator=gen).abs_()
    gen.manual_seed(SEED + 1 + rank)
    for off, n in zip(opt.offsets, numel):
        grads[off:off + n] = torch.empty(n, device="cuda", dtype=torch.float32).normal_(0.0, 1e-3, generator=gen).to(t_dt)
    if separate_work and (world == 1 or mode == ox.SYNC_REPLICATED):
        work.copy_(master.to(t_dt))
    opt.timestep = 1
    torch.cuda.synchronize()

    cfg = ox.StepConfig(**HYPER)

    def barrier():
        torch.cuda.synchronize()
        if comm is not None:
            comm.barrier()

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
                res = opt.step(cfg)
                profs.append(opt.profile())
            t1.record(stream)
        barrier()
        sec = t0.elapsed_time(t1) / 1e3
        if dist is not None:
            t = torch.tensor([sec], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        return sec, profs, res

    for _ in range(max(args.warmup, 3)):
        opt.step(cfg)
    sampler = ClockSampler(local_rank)
    sampler.start()
    sec, profs, res = timed(args.steps)
    clocks = sampler.stop()
    ms_per_step = sec * 1e3 / args.steps
    value = P * args.steps / sec

    # end to end: every step copies that step's gradients from pinned host memory, then reads the result back
    host_off, base = [], 0
    if not args.skip_e2e:
        host = torch.empty(P, dtype=t_dt).pin_memory()
        pos = 0
        for off, n in zip(opt.offsets, numel):
            host[pos:pos + n].copy_(grads[off:off + n])
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
                opt.step_async(cfg)
                if i + 1 < n_steps:
                    upload_next()
                opt.step_wait()
            t1.record(stream)
        barrier()
        sec = t0.elapsed_time(t1) / 1e3
        if dist is not None:
            t = torch.tensor([sec], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sec = float(t.item())
        return sec

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
    if mode in (ox.SYNC_SINGLE, ox.SYNC_P2P):
        nb = info.n_buckets
        early = max(1, (3 * nb) // 4)
        exposed = []
        for _ in range(5):
            opt.grads_ready(cfg, nb - early, early, producer_stream=stream.cuda_stream)
            sec1, _, _ = timed(1)
            exposed.append(sec1 * 1e3)
        overlap = {"buckets": nb, "buckets_reduced_during_backward": early, "exposed_ms_per_step": statistics.median(exposed)}

    aux = None
    if world == 1 and not args.skip_aux:
        aux = aux_measurements(ox, torch, opt, numel, stream, local_rank, t_dt, es)

    peak, peak_kind = measured_peaks()
    totals = sorted(p.total_ms for p in profs)
    pct = lambda q: totals[min(len(totals) - 1, int(q * len(totals)))]  # noqa: E731
    pull_kernel = {0: None, 1: "k_pull_sumsq", 2: "k_pull_bulk"}[opt.last_pull_kernel()]
    upd = statistics.mean(p.update_ms for p in profs)
    nrm = statistics.mean(p.norm_ms for p in profs)
    local_params = P if mode == ox.SYNC_REPLICATED else P / world  # parameters one rank's update kernel covers
    achieved = BYTES_UPDATE * local_params / (upd * 1e-3) / 1e9
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "params": P, "tensors": len(numel), "grad_dtype": args.dtype, "param_dtype": args.dtype,
                   "world": world, "sync": args.sync if world > 1 else "single",
                   "l2": "inputs larger than L2: %d B/param x %d params per rank per step" % (bytes_norm + BYTES_UPDATE, int(local_params)),
                   "hyper": HYPER},
        "roofline": {"bound": "hbm", "kernel": "k_adamw", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": peak_kind,
                     "traffic": ADAMW_TRAFFIC_RATIO * BYTES_UPDATE * local_params if args.dtype == "bf16" else None,
                     "traffic_source": "ncu capture of nano_dense scaled by parameters per launch" if args.dtype == "bf16" else "not captured for f32",
                     "algorithmic_bytes_per_launch": BYTES_UPDATE * local_params, "kernel_ms": upd,
                     "norm_kernel": {"kernel": pull_kernel if mode in (ox.SYNC_P2P, ox.SYNC_REPLICATED) else ("k_sumsq_stream16" if es == 2 else "k_sumsq") if mode == ox.SYNC_SINGLE else "k_sumsq",
                                     "kernel_ms": nrm, "achieved_gbs": bytes_norm * local_params / (nrm * 1e-3) / 1e9 if world == 1 else None}},
        "phases_ms": {k: statistics.mean(getattr(p, k) for p in profs) for k in
                      ("collect_ms", "norm_ms", "decide_ms", "update_ms", "publish_ms", "total_ms")},
        # device time of each timed step on this rank (CUDA events inside the library), for the spread
        "step_ms_device": {"median": statistics.median(totals), "p10": pct(0.10), "p90": pct(0.90)},
        "step_roofline": step_roofline(P, world, ms_per_step, peak, es),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": P * es * world, "d2h_bytes_per_step": 32 * world,
                "ms_per_step": e2e_sec * 1e3 / e2e_steps, "steps": e2e_steps,
                "copy_overlaps_previous_step": bool(pipelined and not args.skip_e2e)},
        # kernels of this library per step: norm (or pull) + reduce_partials + finalize + update; the copy mode runs
        # the pull and the update once per pipeline group (4 groups)
        "gpu_launches": (10 if mode == ox.SYNC_COPY else 4) * args.steps * world,
        "launch_geometry": opt.launch_geometry(),
        "overlap_with_backward": overlap,
        "aux": aux,
        "clocks": clocks,
        "result": {"grad_norm": res.grad_norm, "applied": res.applied, "timestep": res.timestep},
    }
    if rank == 0:
        if not args.no_cpu_baseline and world == 1:
            v, ms, cores, sample = cpu_arm(3, 1)
            v1, _, _, _ = cpu_arm(1, 1, threads=1)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                    "single_thread_value": v1}
        else:
            line["cpu_baseline"] = None
        print(json.dumps(line), flush=True)
    opt.destroy()
    if comm is not None:
        comm.barrier()
        comm.destroy()
    if dist is not None:
        dist.destroy_process_group()


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


def step_roofline(P: int, world: int, ms: float, hbm_gbs: float, es: int = 2) -> dict:
    """Whole-step roofline: the slower of the HBM term (es + 28 B/param on each rank's 1/world: 30 for 16-bit, 32 for
    f32) and, with more ranks, the NVLink term (reduce-scatter in + all-gather out in the gradients' and weights' own
    width, (world-1)/world * es B/param each)."""
    hbm_ms_nominal = (es + BYTES_UPDATE) * P / world / 8.0e12 * 1e3
    hbm_ms_measured = (es + BYTES_UPDATE) * P / world / (hbm_gbs * 1e9) * 1e3
    wire = 2 * (world - 1) / world * es * P
    wire_ms_nominal = wire / 900e9 * 1e3
    wire_ms_measured = wire / 770e9 * 1e3
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
    ap.add_argument("--skip-e2e", action="store_true", help="profiling runs: leave the host-fed leg out")
    ap.add_argument("--skip-aux", action="store_true", help="leave out the flatten and loader timings (1 GPU only)")
    ap.add_argument("--dtype", choices=["bf16", "f32"], default="bf16",
                    help="width of gradients and working weights: bf16 is the headline; f32 is the all-f32 configuration")
    ap.add_argument("--workload", default=WORKLOAD, help="parameter set; the headline is llama-3.2-1b, smaller sets serve profiler captures")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
