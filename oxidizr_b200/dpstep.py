"""Host-side mirror of the reference interface for the data-parallel optimizer step.

Thin Python classes over the C ABI of liboxz_dpstep.so, named after what they replace in oxidizr
(``LossScaler``, ``WeightDecaySpec``/``DecayPlan``, ``SpikeGuard``, ``LrPlan``, ``RowLayout``, the communicator,
and the post-accumulation half of ``LitTrainer::step_once``). All arithmetic and every decision is made by the
library; nothing here computes on the CPU in its place.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import numpy as np

from . import _ffi as ffi
from ._ffi import BF16, F16, F32, OxzError, check, lib

NAN = float("nan")
_NP = {F32: np.float32, BF16: np.uint16, F16: np.uint16}
DTYPE_NAMES = {"f32": F32, "bf16": BF16, "f16": F16}


# ------------------------------------------------------------------ communicator
class Communicator:
    """One rank's communicator (boostr ``Communicator`` as oxidizr uses it, src/dp/launch.rs:82-109)."""

    def __init__(self, handle: int, owns: bool = True):
        self._h = C.c_void_p(handle)
        self._owns = owns

    @staticmethod
    def unique_id() -> bytes:
        buf = (C.c_uint8 * 128)()
        check(lib().oxz_comm_unique_id(buf))
        return bytes(buf)

    @classmethod
    def init_rank(cls, device: int, rank: int, world: int, unique_id: bytes) -> "Communicator":
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        out = C.c_void_p()
        check(lib().oxz_comm_init_rank(device, rank, world, buf, C.byref(out)))
        return cls(out.value)

    @classmethod
    def init_all(cls, devices: list[int]) -> list["Communicator"]:
        n = len(devices)
        out = (C.c_void_p * n)()
        check(lib().oxz_comm_init_all(n, (C.c_int32 * n)(*devices), out))
        return [cls(out[i]) for i in range(n)]

    @classmethod
    def local_group(cls, n: int, devices: list[int] | None = None, timeout: float = 30.0) -> list["Communicator"]:
        """In-process rank threads with a collective timeout (LocalCommunicator::with_timeout, src/dp/launch.rs:58)."""
        out = (C.c_void_p * n)()
        dev = (C.c_int32 * n)(*devices) if devices is not None else None
        check(lib().oxz_comm_init_local(n, dev, timeout, out))
        return [cls(out[i]) for i in range(n)]

    @property
    def handle(self) -> C.c_void_p:
        return self._h

    def world_size(self) -> int:
        v = C.c_int32()
        check(lib().oxz_comm_world_size(self._h, C.byref(v)))
        return v.value

    def rank(self) -> int:
        v = C.c_int32()
        check(lib().oxz_comm_rank(self._h, C.byref(v)))
        return v.value

    def abort(self) -> None:
        check(lib().oxz_comm_abort(self._h))

    def barrier(self) -> None:
        check(lib().oxz_barrier(self._h))

    def sum_counts(self, scored: int, masks: int) -> tuple[int, int]:
        """The I64[2] sum of reduce_step_weighting (src/dp/weighting.rs:63-101)."""
        buf = (C.c_int64 * 2)(scored, masks)
        check(lib().oxz_allreduce_i64x2(self._h, buf))
        return buf[0], buf[1]

    def sum_f64(self, values: list[float]) -> list[float]:
        """Sum of a few host doubles over every rank (the logged loss, src/dp/reduce.rs:57-59). Blocking."""
        n = len(values)
        buf = (C.c_double * n)(*values)
        check(lib().oxz_allreduce_f64(self._h, buf, n))
        return [buf[i] for i in range(n)]

    def broadcast(self, device_ptr: int, nbytes: int, root: int = 0) -> None:
        check(lib().oxz_broadcast(self._h, C.c_void_p(device_ptr), nbytes, root))

    def destroy(self) -> None:
        if self._h and self._owns:
            lib().oxz_comm_destroy(self._h)
        self._h = C.c_void_p()


def run_ranks(comms: list["Communicator"], body):
    """Run ``body(rank, world, comm)`` once per rank, one thread each, and return the values in rank order
    (run_ranks, src/dp/launch.rs:183-272). The first rank to fail aborts the group, so peers blocked in a collective
    return; the error raised is the first failure's, with its rank as context."""
    world = len(comms)
    values: list = [None] * world
    errors: list = [None] * world

    def _body(rank, world_, _user):
        try:
            values[rank] = body(rank, world_, comms[rank])
            return ffi.OK
        except OxzError as e:
            errors[rank] = e
            lib().oxz_set_last_error(e.message.encode())
            return e.status
        except BaseException as e:  # a panic becomes an error
            errors[rank] = e
            lib().oxz_set_last_error(f"panic: {e}".encode())
            return ffi.ERR_INVALID
    cb = ffi.RankBody(_body)
    handles = (C.c_void_p * world)(*[c.handle for c in comms])
    failed = C.c_int32(-1)
    status = lib().oxz_run_ranks(world, handles, cb, None, C.byref(failed))
    if status != ffi.OK:
        err = OxzError(status, lib().oxz_last_error().decode())
        err.failed_rank = failed.value
        raise err from errors[failed.value] if 0 <= failed.value < world else None
    return values


# ------------------------------------------------------------------ loss scale
@dataclass
class LossScaleConfig:
    """``trainer.loss_scale`` (src/loss_scale/config.rs:28-41)."""
    initial: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000

    def _c(self) -> ffi.ScalerConfig:
        return ffi.ScalerConfig(self.initial, self.growth_factor, self.backoff_factor, self.growth_interval)

    def check(self) -> None:
        check(lib().oxz_scaler_check(C.byref(self._c())))


@dataclass
class GradScalerState:
    scale: float
    consecutive_ok: int = 0


class LossScaler:
    """The loss scaler of one run (src/loss_scale/scaler.rs:13-51)."""

    def __init__(self, config: LossScaleConfig | None = None):
        self.config = config or LossScaleConfig()
        self._cfg = self.config._c()
        self._st = ffi.ScalerState()
        check(lib().oxz_scaler_init(C.byref(self._cfg), C.byref(self._st)))

    def scale(self) -> float:
        return self._st.scale

    def state(self) -> GradScalerState:
        return GradScalerState(self._st.scale, self._st.consecutive_ok)

    def restore(self, state: GradScalerState) -> None:
        saved = ffi.ScalerState(state.scale, state.consecutive_ok)
        check(lib().oxz_scaler_restore(C.byref(saved), C.byref(self._st)))

    def record_step(self, overflow: bool, spike_skip: bool = False) -> None:
        check(lib().oxz_scaler_record_step(C.byref(self._cfg), C.byref(self._st), int(overflow), int(spike_skip)))


# ------------------------------------------------------------------ weight decay
_RULES = {"decay_all": ffi.DECAY_ALL, "skip_1d": ffi.SKIP_1D, "skip_all": ffi.SKIP_ALL}


@dataclass
class WeightDecaySpec:
    """The resolved weight decay rule of one run (src/weight_decay/rule.rs:49-118)."""
    rule: str = "skip_1d"
    no_decay_patterns: list[str] = field(default_factory=list)

    def _patterns(self):
        n = len(self.no_decay_patterns)
        return (C.c_char_p * max(n, 1))(*[p.encode() for p in self.no_decay_patterns]), n

    def check(self) -> None:
        arr, n = self._patterns()
        check(lib().oxz_decay_check(_RULES[self.rule], arr, n))

    def excludes(self, name: str, rank: int) -> bool:
        arr, n = self._patterns()
        out = C.c_int32()
        check(lib().oxz_decay_excludes(_RULES[self.rule], arr, n, name.encode(), rank, C.byref(out)))
        return bool(out.value)


@dataclass
class TensorInfo:
    """One trainable tensor as the decay rule sees it (src/weight_decay/plan.rs:10-19)."""
    name: str       # checkpoint name, ``model.``-prefixed
    shape: tuple
    id: int | None = None

    @property
    def elements(self) -> int:
        return int(math.prod(self.shape))


class DecayPlan:
    """The no-decay set of one run (src/weight_decay/plan.rs:22-122). A repeated id counts once."""

    def __init__(self, spec: WeightDecaySpec, tensors: list[TensorInfo]):
        spec.check()
        self.spec = spec
        self.no_decay: list[bool] = []
        self.decay_tensors = self.decay_elements = self.no_decay_elements = 0
        self.tensors: list[TensorInfo] = []
        seen = set()
        for i, t in enumerate(tensors):
            tid = t.id if t.id is not None else ("#", i)
            if tid in seen:
                continue
            seen.add(tid)
            self.tensors.append(t)
            ex = spec.excludes(t.name, len(t.shape))
            self.no_decay.append(ex)
            if ex:
                self.no_decay_elements += t.elements
            else:
                self.decay_tensors += 1
                self.decay_elements += t.elements

    def summary(self, weight_decay: float) -> str:
        return (f"Weight decay {weight_decay} with rule {self.spec.rule}: {self.decay_tensors} tensors "
                f"({self.decay_elements} params) decay, {sum(self.no_decay)} tensors "
                f"({self.no_decay_elements} params) do not")


# ------------------------------------------------------------------ spike guard
@dataclass
class SpikeGuardConfig:
    """``trainer.spike_guard`` (src/metrics/config.rs:69-115)."""
    window: int = 100
    z_threshold: float = 6.0
    min_steps: int = 50
    action: str = "skip"


class SpikeGuard:
    """EMA loss-spike guard (src/metrics/spike.rs:72-168)."""

    def __init__(self, config: SpikeGuardConfig):
        self.config = config
        self._cfg = ffi.SpikeConfig(config.window, config.z_threshold, config.min_steps, int(config.action == "warn"), 0)
        self._st = ffi.SpikeState()
        self.last_flagged = False
        skip, flagged = C.c_int32(), C.c_int32()
        probe = ffi.SpikeState()
        check(lib().oxz_spike_judge(C.byref(self._cfg), C.byref(probe), 0, NAN, C.byref(skip), C.byref(flagged)))

    def judge(self, index: int, loss: float) -> bool:
        """True when the 0-based step ``index`` must skip the optimizer (src/metrics/state.rs:79-86)."""
        skip, flagged = C.c_int32(), C.c_int32()
        check(lib().oxz_spike_judge(C.byref(self._cfg), C.byref(self._st), index, loss, C.byref(skip), C.byref(flagged)))
        self.last_flagged = bool(flagged.value)
        return bool(skip.value)

    @property
    def state(self):
        s = self._st
        return dict(mean=s.mean, variance=s.variance, observed=s.observed, detected=s.detected, skipped=s.skipped)


# ------------------------------------------------------------------ learning rate
_SCHED = {"constant": ffi.LR_CONSTANT, "cosine": ffi.LR_COSINE, "linear": ffi.LR_LINEAR, "wsd": ffi.LR_WSD}
_SHAPE = {"linear": ffi.SHAPE_LINEAR, "cosine": ffi.SHAPE_COSINE, "sqrt": ffi.SHAPE_SQRT}


class LrPlan:
    """Learning rate of every step of one run (src/schedule.rs:135-202)."""

    def __init__(self, base_lr: float, schedule: str = "constant", warmup_steps: int = 0, total_steps: int = 0,
                 min_lr_ratio: float = 0.0, decay_steps: int | None = None, decay_ratio: float | None = None,
                 decay_shape: str = "linear"):
        if schedule == "wsd" and decay_steps is None:
            decay_steps = int(math.ceil(float(total_steps) * (0.1 if decay_ratio is None else decay_ratio)))
        self._c = ffi.LrPlanC(base_lr, min_lr_ratio, warmup_steps, total_steps, decay_steps or 0, _SCHED[schedule],
                              _SHAPE[decay_shape])
        self.lr_at(0)

    def lr_at(self, step: int) -> float:
        out = C.c_double()
        check(lib().oxz_lr_at(C.byref(self._c), step, C.byref(out)))
        return out.value


# ------------------------------------------------------------------ rows
@dataclass(frozen=True)
class DataPosition:
    epoch: int = 0
    row: int = 0


class RowLayout:
    """Row and batch counts of one loader's row range (src/data/rows.rs:53-208)."""

    def __init__(self, num_rows: int, rank_batch_size: int, world_size: int = 1):
        self._c = ffi.RowLayoutC(num_rows, rank_batch_size, world_size)
        check(lib().oxz_rows_check(C.byref(self._c)))
        self.num_rows, self.rank_batch_size, self.world_size = num_rows, rank_batch_size, world_size

    def batch_size(self) -> int:
        return self.rank_batch_size * self.world_size

    def batches_per_epoch(self) -> int:
        return self.num_rows // self.batch_size()

    def total_steps(self, grad_accum: int, num_epochs: int) -> int:
        return self.batches_per_epoch() * num_epochs // max(grad_accum, 1)

    def advance(self, pos: DataPosition, batches: int) -> DataPosition:
        out = ffi.DataPositionC()
        check(lib().oxz_rows_advance(C.byref(self._c), ffi.DataPositionC(pos.epoch, pos.row), batches, C.byref(out)))
        return DataPosition(out.epoch, out.row)

    def position_after_steps(self, steps: int, grad_accum: int) -> DataPosition:
        return self.advance(DataPosition(), steps * grad_accum)

    def batch_epoch(self, pos: DataPosition) -> int:
        """The epoch whose row order the batch drawn at `pos` reads (it rolls over when fewer rows than a global
        batch are left, src/data/rows.rs:153-165)."""
        v = C.c_uint64()
        check(lib().oxz_rows_batch_epoch(C.byref(self._c), ffi.DataPositionC(pos.epoch, pos.row), C.byref(v)))
        return v.value

    def next_window(self, pos: DataPosition, rank: int, seq_len: int, tokens: np.ndarray | None = None,
                    first_row: int = 0, row_order: tuple[int, np.ndarray] | None = None):
        """One rank's rows of the next global batch: (rows, inputs, targets, next position). Stream order, or with
        row_order = (epoch, permutation) the reference's shuffled order with the permutation the caller made
        (EpochOrder::row, src/data/rows.rs:240-256)."""
        B = self.rank_batch_size
        rows = np.empty(B, dtype=np.uint64)
        nxt = ffi.DataPositionC()
        inputs = targets = None
        tok_p, n_tok, in_p, tg_p = None, 0, None, None
        if tokens is not None:
            tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
            inputs = np.empty((B, seq_len), dtype=np.int64)
            targets = np.empty((B, seq_len), dtype=np.int64)
            tok_p = tokens.ctypes.data_as(C.POINTER(C.c_uint32))
            n_tok = tokens.size
            in_p, tg_p = inputs.ctypes.data_as(ffi.i64p), targets.ctypes.data_as(ffi.i64p)
        if row_order is not None:
            epoch, perm = row_order
            perm = np.ascontiguousarray(perm, dtype=np.uint32)
            check(lib().oxz_rows_next_window_ordered(C.byref(self._c), ffi.DataPositionC(pos.epoch, pos.row), rank, seq_len,
                                                     first_row, tok_p, n_tok, epoch, perm.ctypes.data_as(C.POINTER(C.c_uint32)),
                                                     perm.size, rows.ctypes.data_as(ffi.u64p), in_p, tg_p, C.byref(nxt)))
            return rows, inputs, targets, DataPosition(nxt.epoch, nxt.row)
        check(lib().oxz_rows_next_window(C.byref(self._c), ffi.DataPositionC(pos.epoch, pos.row), rank, seq_len,
                                         first_row, tok_p, n_tok, rows.ctypes.data_as(ffi.u64p), in_p, tg_p,
                                         C.byref(nxt)))
        return rows, inputs, targets, DataPosition(nxt.epoch, nxt.row)


class LitDataLoader:
    """The rank-sliced loader over one u32 token file in stream order (src/data/ranks.rs:25-41, src/data/batch.rs:51-71)."""

    def __init__(self, path: str, batch_size: int, seq_len: int, rank: int = 0, world_size: int = 1, first_row: int = 0,
                 end_row: int = 0, device: int = 0):
        self._h = C.c_void_p()
        check(lib().oxz_loader_open(path.encode(), seq_len, batch_size, rank, world_size, first_row, end_row, device,
                                    C.byref(self._h)))
        self.batch_size, self.seq_len, self.rank, self.world_size = batch_size, seq_len, rank, world_size

    @classmethod
    def from_files(cls, paths: list[str], batch_size: int, seq_len: int, rank: int = 0, world_size: int = 1,
                   row_ranges: list[tuple[int, int]] | None = None, device: int = 0) -> "LitDataLoader":
        """from_files + with_row_ranges + with_rank (src/data/multi_source.rs:17-52): the files' whole rows in order,
        restricted to ascending global row ranges (end exclusive)."""
        self = cls.__new__(cls)
        self._h = C.c_void_p()
        spans = [v for span in (row_ranges or []) for v in span]
        check(lib().oxz_loader_open_files((C.c_char_p * max(len(paths), 1))(*[p.encode() for p in paths]), len(paths), seq_len,
                                          batch_size, rank, world_size, (C.c_uint64 * max(len(spans), 1))(*spans),
                                          len(spans) // 2, device, C.byref(self._h)))
        self.batch_size, self.seq_len, self.rank, self.world_size = batch_size, seq_len, rank, world_size
        return self

    def source_rows(self) -> list[int]:
        n = C.c_uint32()
        check(lib().oxz_loader_source_rows(self._h, None, 0, C.byref(n)))
        rows = (C.c_uint64 * max(n.value, 1))()
        check(lib().oxz_loader_source_rows(self._h, rows, n.value, C.byref(n)))
        return list(rows)[:n.value]

    def num_rows(self) -> int:
        v = C.c_uint64()
        check(lib().oxz_loader_num_rows(self._h, C.byref(v)))
        return v.value

    def position(self) -> DataPosition:
        p = ffi.DataPositionC()
        check(lib().oxz_loader_position(self._h, C.byref(p)))
        return DataPosition(p.epoch, p.row)

    def seek(self, pos: DataPosition) -> None:
        check(lib().oxz_loader_seek(self._h, ffi.DataPositionC(pos.epoch, pos.row)))

    def next_batch(self, stream: int | None = None):
        """(inputs device address, targets device address, global rows): [batch, seq_len] i64 each."""
        i, t = C.c_void_p(), C.c_void_p()
        rows = (C.c_uint64 * self.batch_size)()
        check(lib().oxz_loader_next_batch_async(self._h, C.c_void_p(stream) if stream else None, C.byref(i), C.byref(t), rows))
        return i.value, t.value, list(rows)

    def with_prefetch(self, depth: int = 2) -> "LitDataLoader":
        """PrefetchDataLoader::new (src/data/prefetch.rs:86-115): a host thread keeps the coming batches' rows ready in
        pinned memory; the batches are the unprefetched loader's."""
        check(lib().oxz_loader_set_prefetch(self._h, depth))
        return self

    def set_row_order(self, epoch: int, perm: np.ndarray | None) -> "LitDataLoader":
        """with_row_order(RowOrder::Shuffled) (src/data/construction.rs:140) with the epoch's permutation made by the
        caller (epoch_permutation, src/data/rows.rs:258-263): perm[slot] is the loader row read at `slot`. The loader
        keeps two epochs' orders; None returns to stream order."""
        if perm is None:
            check(lib().oxz_loader_set_row_order(self._h, epoch, None, 0))
            return self
        perm = np.ascontiguousarray(perm, dtype=np.uint32)
        check(lib().oxz_loader_set_row_order(self._h, epoch, perm.ctypes.data_as(C.POINTER(C.c_uint32)), perm.size))
        return self

    def next_rows(self) -> list[int]:
        """The global rows of the next batch, without touching the device; the position moves on as after a batch."""
        rows = (C.c_uint64 * self.batch_size)()
        check(lib().oxz_loader_next_rows(self._h, rows))
        return list(rows)

    def with_mixture(self, weights: list[float], rows_per_epoch: int | None = None) -> "LitDataLoader":
        """src/data/mixture/loader.rs:16-33, stream order: one weight per source; the layout then counts rows_per_epoch
        rows (default: the sources' training rows) and the position returns to the start."""
        check(lib().oxz_loader_set_mixture(self._h, (C.c_double * max(len(weights), 1))(*weights), len(weights),
                                           int(rows_per_epoch is not None), rows_per_epoch or 0))
        return self

    def mixture_sources(self) -> list[dict] | None:
        n = C.c_uint32()
        check(lib().oxz_loader_mixture_sources(self._h, None, 0, C.byref(n)))
        if n.value == 0:
            return None
        out = (ffi.MixtureSource * n.value)()
        check(lib().oxz_loader_mixture_sources(self._h, out, n.value, C.byref(n)))
        return [dict(weight=s.weight, rows_per_epoch=s.rows_per_epoch, train_rows=s.train_rows,
                     repeats=s.rows_per_epoch / max(s.train_rows, 1)) for s in out]

    def with_target_mask(self, target_base: int, always_score: list[int] = ()) -> "LitDataLoader":
        """TargetMask::PrefixLm (src/data/mask.rs:21-47): a position scores iff its target id is at least target_base
        or is one of always_score."""
        ids = list(always_score)
        check(lib().oxz_loader_set_target_mask(self._h, 1, target_base, (C.c_uint32 * max(len(ids), 1))(*ids), len(ids)))
        return self

    def with_document_mask(self, separator_id: int) -> "LitDataLoader":
        """src/data/host_masks.rs:28-35: separator inputs are unscored and each batch carries its document segments."""
        check(lib().oxz_loader_set_document_mask(self._h, 1, separator_id))
        return self

    def batch_masks(self) -> dict:
        """Of the batch drawn last: device addresses of loss_mask [B,S] f32, segment_ids [B,S] i32 and cu_seqlens
        (None for what is off), and two callables that read scored / n_segments from pinned host memory: call them
        once the stream has passed the batch."""
        m = ffi.BatchMasks()
        check(lib().oxz_loader_batch_masks(self._h, C.byref(m)))
        return dict(loss_mask=m.loss_mask, segment_ids=m.segment_ids, cu_seqlens=m.cu_seqlens,
                    scored=lambda: int(m.scored[0]), n_segments=lambda: int(m.n_segments[0]))

    def close(self) -> None:
        if self._h:
            lib().oxz_loader_close(self._h)
            self._h = C.c_void_p()


# ------------------------------------------------------------------ the checkpoint meta's keys on this path
@dataclass
class SpikeGuardState:
    """src/metrics/spike.rs:14-26."""
    mean: float = 0.0
    variance: float = 0.0
    observed: int = 0
    detected: int = 0
    skipped: int = 0


@dataclass
class MixtureRecord:
    """What a checkpoint meta records of a weighted mixture (src/data/mixture/record.rs:13-19)."""
    weights: list[float]
    rows_per_epoch: int


@dataclass
class CheckpointMeta:
    """The keys of ``checkpoint_step_N.meta.json`` (CheckpointMeta, src/config.rs:1223-1302) that the optimizer path
    records and reads on resume (src/checkpoint_set/snapshot.rs:245-262). ``None`` is a key the file does not hold."""
    step: int
    checkpoint_file: str = ""
    optimizer_file: str | None = None
    data_position: DataPosition | None = None
    weight_decay_rule: str | None = None
    no_decay_patterns: list[str] = field(default_factory=list)
    loss_scale: GradScalerState | None = None
    world_size: int | None = None
    global_batch_rows: int | None = None
    spike_guard: SpikeGuardState | None = None
    mixture: "MixtureRecord | None" = None

    def weight_decay_spec(self) -> WeightDecaySpec:
        """WeightDecaySpec::of_meta (src/weight_decay/rule.rs:68-74): a meta without the rule is a legacy run."""
        return WeightDecaySpec(self.weight_decay_rule or "decay_all", list(self.no_decay_patterns))

    def save_to(self, path: str) -> None:
        m = ffi.ResumeMeta()
        m.step = self.step
        m.checkpoint_file = self.checkpoint_file.encode()
        m.optimizer_file = (self.optimizer_file or "").encode()
        if self.data_position is not None:
            m.has_data_position, m.data_position = 1, ffi.DataPositionC(self.data_position.epoch, self.data_position.row)
        if self.weight_decay_rule is not None:
            m.has_weight_decay_rule, m.weight_decay_rule = 1, _RULES[self.weight_decay_rule]
        if self.loss_scale is not None:
            m.has_loss_scale, m.loss_scale = 1, ffi.ScalerState(self.loss_scale.scale, self.loss_scale.consecutive_ok)
        if self.world_size is not None:
            m.has_world_size, m.world_size = 1, self.world_size
        if self.global_batch_rows is not None:
            m.has_global_batch_rows, m.global_batch_rows = 1, self.global_batch_rows
        if self.spike_guard is not None:
            g = self.spike_guard
            m.has_spike_guard, m.spike_guard = 1, ffi.SpikeState(g.mean, g.variance, g.observed, g.detected, g.skipped)
        n = len(self.no_decay_patterns)
        m.n_no_decay_patterns = n
        arr = (C.c_char_p * max(n, 1))(*[p.encode() for p in self.no_decay_patterns])
        weights = list(self.mixture.weights) if self.mixture is not None else []
        if self.mixture is not None:
            m.has_mixture, m.n_mixture_weights, m.mixture_rows_per_epoch = 1, len(weights), self.mixture.rows_per_epoch
        check(lib().oxz_meta_save(path.encode(), C.byref(m), arr, (C.c_double * max(len(weights), 1))(*weights)))

    @classmethod
    def load(cls, path: str) -> "CheckpointMeta":
        m = ffi.ResumeMeta()
        check(lib().oxz_meta_load(path.encode(), C.byref(m)))
        patterns = []
        for i in range(m.n_no_decay_patterns):
            buf = C.create_string_buffer(4096)
            check(lib().oxz_meta_no_decay_pattern(path.encode(), i, buf, len(buf)))
            patterns.append(buf.value.decode())
        rules = {v: k for k, v in _RULES.items()}
        g = m.spike_guard
        mixture = None
        if m.has_mixture:
            w, nw = (C.c_double * max(m.n_mixture_weights, 1))(), C.c_uint32()
            check(lib().oxz_meta_mixture_weights(path.encode(), w, m.n_mixture_weights, C.byref(nw)))
            mixture = MixtureRecord(list(w)[:nw.value], m.mixture_rows_per_epoch)
        return cls(
            mixture=mixture,
            step=m.step, checkpoint_file=m.checkpoint_file.decode(), optimizer_file=m.optimizer_file.decode() or None,
            data_position=DataPosition(m.data_position.epoch, m.data_position.row) if m.has_data_position else None,
            weight_decay_rule=rules[m.weight_decay_rule] if m.has_weight_decay_rule else None, no_decay_patterns=patterns,
            loss_scale=GradScalerState(m.loss_scale.scale, m.loss_scale.consecutive_ok) if m.has_loss_scale else None,
            world_size=m.world_size if m.has_world_size else None,
            global_batch_rows=m.global_batch_rows if m.has_global_batch_rows else None,
            spike_guard=SpikeGuardState(g.mean, g.variance, g.observed, g.detected, g.skipped) if m.has_spike_guard else None)


def check_resume_world(meta_path: str | None, start_step: int, world: int, global_batch_rows: int) -> str | None:
    """src/dp/resume.rs:19-55: raises when the meta records another world size; returns a warning for another global
    batch, else None."""
    buf = C.create_string_buffer(1024)
    check(lib().oxz_check_resume_world(meta_path.encode() if meta_path else None, start_step, world, global_batch_rows,
                                       buf, len(buf)))
    return buf.value.decode() or None


def check_mixture_resume(meta_path: str | None, start_step: int, current: MixtureRecord | None) -> None:
    """src/data/mixture/record.rs:40-70: a resume must run the mixture the meta records."""
    w = list(current.weights) if current is not None else []
    check(lib().oxz_check_mixture_resume(meta_path.encode() if meta_path else None, start_step, int(current is not None),
                                         (C.c_double * max(len(w), 1))(*w), len(w), current.rows_per_epoch if current else 0))


def read_loss_scale_state(meta_path: str | None, start_step: int) -> GradScalerState | None:
    """src/loss_scale/resume.rs:14-29."""
    has, st = C.c_int32(), ffi.ScalerState()
    check(lib().oxz_read_loss_scale_state(meta_path.encode() if meta_path else None, start_step, C.byref(has), C.byref(st)))
    return GradScalerState(st.scale, st.consecutive_ok) if has.value else None


def mixture_quotas(weights: list[float], rows: int) -> list[int]:
    """src/data/mixture/quota.rs:22-57."""
    out = (C.c_uint64 * len(weights))()
    check(lib().oxz_mixture_quotas((C.c_double * len(weights))(*weights), len(weights), rows, out))
    return list(out)


def step_weighting(local_micro_batches: int, world: int, scored: int, masked_ranks: int):
    """StepWeighting::over_ranks on the summed counts (src/dp/weighting.rs:46-61): (micro_batches, scored or None)."""
    mb, gs = C.c_uint64(), C.c_int64()
    check(lib().oxz_step_weighting(local_micro_batches, world, (C.c_int64 * 2)(scored, masked_ranks), C.byref(mb),
                                   C.byref(gs)))
    return mb.value, (None if gs.value < 0 else gs.value)


# ------------------------------------------------------------------ the optimizer step
@dataclass
class StepConfig:
    """The trainer keys the step reads, with the reference's defaults (src/config.rs:40-62)."""
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-6
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    max_grad_value: float = NAN
    target_grad_norm: float = NAN
    loss_scale: float = NAN
    clip_eps: float = 1e-6
    decay_after: int = 0
    eps_mode: int = 0
    spike_skip: bool = False

    def hyper(self) -> ffi.Hyper:
        return ffi.Hyper(self.lr, self.beta1, self.beta2, self.eps, self.weight_decay, self.max_grad_norm,
                         self.max_grad_value, self.target_grad_norm, self.loss_scale, self.clip_eps,
                         self.decay_after, self.eps_mode, int(self.spike_skip), 0)


class DpOptimizer:
    """Flat-buffer AdamW state of one rank plus the fused step (replaces boostr FusedAdamW + the collectives).

    ``numel`` keeps ``parameter_ids`` order. ``no_decay`` comes from :class:`DecayPlan`.
    """

    def __init__(self, numel: list[int], no_decay: list[bool] | None = None, grad_dtype: int = BF16,
                 param_dtype: int = BF16, world: int = 1, rank: int = 0, sync_mode: int | None = None,
                 device: int = 0, bucket_bytes: int = 0, lr_scale: list[float] | None = None,
                 comm: Communicator | None = None, allocate: bool = True):
        T = len(numel)
        self.numel = [int(n) for n in numel]
        self.grad_dtype, self.param_dtype, self.world, self.rank, self.device = grad_dtype, param_dtype, world, rank, device
        if sync_mode is None:
            sync_mode = ffi.SYNC_SINGLE if world == 1 else ffi.SYNC_P2P
        self.sync_mode = sync_mode
        self._numel = (C.c_uint64 * max(T, 1))(*self.numel)
        self._nd = (C.c_uint8 * max(T, 1))(*[int(bool(x)) for x in (no_decay or [False] * T)])
        self._ls = (C.c_float * max(T, 1))(*(lr_scale or [1.0] * T))
        desc = ffi.PlanDesc(T, self._numel, self._nd, self._ls, grad_dtype, param_dtype, world, rank, sync_mode, device,
                            bucket_bytes)
        self._h = C.c_void_p()
        check(lib().oxz_plan_create(C.byref(desc), C.byref(self._h)))
        self.comm = comm
        self.info = ffi.PlanInfo()
        check(lib().oxz_plan_query(self._h, C.byref(self.info)))
        off = (C.c_uint64 * max(T, 1))()
        check(lib().oxz_plan_tensor_offsets(self._h, off))
        self.offsets = [off[i] for i in range(T)]
        self.allocated = False
        if allocate:
            self.alloc()

    # -- layout
    def bucket(self, b: int, rank: int | None = None):
        vals = [C.c_uint64() for _ in range(4)]
        check(lib().oxz_plan_bucket(self._h, b, self.rank if rank is None else rank, *[C.byref(v) for v in vals]))
        return tuple(v.value for v in vals)

    def local_index(self, flat_index: int, rank: int | None = None) -> int | None:
        out = C.c_uint64()
        check(lib().oxz_plan_local_index(self._h, self.rank if rank is None else rank, flat_index, C.byref(out)))
        return None if out.value == 0xFFFFFFFFFFFFFFFF else out.value

    # -- state
    def alloc(self) -> None:
        check(lib().oxz_state_alloc(self._h, self.comm.handle if self.comm else None))
        self.allocated = True

    def set_stream(self, stream: int | None) -> None:
        check(lib().oxz_plan_set_stream(self._h, C.c_void_p(stream) if stream else None))

    def pointers(self) -> dict:
        """Device addresses of the flat buffers: grads, work, master, exp_avg, exp_avg_sq."""
        ps = [C.c_void_p() for _ in range(5)]
        check(lib().oxz_state_pointers(self._h, *[C.byref(p) for p in ps]))
        return dict(zip(("grads", "work", "master", "exp_avg", "exp_avg_sq"), [p.value for p in ps]))

    def _dtype_of(self, kind: int):
        return _NP[self.grad_dtype] if kind == ffi.STATE_GRADS else _NP[self.param_dtype] if kind == ffi.STATE_WORK else np.float32

    def import_tensor(self, kind: int, tensor: int, host: np.ndarray) -> None:
        host = np.ascontiguousarray(host, dtype=self._dtype_of(kind)).reshape(-1)
        if host.size != self.numel[tensor]:
            raise ValueError(f"tensor {tensor} has {self.numel[tensor]} elements, got {host.size}")
        if host.size:
            check(lib().oxz_state_import(self._h, kind, tensor, host.ctypes.data))

    def export_tensor(self, kind: int, tensor: int, out: np.ndarray | None = None) -> np.ndarray:
        if out is None:
            out = np.zeros(self.numel[tensor], dtype=self._dtype_of(kind))
        if out.size:
            check(lib().oxz_state_export(self._h, kind, tensor, out.ctypes.data))
        return out

    @property
    def timestep(self) -> int:
        """Applied optimizer steps (LitTrainer::optimizer_timestep, src/trainer.rs:906-908)."""
        v = C.c_uint64()
        check(lib().oxz_state_timestep(self._h, C.byref(v)))
        return v.value

    @timestep.setter
    def timestep(self, t: int) -> None:
        check(lib().oxz_state_set_timestep(self._h, t))

    # -- optimizer state file
    def _names_shapes(self, tensors):
        T = len(tensors)
        if T != len(self.numel):
            raise ValueError(f"{T} tensors named, the optimizer holds {len(self.numel)}")
        names = (C.c_char_p * max(T, 1))(*[t.name.encode() for t in tensors])
        ndim = (C.c_uint32 * max(T, 1))(*[len(t.shape) for t in tensors])
        flat = [d for t in tensors for d in t.shape]
        dims = (C.c_uint64 * max(len(flat), 1))(*flat)
        return names, ndim, dims

    def save_optimizer(self, path: str, tensors: list["TensorInfo"]) -> None:
        """Write `<name>.exp_avg/.exp_avg_sq/.master` and `__step` as the reference's optimizer file does
        (src/checkpoint_set/optimizer_io.rs:62-74). Collective at world > 1; rank 0 writes."""
        names, ndim, dims = self._names_shapes(tensors)
        check(lib().oxz_optimizer_save(self._h, self.comm.handle if self.comm else None, path.encode(), names, ndim, dims))

    def load_optimizer(self, path: str, tensors: list["TensorInfo"]) -> None:
        """Strict load of an optimizer file (src/checkpoint_set/optimizer_io.rs:113-137)."""
        names, ndim, dims = self._names_shapes(tensors)
        check(lib().oxz_optimizer_load(self._h, path.encode(), names, ndim, dims))

    # -- gradients in
    def flatten_grads(self, device_ptrs: list[int | None], accumulate: bool = False) -> None:
        arr = (C.c_void_p * max(len(device_ptrs), 1))(*[C.c_void_p(p) if p else None for p in device_ptrs])
        check(lib().oxz_grads_flatten_async(self._h, arr, int(accumulate)))

    def upload_grads(self, tensor: int, host_ptr: int) -> None:
        check(lib().oxz_grads_upload_async(self._h, tensor, C.c_void_p(host_ptr)))

    def double_buffer_grads(self) -> None:
        """A second gradient buffer: the next step's gradients can arrive while this step still reads its own."""
        check(lib().oxz_grads_double_buffer(self._h, self.comm.handle if self.comm else None))

    def upload_next_grads(self, tensor: int, host_ptr: int) -> None:
        """Into the buffer that is not current, on the plan's upload stream; allowed while a step is in flight."""
        check(lib().oxz_grads_upload_next_async(self._h, tensor, C.c_void_p(host_ptr)))

    def swap_grads(self) -> None:
        """The other buffer becomes the current one; the next step waits for the uploads into it."""
        check(lib().oxz_grads_swap(self._h))

    # -- the step
    def step_async(self, cfg: StepConfig, present: list[bool] | None = None, extras: list[float] | None = None) -> None:
        h = cfg.hyper()
        pres = (C.c_uint8 * max(len(present), 1))(*[int(bool(x)) for x in present]) if present is not None else None
        n = len(extras) if extras else 0
        self._extras = (C.c_double * max(n, 1))(*(extras or [0.0]))
        self._n_extras = n
        check(lib().oxz_step_async(self._h, self.comm.handle if self.comm else None, C.byref(h), pres, self._extras, n))

    def grads_ready(self, cfg: StepConfig, first_bucket: int, n_buckets: int, present: list[bool] | None = None,
                    producer_stream: int | None = None) -> None:
        """Reduce buckets [first_bucket, first_bucket + n_buckets) now, on a side stream, while backward still
        produces the others; the step's step_async/step then handles what is left. Collective at world > 1."""
        h = cfg.hyper()
        pres = (C.c_uint8 * max(len(present), 1))(*[int(bool(x)) for x in present]) if present is not None else None
        check(lib().oxz_grads_ready_async(self._h, self.comm.handle if self.comm else None, C.byref(h), pres, first_bucket,
                                          n_buckets, C.c_void_p(producer_stream) if producer_stream else None))

    def step_wait(self) -> ffi.StepResult:
        res = ffi.StepResult()
        check(lib().oxz_step_wait(self._h, C.byref(res)))
        self.last_extras = [self._extras[i] for i in range(self._n_extras)]
        return res

    def step(self, cfg: StepConfig, present: list[bool] | None = None, extras: list[float] | None = None) -> ffi.StepResult:
        self.step_async(cfg, present, extras)
        return self.step_wait()

    def launch_geometry(self) -> dict:
        v = [C.c_int32() for _ in range(3)]
        check(lib().oxz_plan_launch_geometry(self._h, *[C.byref(x) for x in v]))
        return dict(sm_count=v[0].value, norm_blocks=v[1].value, update_blocks=v[2].value)

    def last_pull_kernel(self) -> int:
        """0 none yet, 1 per-lane loads, 2 bulk asynchronous copies: the kernel of the most recent peer pull."""
        v = C.c_int32()
        check(lib().oxz_plan_last_pull_kernel(self._h, C.byref(v)))
        return v.value

    def last_update_kernel(self) -> int:
        """0 none yet, 1 k_adamw (one tile per warp), 2 k_adamw_wide (256-bit weight stores), 3 k_adamw_staged."""
        v = C.c_int32()
        check(lib().oxz_plan_last_update_kernel(self._h, C.byref(v)))
        return v.value

    def exchange_kind(self) -> int:
        """How the ranks meet for the step's barriers and small sum: 0 one rank, 1 the communicator's collectives,
        2 mailboxes in peer memory."""
        v = C.c_int32()
        check(lib().oxz_plan_exchange_kind(self._h, C.byref(v)))
        return v.value

    def grad_norms_per_tensor(self, loss_scale: float = NAN, max_grad_value: float = NAN) -> list[float]:
        """grad_norm_for_tensor for every tensor (src/trainer.rs:933-937): what diagnose_bad_gradients and the
        DEBUG_GRAD breakdown read (src/trainer.rs:940-1020). -1 marks a tensor no rank had a gradient for.
        Collective at world > 1; call after a step, before the gradients change."""
        T = len(self.numel)
        out = (C.c_double * max(T, 1))()
        check(lib().oxz_grad_norms_per_tensor(self._h, self.comm.handle if self.comm else None, loss_scale, max_grad_value, out))
        return [out[i] for i in range(T)]

    def set_profile(self, on: bool) -> None:
        """Per-phase CUDA-event timing of each step (the PROFILE_TRAIN switch, src/trainer.rs:262-263)."""
        check(lib().oxz_plan_set_profile(self._h, int(on)))

    def profile(self) -> ffi.StepProfile:
        out = ffi.StepProfile()
        check(lib().oxz_step_profile_read(self._h, C.byref(out)))
        return out

    def destroy(self) -> None:
        if self._h:
            lib().oxz_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass


def compute_grad_norm(device_ptr: int, dtype: int, n: int, loss_scale: float = NAN, max_grad_value: float = NAN,
                      stream: int | None = None) -> float:
    """Global L2 norm of device gradients as a pure measurement (compute_grad_norm(.., f64::MAX), src/grad_clip.rs:49)."""
    out = C.c_double()
    check(lib().oxz_grad_norm(C.c_void_p(device_ptr), dtype, n, loss_scale, max_grad_value,
                              C.c_void_p(stream) if stream else None, C.byref(out)))
    return out.value


def diagnose_bad_gradients(names: list[str], norms: list[float], top: int = 5) -> list[tuple[str, float]]:
    """The reference's report after a non-finite norm (diagnose_bad_gradients, src/trainer.rs:990-1020): the tensors
    whose own norm is inf, NaN or above 1e6, non-finite ones first, then by falling norm; at most `top` of them."""
    bad = [(n, v) for n, v in zip(names, norms) if math.isinf(v) or math.isnan(v) or v > 1e6]
    bad.sort(key=lambda nv: (0 if (math.isnan(nv[1]) or math.isinf(nv[1])) else 1, -nv[1] if math.isfinite(nv[1]) else 0.0))
    return bad[:top]


def selftest_bounded_wait(device: int = 0, limit_ms: int = 50) -> int:
    """What a rank sees when a peer never arrives, shown on one GPU without any fault: returns what the gate kernel
    recorded (1 = its wait ran out after limit_ms); raises if the context did not stay usable."""
    out = C.c_int32(-1)
    check(lib().oxz_selftest_bounded_wait(device, limit_ms, C.byref(out)))
    return out.value


STATIC_NORM_MAX_CLUSTERS = 256


def compute_grad_norm_static(device_ptr: int, dtype: int, n: int, loss_scale: float = NAN,
                             max_grad_value: float = NAN, clusters: int = 0, stream: int | None = None) -> float:
    """compute_grad_norm for a host that must not allocate: same kernels, scratch in a static device array of the
    library (partial sums of at most STATIC_NORM_MAX_CLUSTERS clusters). Calls on one device share that array and
    must not overlap on the GPU; the first call on a device does the one-time set-up."""
    out = C.c_double()
    check(lib().oxz_grad_norm_static(C.c_void_p(device_ptr), dtype, n, loss_scale, max_grad_value, clusters,
                                     C.c_void_p(stream) if stream else None, C.byref(out)))
    return out.value


# ------------------------------------------------------------------ the trainer's half of the step
@dataclass
class TrainerConfig:
    """The optimizer keys of oxidizr's TrainerConfig (src/config.rs:40-62, 641-727)."""
    learning_rate: float = 3e-4
    adamw_beta1: float = 0.9
    adamw_beta2: float = 0.95
    adamw_eps: float = 1e-6
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    target_grad_norm: float | None = None
    max_grad_value: float | None = None
    loss_scale: LossScaleConfig | None = None   # f16 runs only (src/loss_scale/config.rs:103-128)
    spike_guard: SpikeGuardConfig | None = None
    lr_schedule: str = "constant"
    warmup_steps: int = 0
    total_steps: int = 0
    min_lr_ratio: float = 0.0


class LitTrainerStep:
    """The post-accumulation half of LitTrainer::step_once (src/trainer.rs:515-695) over a :class:`DpOptimizer`.

    ``training_step(local_loss)`` expects this rank's summed micro-batch gradients in the optimizer's flat gradient
    buffer and returns ``(loss, grad_norm)`` exactly as the reference does.
    """

    def __init__(self, config: TrainerConfig, optimizer: DpOptimizer, start_step: int = 0):
        self.config = config
        self.optimizer = optimizer
        self.global_step = start_step
        self.lr_plan = LrPlan(config.learning_rate, config.lr_schedule, config.warmup_steps, config.total_steps,
                              config.min_lr_ratio)
        self.loss_scaler = LossScaler(config.loss_scale) if config.loss_scale is not None else None
        self.spike_guard = SpikeGuard(config.spike_guard) if config.spike_guard is not None else None
        self.loss_probe = None  # (index, loss) -> loss, the fault-injection hook of src/metrics/state.rs:10-14
        self.last_loss = None
        self.prev_grad_norm = None

    def optimizer_timestep(self) -> int:
        return self.optimizer.timestep

    def loss_scale_state(self) -> GradScalerState | None:
        return self.loss_scaler.state() if self.loss_scaler else None

    # -- the data-parallel hooks of src/dp/trainer_hooks.rs:36-107
    def with_communicator(self, comm: "Communicator", row_layout: "RowLayout") -> "LitTrainerStep":
        """Checks of LitTrainer::with_communicator: the rank is below the world size, and the world size is the row
        layout's (the layout of a loader built with this rank and world, so that steps count global batches)."""
        rank, world = comm.rank(), comm.world_size()
        if rank >= world:
            raise ValueError(f"communicator rank {rank} is not below its world size {world}. Pass a communicator of a valid group")
        if world != row_layout.world_size:
            raise ValueError(f"communicator world size {world} differs from the row layout's {row_layout.world_size}. Build "
                             f"the loader with LitDataLoader::with_rank(rank, {world}) and take its row layout")
        self.comm, self.row_layout = comm, row_layout
        return self

    def with_abort_hook(self, hook) -> "LitTrainerStep":
        self.abort_hook = hook
        return self

    def world_size(self) -> int:
        return self.optimizer.world

    def rank(self) -> int:
        return self.optimizer.rank

    def quiet(self) -> bool:
        """True on ranks other than 0: a quiet rank prints no diagnostic and writes no file."""
        return self.rank() != 0

    def abort_collectives(self) -> None:
        """Does nothing in a world of 1 or without a hook; after an abort every later collective of the group fails."""
        if self.world_size() > 1 and getattr(self, "abort_hook", None) is not None:
            self.abort_hook()

    def barrier(self) -> None:
        if self.world_size() <= 1:
            return
        try:
            self.optimizer.comm.barrier()
        except OxzError as e:
            raise OxzError(e.status, f"rank {self.rank()} barrier failed: {e.message}") from None

    # -- resume (src/trainer.rs:883-897, src/loss_scale/scaler.rs:123-153)
    def restore_loss_scale(self, saved: GradScalerState | None, start_step: int) -> str | None:
        """Both present: the run continues from ``saved``. A scaler without a saved state past step 0, or a saved state
        without a scaler: the returned warning says what was lost. A saved scale that is not finite and positive
        raises."""
        if self.loss_scaler is not None and saved is not None:
            self.loss_scaler.restore(saved)
            return None
        if self.loss_scaler is not None and start_step > 0:
            return (f"WARNING: the checkpoint records no loss scale state. The scale restarts at {self.loss_scaler.scale()}. "
                    "Training continues, but it does not match an uninterrupted run.")
        if saved is not None:
            return (f"WARNING: the checkpoint records loss scale {saved.scale}, but this run does not train in f16. "
                    "The loss scale state is dropped.")
        return None

    def checkpoint_meta(self, step: int, checkpoint_file: str, optimizer_file: str | None, decay: WeightDecaySpec,
                        position: DataPosition | None = None, mixture: "MixtureRecord | None" = None) -> "CheckpointMeta":
        """The keys this path contributes to a checkpoint's meta (src/checkpoint_set/snapshot.rs:245-262)."""
        layout = getattr(self, "row_layout", None)
        guard = SpikeGuardState(**self.spike_guard.state) if self.spike_guard is not None else None
        return CheckpointMeta(step=step, checkpoint_file=checkpoint_file, optimizer_file=optimizer_file, data_position=position,
                              weight_decay_rule=decay.rule, no_decay_patterns=list(decay.no_decay_patterns),
                              loss_scale=self.loss_scale_state(), world_size=self.world_size(),
                              global_batch_rows=layout.batch_size() if layout is not None else None, spike_guard=guard,
                              mixture=mixture)

    def training_step(self, local_loss: float, present: list[bool] | None = None) -> tuple[float, float]:
        opt = self.optimizer
        judged = self.spike_guard is not None or self.loss_probe is not None
        if opt.world > 1 and judged:
            # The guard judges the loss summed over ranks, so every rank decides alike (src/trainer.rs:611-612).
            # Its verdict must be known before the update is enqueued: one blocking 8-byte sum, as the reference's
            # step-weighting collective is (src/dp/weighting.rs:63-101).
            loss = opt.comm.sum_f64([local_loss])[0]
            extras = None
        elif opt.world > 1:
            loss, extras = None, [local_loss]  # the loss rides on the norm all-reduce
        else:
            loss, extras = local_loss, None
        spike_skip = False
        if judged:
            if self.loss_probe is not None:
                loss = self.loss_probe(self.global_step, loss)
            if self.spike_guard is not None:
                spike_skip = self.spike_guard.judge(self.global_step, loss)
        res = opt.step(self._cfg(spike_skip), present, extras)
        if loss is None:
            loss = opt.last_extras[0]
        overflow = bool(res.overflow)
        if self.loss_scaler is not None:
            self.loss_scaler.record_step(overflow, spike_skip)
        self.prev_grad_norm = res.reported_norm
        self.global_step += 1
        self.last_loss = loss
        return loss, res.reported_norm

    def _cfg(self, spike_skip: bool) -> StepConfig:
        c = self.config
        return StepConfig(
            lr=self.lr_plan.lr_at(self.global_step), beta1=c.adamw_beta1, beta2=c.adamw_beta2, eps=c.adamw_eps,
            weight_decay=c.weight_decay, max_grad_norm=c.max_grad_norm,
            max_grad_value=NAN if c.max_grad_value is None else c.max_grad_value,
            target_grad_norm=NAN if c.target_grad_norm is None else c.target_grad_norm,
            loss_scale=self.loss_scaler.scale() if self.loss_scaler else NAN, spike_skip=spike_skip)
