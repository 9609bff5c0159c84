"""Python restatement of the host-side decisions around oxidizr's optimizer step.

Test infrastructure only (the checker for the C++ host logic in the product library):
loss-scaler state machine, weight-decay rule, spike guard, learning-rate plan, rank/slot
row arithmetic and step weighting. Every function cites the reference lines it follows.
All of these are pinned by known answers in the reference's own tests (tests/test_oracle_pins.py),
except the shuffled row permutation (rand 0.10.3 StdRng, un-vendored: not restated; stream order only).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field


# ---------------------------------------------------------------- loss scaler
@dataclass
class LossScaleConfig:
    """src/loss_scale/config.rs:28-41; defaults pinned at src/loss_scale/config.rs:134-235."""
    initial: float = 65536.0
    growth_factor: float = 2.0
    backoff_factor: float = 0.5
    growth_interval: int = 2000

    def check(self) -> None:
        """src/loss_scale/config.rs:70-100: the first key out of range is named."""
        def bad(key, value, rule):
            raise ValueError(f"trainer.loss_scale.{key} is {value}: it must be {rule}.")
        if not (math.isfinite(self.initial) and self.initial > 0.0):
            bad("initial", self.initial, "finite and positive")
        if not (math.isfinite(self.growth_factor) and self.growth_factor > 1.0):
            bad("growth_factor", self.growth_factor, "finite and above 1")
        if not (0.0 < self.backoff_factor < 1.0):
            bad("backoff_factor", self.backoff_factor, "above 0 and below 1")
        if self.growth_interval == 0:
            bad("growth_interval", 0, "at least 1")


@dataclass
class GradScalerState:
    scale: float
    consecutive_ok: int = 0


class LossScaler:
    """src/loss_scale/scaler.rs:13-51 over boostr GradScaler::update_scale.

    Known answers: src/loss_scale/scaler.rs:275-289 (64 -> 32 -> 32 -> 64 at interval 2) and
    tests/loss_scale.rs:180-214 ((64,1),(128,0),(128,1),(256,0)).
    """

    def __init__(self, config: LossScaleConfig | None = None):
        self.config = config or LossScaleConfig()
        self.config.check()
        self._state = GradScalerState(self.config.initial, 0)

    def scale(self) -> float:
        return self._state.scale

    def state(self) -> GradScalerState:
        return GradScalerState(self._state.scale, self._state.consecutive_ok)

    def restore(self, state: GradScalerState) -> None:
        """src/loss_scale/scaler.rs:30-37: a scale that is not finite and positive is an error."""
        if not (math.isfinite(state.scale) and state.scale > 0.0):
            raise ValueError(f"loss scale {state.scale} is not finite and positive")
        self._state = GradScalerState(state.scale, state.consecutive_ok)

    def record_step(self, overflow: bool) -> None:
        s = self._state
        if overflow:
            s.scale *= self.config.backoff_factor
            s.consecutive_ok = 0
        else:
            s.consecutive_ok += 1
            if s.consecutive_ok >= self.config.growth_interval:
                s.scale *= self.config.growth_factor
                s.consecutive_ok = 0


def record_after_step(scaler: LossScaler | None, overflow: bool, spike_skip: bool) -> None:
    """src/trainer.rs:666-681: a spike skip with finite gradients leaves the scale untouched."""
    if scaler is not None and (overflow or not spike_skip):
        scaler.record_step(overflow)


# ---------------------------------------------------------------- weight decay rule
SSM_NO_DECAY = ("a_log", "A_log", "d_param", "D")  # src/weight_decay/rule.rs:46


@dataclass
class WeightDecaySpec:
    """src/weight_decay/rule.rs:49-118."""
    rule: str = "skip_1d"  # decay_all | skip_1d | skip_all ; fresh default src/weight_decay/rule.rs:26
    no_decay_patterns: list[str] = field(default_factory=list)

    def check(self) -> None:
        """src/weight_decay/rule.rs:78-100."""
        for i, p in enumerate(self.no_decay_patterns):
            if p == "":
                raise ValueError(f"trainer.no_decay_patterns[{i}] is empty")
        if self.no_decay_patterns and self.rule != "skip_1d":
            raise ValueError(f"trainer.no_decay_patterns needs weight_decay_rule skip_1d, but the rule is {self.rule}")

    def excludes(self, name: str, rank: int) -> bool:
        """src/weight_decay/rule.rs:103-118; golden names at :142-176."""
        if self.rule == "decay_all":
            return False
        if self.rule == "skip_all":
            return True
        last = name.rsplit(".", 1)[-1]
        return (rank < 2 or last.endswith("bias") or last in SSM_NO_DECAY
                or any(p in name for p in self.no_decay_patterns))


def decay_plan(spec: WeightDecaySpec, tensors: list[tuple[int, str, int, int]]):
    """src/weight_decay/plan.rs:41-60: (id, name, rank, elements); a repeated id counts once.

    Returns (no_decay ids, decay tensors, decay elements, no-decay elements); the single
    param group is {ids: no_decay, lr_scale 1.0, weight_decay 0.0} (src/weight_decay/plan.rs:113-122).
    """
    seen, no_decay = set(), set()
    decay_tensors = decay_elements = no_decay_elements = 0
    for tid, name, rank, elements in tensors:
        if tid in seen:
            continue
        seen.add(tid)
        if spec.excludes(name, rank):
            no_decay.add(tid)
            no_decay_elements += elements
        else:
            decay_tensors += 1
            decay_elements += elements
    return no_decay, decay_tensors, decay_elements, no_decay_elements


# ---------------------------------------------------------------- spike guard
@dataclass
class SpikeGuardConfig:
    """src/metrics/config.rs:69-115."""
    window: int = 100
    z_threshold: float = 6.0
    min_steps: int = 50
    action: str = "skip"  # skip | warn

    def alpha(self) -> float:
        return 2.0 / (float(self.window) + 1.0)

    def warmup_losses(self) -> int:
        return max(self.min_steps, 2)


@dataclass
class SpikeGuardState:
    mean: float = 0.0
    variance: float = 0.0
    observed: int = 0
    detected: int = 0
    skipped: int = 0


class SpikeGuard:
    """src/metrics/spike.rs:72-168; hand-computed EMA at :204-217, skip list at src/metrics/state.rs:122-152."""

    def __init__(self, config: SpikeGuardConfig):
        if config.window == 0:
            raise ValueError("trainer.spike_guard.window is 0")
        if not (math.isfinite(config.z_threshold) and config.z_threshold > 0.0):
            raise ValueError(f"trainer.spike_guard.z_threshold is {config.z_threshold}")
        self.config = config
        self.state = SpikeGuardState()

    def observe(self, step: int, loss: float):
        """Returns (mean, std) of a flagged step, else None."""
        if not math.isfinite(loss):
            return None
        s = self.state
        if s.observed >= self.config.warmup_losses():
            std = math.sqrt(s.variance)
            if loss > s.mean + self.config.z_threshold * std:
                s.detected += 1
                if self.config.action == "skip":
                    s.skipped += 1
                return (s.mean, std)
        if s.observed == 0:
            s.mean, s.variance = loss, 0.0
        else:
            a = self.config.alpha()
            diff = loss - s.mean
            incr = a * diff
            s.mean += incr
            s.variance = (1.0 - a) * (s.variance + diff * incr)
        s.observed += 1
        return None

    def judge(self, index: int, loss: float) -> bool:
        """src/metrics/state.rs:79-86: true when the 0-based step `index` must skip the optimizer."""
        return self.observe(index + 1, loss) is not None and self.config.action == "skip"


# ---------------------------------------------------------------- learning rate
MIN_WARMUP_LR = 1e-7  # src/schedule.rs:18


def lr_at(step: int, base_lr: float, schedule: str, warmup_steps: int, total_steps: int, min_lr_ratio: float,
          decay_steps: int | None = None, decay_shape: str = "linear") -> float:
    """src/schedule.rs:177-183 with the in-file closed form of src/schedule.rs:284-321.

    `schedule` is constant | cosine | linear | wsd. For wsd, `decay_steps` is the resolved span
    (src/schedule.rs:124-132) and the decay runs over the last `decay_steps` steps of the run.
    """
    if warmup_steps > 0 and step < warmup_steps:
        return max(base_lr * (float(step + 1) / float(warmup_steps)), MIN_WARMUP_LR)
    if schedule == "constant":
        return base_lr * 1.0
    if schedule == "wsd":
        stable, span, shape_kind = total_steps - decay_steps, decay_steps, decay_shape
    else:
        shape_kind = schedule
        if total_steps > warmup_steps:
            stable, span = warmup_steps, total_steps - warmup_steps
        else:
            stable, span = warmup_steps + 1, 0
    if (step <= stable) if span > 0 else (step < stable):
        return base_lr * 1.0
    if span == 0:
        return base_lr * min_lr_ratio
    progress = min(float(step - stable) / float(span), 1.0)
    if shape_kind == "cosine":
        shape = 0.5 * (1.0 + math.cos(math.pi * progress))
    elif shape_kind == "linear":
        shape = 1.0 - progress
    else:  # sqrt
        shape = 1.0 - math.sqrt(progress)
    return base_lr * (min_lr_ratio + (1.0 - min_lr_ratio) * shape)


def wsd_decay_steps(total_steps: int, decay_steps: int | None, decay_ratio: float | None) -> int:
    """src/schedule.rs:124-132; DEFAULT_DECAY_RATIO 0.1 at :14."""
    if decay_steps is not None:
        return decay_steps
    return int(math.ceil(float(total_steps) * (0.1 if decay_ratio is None else decay_ratio)))


# ---------------------------------------------------------------- rows and ranks
@dataclass(frozen=True)
class DataPosition:
    """src/data/rows.rs:29-35."""
    epoch: int = 0
    row: int = 0


class RowLayout:
    """src/data/rows.rs:53-208."""

    def __init__(self, num_rows: int, rank_batch_size: int, world_size: int = 1):
        if rank_batch_size == 0:
            raise ValueError("trainer.batch_size is 0")
        if world_size == 0:
            raise ValueError("world size is 0")
        g = rank_batch_size * world_size
        if g >= 1 << 64:
            raise ValueError("overflows a row count")
        if num_rows < g:
            if world_size == 1:
                raise ValueError(f"data shard holds {num_rows} whole rows, fewer than batch_size {rank_batch_size}")
            raise ValueError(f"data shard holds {num_rows} whole rows, fewer than one global batch of {g} rows "
                             f"(batch_size {rank_batch_size} x {world_size} ranks)")
        if num_rows > 0xFFFFFFFF:
            raise ValueError("more rows than a row order can index")
        self.num_rows, self.rank_batch_size, self.world_size = num_rows, rank_batch_size, world_size

    def batch_size(self) -> int:
        return self.rank_batch_size * self.world_size

    def batches_per_epoch(self) -> int:
        return self.num_rows // self.batch_size()

    def batch_start(self, pos: DataPosition) -> DataPosition:
        if pos.row + self.batch_size() > self.num_rows:
            return DataPosition(pos.epoch + 1, 0)
        return pos

    def advance(self, pos: DataPosition, batches: int) -> DataPosition:
        if batches == 0:
            return pos
        start = self.batch_start(pos)
        left = (self.num_rows - start.row) // self.batch_size()
        if batches <= left:
            return DataPosition(start.epoch, start.row + batches * self.batch_size())
        rest = batches - left
        per = self.batches_per_epoch()
        return DataPosition(start.epoch + 1 + (rest - 1) // per, ((rest - 1) % per + 1) * self.batch_size())

    def total_steps(self, grad_accum: int, num_epochs: int) -> int:
        return self.batches_per_epoch() * num_epochs // max(grad_accum, 1)

    def position_after_steps(self, steps: int, grad_accum: int) -> DataPosition:
        return self.advance(DataPosition(), steps * grad_accum)


def rank_window(layout: RowLayout, pos: DataPosition, rank: int, seq_len: int, first_row: int = 0, order=None):
    """One rank's draw of the next global batch, in stream order or, with `order`, in the reference's shuffled order.

    order: a callable epoch -> permutation of range(num_rows), standing for epoch_permutation(num_rows, seed, epoch)
    (src/data/rows.rs:258-263: rand 0.10.3's StdRng + SliceRandom::shuffle, un-vendored, so the VALUES of the
    reference's permutations are not restated; what is restated is EpochOrder::row, src/data/rows.rs:240-256: the
    row at `slot` of `epoch` is perm(epoch)[slot], asked for the epoch of layout.batch_start(pos)).

    src/data/positioning.rs:44-68 (slots [start.row + rank*B, +B)), src/data/rows.rs:243-246 (stream order:
    row = slot), src/data/row_ranges.rs:100-106 (one range: first_row + row), src/data/rows.rs:4-7
    (row r is tokens [r*(S+1), (r+1)*(S+1))), src/data/batch.rs:51-71 (inputs [0,S), targets [1,S+1)).
    Returns (rows, input token indices, target token indices, next position).
    """
    if rank >= layout.world_size:
        raise ValueError(f"rank {rank} is not below world size {layout.world_size}")
    start = layout.batch_start(pos)
    width = seq_len + 1
    first = start.row + rank * layout.rank_batch_size
    slots = range(first, first + layout.rank_batch_size)
    if order is None:
        rows = [first_row + slot for slot in slots]
    else:
        perm = order(start.epoch)
        rows = [first_row + int(perm[slot]) for slot in slots]
    inputs = [[r * width + j for j in range(seq_len)] for r in rows]
    targets = [[r * width + j + 1 for j in range(seq_len)] for r in rows]
    return rows, inputs, targets, DataPosition(start.epoch, start.row + layout.batch_size())


class RowRanges:
    """Ascending, disjoint, non-empty global row ranges (src/data/row_ranges.rs:9-106): loader row r is the r-th row
    across the ranges in order."""

    def __init__(self, spans, total: int):
        if not spans:
            raise ValueError("an empty list of row ranges reads no rows. Pass at least one range.")
        self.spans, self.before, self.len = list(spans), [], 0
        prev_end = 0
        for i, (start, end) in enumerate(spans):
            if start >= end or end > total:
                raise ValueError(f"row range [{start}, {end}) is not a non-empty range inside the {total} whole rows of "
                                 f"this data. Pick a range inside [0, {total}).")
            if i > 0 and start < prev_end:
                raise ValueError(f"row range [{start}, {end}) starts before row {prev_end}, the end of the range before "
                                 "it. Pass ranges in ascending order without overlap.")
            self.before.append(self.len)
            self.len += end - start
            prev_end = end

    def global_row(self, row: int) -> int:
        index = max(sum(1 for b in self.before if b <= row) - 1, 0)
        return self.spans[index][0] + (row - self.before[index])


def store_row(sources, width: int, global_row: int):
    """RowStore::row over in-memory sources (src/data/source.rs:96-158): each source keeps its own whole rows of
    `width` tokens and drops its own tail; global rows count from the start of source 0."""
    first = 0
    for tokens in sources:
        rows = len(tokens) // width
        if global_row < first + rows:
            at = (global_row - first) * width
            return list(tokens[at:at + width])
        first += rows
    raise IndexError(f"row {global_row} is past the {first} whole rows of this data")


# ---------------------------------------------------------------- weighted mixture of sources, stream order
def mixture_quotas(weights, rows: int):
    """Rows of one epoch per source by largest remainder, lower index first on a tie (src/data/mixture/quota.rs:22-57)."""
    total = sum(weights)
    shares = [w / total * rows for w in weights]
    counts = [min(int(math.floor(s)), rows) for s in shares]
    order = sorted(range(len(weights)), key=lambda i: (-(shares[i] - math.floor(shares[i])), i))
    assigned = sum(counts)
    if assigned <= rows:
        for k in range(rows - assigned):
            counts[order[k % len(order)]] += 1
    else:
        excess, k = assigned - rows, 0
        back = order[::-1]
        while excess:
            i = back[k % len(back)]
            if counts[i] > 0:
                counts[i] -= 1
                excess -= 1
            k += 1
    return counts


def mixture_round_robin(quotas):
    """Smooth weighted round-robin over the quotas: the source of each slot of an epoch in stream order, the same
    every epoch (src/data/mixture/schedule.rs:103-122)."""
    total = sum(quotas)
    credit = [0] * len(quotas)
    out = []
    for _ in range(total):
        pick = 0
        for i, q in enumerate(quotas):
            credit[i] += q
            if credit[i] > credit[pick]:
                pick = i
        credit[pick] -= total
        out.append(pick)
    return out


class Mixture:
    """A weighted mixture as a virtual row order, stream order (src/data/mixture/state.rs:33-178, draw.rs:44-62):
    slot s of epoch e belongs to source i = schedule[s]; it is that source's draw e * quota_i + (slots of i before s),
    and draw k of a source of n rows reads its row k % n."""

    def __init__(self, weights, rows_per_epoch, source_rows: list):
        if len(weights) != len(source_rows):
            raise ValueError(f"trainer.data.sources sets {len(weights)} weight(s), and the loader reads "
                             f"{len(source_rows)} source(s).")
        for i, (w, rows) in enumerate(zip(weights, source_rows)):
            if not (math.isfinite(w) and w > 0.0):
                raise ValueError(f"trainer.data.sources[{i}].weight is {w}: a weight must be a finite number above 0.")
            if rows is None or rows.len == 0:
                raise ValueError(f"trainer.data.sources[{i}] holds no training rows, and its weight {w} asks for rows.")
        total = sum(r.len for r in source_rows)
        rows = rows_per_epoch if rows_per_epoch is not None else total
        if rows == 0 or rows > (1 << 28):
            raise ValueError(f"trainer.data.rows_per_epoch is {rows}: an epoch needs at least 1 row and at most "
                             f"{1 << 28} rows")
        self.rows_per_epoch = rows
        self.quotas = mixture_quotas(weights, rows)
        self.sources = source_rows
        self.schedule = mixture_round_robin(self.quotas)

    def global_row(self, epoch: int, slot: int) -> int:
        source = self.schedule[slot]
        before = sum(1 for s in self.schedule[:slot] if s == source)
        draw = epoch * self.quotas[source] + before
        return self.sources[source].global_row(draw % self.sources[source].len)


def source_train_rows(source_rows, spans, total):
    """The training rows of each source: the loader's ranges cut at the source's bounds (src/data/mixture/loader.rs:60-84).
    None for a source without training rows."""
    out, first = [], 0
    for rows in source_rows:
        end = first + rows
        inside = [(max(a, first), min(b, end)) for a, b in spans if max(a, first) < min(b, end)]
        out.append(RowRanges(inside, total) if inside else None)
        first = end
    return out


# ---------------------------------------------------------------- loss mask and document segments of one window
def build_target_mask(window, batch_size: int, seq_len: int, target_base: int, always_score=()):
    """TargetMask::PrefixLm over a raw [batch_size, seq_len + 1] window (src/data/mask.rs:36-47, 72-88): position
    (b, s) scores iff its TARGET window[b*(S+1) + s + 1] is at least target_base or is listed in always_score."""
    out = []
    for b in range(batch_size):
        row = b * (seq_len + 1)
        for s in range(seq_len):
            t = window[row + s + 1]
            out.append(1.0 if (t >= target_base or t in always_score) else 0.0)
    return out


def host_segments(window, batch_size: int, seq_len: int, separator: int):
    """HostSegments::build (src/data/segments.rs:62-101): (offsets, ids) over the flattened inputs. A separator ends
    its segment and belongs to it; every row start begins a segment; a row ending on a separator adds no empty one."""
    if batch_size * seq_len > 2**31 - 1:
        raise ValueError(f"a batch of {batch_size} x {seq_len} tokens overflows the i32 segment offsets. "
                         "Lower trainer.batch_size or model.max_seq_len.")
    offsets, ids = [0], []
    for b in range(batch_size):
        row = window[b * (seq_len + 1): b * (seq_len + 1) + seq_len]
        for s, token in enumerate(row):
            ids.append(len(offsets) - 1)
            if token == separator:
                offsets.append(b * seq_len + s + 1)
        if offsets[-1] != (b + 1) * seq_len:
            offsets.append((b + 1) * seq_len)
    return offsets, ids


def host_masks(window, batch_size: int, seq_len: int, target_mask=None, separator=None):
    """LitDataLoader::host_masks (src/data/host_masks.rs:49-77). target_mask = (target_base, always_score) or None;
    separator = the document mask's separator id or None. Returns (loss_mask or None, scored, (offsets, ids) or None):
    the target mask scores by target id, the document mask clears every position whose INPUT is the separator."""
    target = build_target_mask(window, batch_size, seq_len, *target_mask) if target_mask is not None else None
    if separator is None:
        scored = batch_size * seq_len if target is None else sum(1 for m in target if m != 0.0)
        return target, scored, None
    mask = target if target is not None else [1.0] * (batch_size * seq_len)
    for b in range(batch_size):
        for s in range(seq_len):
            if window[b * (seq_len + 1) + s] == separator:
                mask[b * seq_len + s] = 0.0
    return mask, sum(1 for m in mask if m != 0.0), host_segments(window, batch_size, seq_len, separator)


# ---------------------------------------------------------------- step weighting
def reduce_step_weighting(local: list[tuple[int, int | None]]):
    """src/dp/weighting.rs:32-61 over src/step_loss.rs:79-112.

    local[r] = (micro_batches, total_scored or None) of rank r. Returns the per-rank result:
    (micro_batches * world, global scored or None); mixed masks raise on every rank.
    """
    world = len(local)
    if world <= 1:
        return list(local)
    scored = sum(s if s is not None else 0 for _, s in local)
    masked = sum(1 for _, s in local if s is not None)
    if masked not in (0, world):
        raise ValueError(f"{masked} of {world} data-parallel ranks carry a loss mask in this step")
    return [(mb * world, scored if masked else None) for mb, _ in local]
