// Host-side decisions around the step, restated from the reference in C++: loss-scaler state machine,
// weight-decay rule, spike guard, learning-rate plan, row/rank arithmetic and step weighting. No GPU is touched.
#include <cmath>
#include <cstring>
#include <string>

#include <vector>

#include "oxz_internal.h"

using namespace oxz;

extern "C" {

// ---- loss scaler: src/loss_scale/config.rs:66-100, src/loss_scale/scaler.rs:19-51 ----

int32_t oxz_scaler_check(const oxz_scaler_config* c) {
    return oxz::guarded("oxz_scaler_check", [&]() -> int32_t {
        if (!c) return fail(OXZ_ERR_INVALID, "oxz_scaler_check: null config");
        auto bad = [](const char* key, double v, const char* rule) {
            return fail(OXZ_ERR_INVALID,
                        "trainer.loss_scale.%s is %g: it must be %s. Fix the value, or remove the key to use its default.",
                        key, v, rule);
        };
        if (!(std::isfinite(c->initial) && c->initial > 0.0)) return bad("initial", c->initial, "finite and positive");
        if (!(std::isfinite(c->growth_factor) && c->growth_factor > 1.0)) return bad("growth_factor", c->growth_factor, "finite and above 1");
        if (!(c->backoff_factor > 0.0 && c->backoff_factor < 1.0)) return bad("backoff_factor", c->backoff_factor, "above 0 and below 1");
        if (c->growth_interval == 0) return bad("growth_interval", 0.0, "at least 1");
        return OXZ_OK;
    });
}

int32_t oxz_scaler_init(const oxz_scaler_config* c, oxz_scaler_state* st) {
    return oxz::guarded("oxz_scaler_init", [&]() -> int32_t {
        if (!st) return fail(OXZ_ERR_INVALID, "oxz_scaler_init: null state");
        OXZ_TRY(oxz_scaler_check(c));
        st->scale = c->initial;
        st->consecutive_ok = 0;
        return OXZ_OK;
    });
}

int32_t oxz_scaler_restore(const oxz_scaler_state* saved, oxz_scaler_state* st) {
    return oxz::guarded("oxz_scaler_restore", [&]() -> int32_t {
        if (!saved || !st) return fail(OXZ_ERR_INVALID, "oxz_scaler_restore: null argument");
        if (!(std::isfinite(saved->scale) && saved->scale > 0.0))
            return fail(OXZ_ERR_INVALID, "the saved loss scale is %g: it must be finite and positive", saved->scale);
        *st = *saved;
        return OXZ_OK;
    });
}

int32_t oxz_scaler_record_step(const oxz_scaler_config* c, oxz_scaler_state* st, int32_t overflow, int32_t spike_skip) {
    return oxz::guarded("oxz_scaler_record_step", [&]() -> int32_t {
        if (!c || !st) return fail(OXZ_ERR_INVALID, "oxz_scaler_record_step: null argument");
        // A spike skip with finite gradients leaves the loss scale untouched (src/trainer.rs:666-670).
        if (!overflow && spike_skip) return OXZ_OK;
        if (overflow) {
            st->scale *= c->backoff_factor;
            st->consecutive_ok = 0;
        } else {
            st->consecutive_ok += 1;
            if (st->consecutive_ok >= c->growth_interval) {
                st->scale *= c->growth_factor;
                st->consecutive_ok = 0;
            }
        }
        return OXZ_OK;
    });
}

// ---- weight decay rule: src/weight_decay/rule.rs:78-118 ----

int32_t oxz_decay_check(int32_t rule, const char* const* patterns, uint32_t n) {
    return oxz::guarded("oxz_decay_check", [&]() -> int32_t {
        if (rule < OXZ_DECAY_ALL || rule > OXZ_SKIP_ALL) return fail(OXZ_ERR_INVALID, "unknown weight_decay_rule %d", rule);
        if (n && !patterns) return fail(OXZ_ERR_INVALID, "oxz_decay_check: null patterns");
        for (uint32_t i = 0; i < n; i++)
            if (!patterns[i] || patterns[i][0] == '\0')
                return fail(OXZ_ERR_INVALID,
                            "trainer.no_decay_patterns[%u] is empty, and an empty pattern matches every parameter. "
                            "Remove it, or set trainer.weight_decay_rule: skip_all.", i);
        if (n && rule != OXZ_SKIP_1D) {
            static const char* names[] = {"decay_all", "skip_1d", "skip_all"};
            return fail(OXZ_ERR_INVALID,
                        "trainer.no_decay_patterns needs weight_decay_rule skip_1d, but the rule is %s. Set "
                        "trainer.weight_decay_rule: skip_1d, or remove trainer.no_decay_patterns.", names[rule]);
        }
        return OXZ_OK;
    });
}

int32_t oxz_decay_excludes(int32_t rule, const char* const* patterns, uint32_t n, const char* name, uint32_t rank,
                           int32_t* excluded) {
    return oxz::guarded("oxz_decay_excludes", [&]() -> int32_t {
        if (!name || !excluded) return fail(OXZ_ERR_INVALID, "oxz_decay_excludes: null argument");
        if (rule < OXZ_DECAY_ALL || rule > OXZ_SKIP_ALL) return fail(OXZ_ERR_INVALID, "unknown weight_decay_rule %d", rule);
        if (rule == OXZ_DECAY_ALL) { *excluded = 0; return OXZ_OK; }
        if (rule == OXZ_SKIP_ALL) { *excluded = 1; return OXZ_OK; }
        const char* dot = strrchr(name, '.');
        const std::string last = dot ? dot + 1 : name;
        bool ex = rank < 2;
        if (!ex && last.size() >= 4 && last.compare(last.size() - 4, 4, "bias") == 0) ex = true;
        if (!ex) for (const char* ssm : {"a_log", "A_log", "d_param", "D"}) if (last == ssm) ex = true;
        if (!ex) for (uint32_t i = 0; i < n; i++) if (patterns[i] && strstr(name, patterns[i])) { ex = true; break; }
        *excluded = ex ? 1 : 0;
        return OXZ_OK;
    });
}

// ---- spike guard: src/metrics/spike.rs:124-168, src/metrics/state.rs:79-86 ----

int32_t oxz_spike_judge(const oxz_spike_config* c, oxz_spike_state* s, uint64_t index, double loss, int32_t* skip,
                        int32_t* flagged) {
    return oxz::guarded("oxz_spike_judge", [&]() -> int32_t {
        (void)index;
        if (!c || !s || !skip) return fail(OXZ_ERR_INVALID, "oxz_spike_judge: null argument");
        if (c->window == 0)
            return fail(OXZ_ERR_INVALID, "trainer.spike_guard.window is 0: the EMA span must be at least 1 step. Set a positive window.");
        if (!(std::isfinite(c->z_threshold) && c->z_threshold > 0.0))
            return fail(OXZ_ERR_INVALID, "trainer.spike_guard.z_threshold is %g: it must be a finite positive number. Set a positive threshold, such as 6.0.", c->z_threshold);
        *skip = 0;
        if (flagged) *flagged = 0;
        if (!std::isfinite(loss)) return OXZ_OK;
        const uint64_t warm = c->min_steps > 2 ? c->min_steps : 2;
        if (s->observed >= warm) {
            const double sd = std::sqrt(s->variance);
            if (loss > s->mean + c->z_threshold * sd) {
                s->detected += 1;
                if (!c->action_warn) {
                    s->skipped += 1;
                    *skip = 1;
                }
                if (flagged) *flagged = 1;
                return OXZ_OK;
            }
        }
        if (s->observed == 0) {
            s->mean = loss;
            s->variance = 0.0;
        } else {
            const double alpha = 2.0 / ((double)c->window + 1.0);
            const double diff = loss - s->mean;
            const double incr = alpha * diff;
            s->mean += incr;
            s->variance = (1.0 - alpha) * (s->variance + diff * incr);
        }
        s->observed += 1;
        return OXZ_OK;
    });
}

// ---- learning rate: src/schedule.rs:177-183 with the closed form of src/schedule.rs:284-321 ----

int32_t oxz_lr_at(const oxz_lr_plan* p, uint64_t step, double* lr) {
    return oxz::guarded("oxz_lr_at", [&]() -> int32_t {
        if (!p || !lr) return fail(OXZ_ERR_INVALID, "oxz_lr_at: null argument");
        if (p->schedule < OXZ_LR_CONSTANT || p->schedule > OXZ_LR_WSD) return fail(OXZ_ERR_INVALID, "unknown lr_schedule %d", p->schedule);
        if (!(p->min_lr_ratio >= 0.0 && p->min_lr_ratio <= 1.0))
            return fail(OXZ_ERR_INVALID, "trainer.min_lr_ratio (%g) must be between 0.0 and 1.0: it names the fraction of learning_rate the schedule decays to.", p->min_lr_ratio);
        if (p->schedule == OXZ_LR_WSD && p->warmup_steps + p->decay_steps > p->total_steps)
            return fail(OXZ_ERR_INVALID,
                        "lr_schedule: wsd needs %llu warmup steps plus %llu decay steps, but the run has %llu steps. "
                        "Lower trainer.decay_steps, trainer.decay_ratio or the warmup, or raise trainer.max_steps.",
                        (unsigned long long)p->warmup_steps, (unsigned long long)p->decay_steps, (unsigned long long)p->total_steps);
        if (p->warmup_steps > 0 && step < p->warmup_steps) {
            const double v = p->base_lr * ((double)(step + 1) / (double)p->warmup_steps);
            *lr = v > 1e-7 ? v : 1e-7;
            return OXZ_OK;
        }
        if (p->schedule == OXZ_LR_CONSTANT) { *lr = p->base_lr * 1.0; return OXZ_OK; }
        uint64_t stable, span;
        int shape;
        if (p->schedule == OXZ_LR_WSD) {
            stable = p->total_steps - p->decay_steps;
            span = p->decay_steps;
            shape = p->decay_shape;
        } else {
            shape = p->schedule == OXZ_LR_COSINE ? OXZ_SHAPE_COSINE : OXZ_SHAPE_LINEAR;
            if (p->total_steps > p->warmup_steps) { stable = p->warmup_steps; span = p->total_steps - p->warmup_steps; }
            else { stable = p->warmup_steps + 1; span = 0; }
        }
        if (span > 0 ? step <= stable : step < stable) { *lr = p->base_lr * 1.0; return OXZ_OK; }
        if (span == 0) { *lr = p->base_lr * p->min_lr_ratio; return OXZ_OK; }
        double progress = (double)(step - stable) / (double)span;
        if (progress > 1.0) progress = 1.0;
        double sh;
        if (shape == OXZ_SHAPE_COSINE) sh = 0.5 * (1.0 + std::cos(M_PI * progress));
        else if (shape == OXZ_SHAPE_LINEAR) sh = 1.0 - progress;
        else sh = 1.0 - std::sqrt(progress);
        *lr = p->base_lr * (p->min_lr_ratio + (1.0 - p->min_lr_ratio) * sh);
        return OXZ_OK;
    });
}

// ---- rows and ranks: src/data/rows.rs:66-191, src/data/positioning.rs:44-68, src/data/batch.rs:51-71 ----

int32_t oxz_rows_check(const oxz_row_layout* l) {
    return oxz::guarded("oxz_rows_check", [&]() -> int32_t {
        if (!l) return fail(OXZ_ERR_INVALID, "oxz_rows_check: null layout");
        if (l->rank_batch_size == 0)
            return fail(OXZ_ERR_DATA, "trainer.batch_size is 0: a batch needs at least one row. Set trainer.batch_size to a positive number.");
        if (l->world_size == 0)
            return fail(OXZ_ERR_DATA, "world size is 0: a run needs at least one rank. Pass a world size of 1 or more.");
        uint64_t global;
        if (__builtin_mul_overflow(l->rank_batch_size, l->world_size, &global))
            return fail(OXZ_ERR_DATA, "batch_size %llu x %llu ranks overflows a row count. Use a smaller trainer.batch_size or fewer ranks.",
                        (unsigned long long)l->rank_batch_size, (unsigned long long)l->world_size);
        if (l->num_rows < global) {
            if (l->world_size == 1)
                return fail(OXZ_ERR_DATA, "data shard holds %llu whole rows, fewer than batch_size %llu, so no batch fits. Use more data, a smaller trainer.batch_size, or a smaller model.max_seq_len.",
                            (unsigned long long)l->num_rows, (unsigned long long)l->rank_batch_size);
            return fail(OXZ_ERR_DATA, "data shard holds %llu whole rows, fewer than one global batch of %llu rows (batch_size %llu x %llu ranks), so no batch fits. Use more data, a smaller trainer.batch_size, fewer ranks, or a smaller model.max_seq_len.",
                        (unsigned long long)l->num_rows, (unsigned long long)global, (unsigned long long)l->rank_batch_size, (unsigned long long)l->world_size);
        }
        if (l->num_rows > 0xFFFFFFFFull)
            return fail(OXZ_ERR_DATA, "data shard holds %llu rows, more than the %u a row order can index. Split the data file.", (unsigned long long)l->num_rows, 0xFFFFFFFFu);
        return OXZ_OK;
    });
}

static oxz_data_position batch_start(const oxz_row_layout* l, oxz_data_position pos) {
    const uint64_t g = l->rank_batch_size * l->world_size;
    if (pos.row + g > l->num_rows) return oxz_data_position{pos.epoch + 1, 0};
    return pos;
}

int32_t oxz_rows_advance(const oxz_row_layout* l, oxz_data_position pos, uint64_t batches, oxz_data_position* out) {
    return oxz::guarded("oxz_rows_advance", [&]() -> int32_t {
        if (!out) return fail(OXZ_ERR_INVALID, "oxz_rows_advance: null argument");
        OXZ_TRY(oxz_rows_check(l));
        if (batches == 0) { *out = pos; return OXZ_OK; }
        const uint64_t g = l->rank_batch_size * l->world_size;
        const oxz_data_position start = batch_start(l, pos);
        const uint64_t left = (l->num_rows - start.row) / g;
        if (batches <= left) { *out = oxz_data_position{start.epoch, start.row + batches * g}; return OXZ_OK; }
        const uint64_t rest = batches - left, per = l->num_rows / g;
        *out = oxz_data_position{start.epoch + 1 + (rest - 1) / per, ((rest - 1) % per + 1) * g};
        return OXZ_OK;
    });
}

int32_t oxz_rows_next_window(const oxz_row_layout* l, oxz_data_position pos, uint64_t rank, uint64_t seq_len,
                             uint64_t first_row, const uint32_t* tokens, uint64_t n_tokens, uint64_t* rows,
                             int64_t* inputs, int64_t* targets, oxz_data_position* next) {
    return oxz::guarded("oxz_rows_next_window", [&]() -> int32_t {
        OXZ_TRY(oxz_rows_check(l));
        if (rank >= l->world_size)
            return fail(OXZ_ERR_DATA, "rank %llu is not below world size %llu. Pass a rank in [0, %llu).", (unsigned long long)rank,
                        (unsigned long long)l->world_size, (unsigned long long)l->world_size);
        if (pos.row > l->num_rows)
            return fail(OXZ_ERR_DATA, "data position epoch %llu row %llu is past this shard's %llu rows", (unsigned long long)pos.epoch,
                        (unsigned long long)pos.row, (unsigned long long)l->num_rows);
        const oxz_data_position start = batch_start(l, pos);
        const uint64_t B = l->rank_batch_size, width = seq_len + 1;
        const uint64_t first_slot = start.row + rank * B;
        for (uint64_t k = 0; k < B; k++) {
            const uint64_t row = first_row + first_slot + k;  // stream order: the row at slot i is row i
            if (rows) rows[k] = row;
            if (tokens) {
                if ((row + 1) * width > n_tokens)
                    return fail(OXZ_ERR_DATA, "row %llu lies past the %llu tokens of the stream", (unsigned long long)row, (unsigned long long)n_tokens);
                const uint32_t* src = tokens + row * width;
                for (uint64_t j = 0; j < seq_len; j++) {
                    if (inputs) inputs[k * seq_len + j] = (int64_t)src[j];
                    if (targets) targets[k * seq_len + j] = (int64_t)src[j + 1];
                }
            }
        }
        if (next) *next = oxz_data_position{start.epoch, start.row + B * l->world_size};
        return OXZ_OK;
    });
}

int32_t oxz_rows_batch_epoch(const oxz_row_layout* l, oxz_data_position pos, uint64_t* epoch) {
    return oxz::guarded("oxz_rows_batch_epoch", [&]() -> int32_t {
        if (!epoch) return fail(OXZ_ERR_INVALID, "oxz_rows_batch_epoch: null argument");
        OXZ_TRY(oxz_rows_check(l));
        if (pos.row > l->num_rows)
            return fail(OXZ_ERR_DATA, "data position epoch %llu row %llu is past this shard's %llu rows", (unsigned long long)pos.epoch,
                        (unsigned long long)pos.row, (unsigned long long)l->num_rows);
        *epoch = batch_start(l, pos).epoch;
        return OXZ_OK;
    });
}

int32_t oxz_rows_check_permutation(const uint32_t* perm, uint64_t n) {
    return oxz::guarded("oxz_rows_check_permutation", [&]() -> int32_t {
        if (!perm && n) return fail(OXZ_ERR_INVALID, "oxz_rows_check_permutation: null argument");
        std::vector<uint64_t> seen((n + 63) / 64, 0);
        for (uint64_t i = 0; i < n; i++) {
            const uint64_t v = perm[i];
            if (v >= n) return fail(OXZ_ERR_DATA, "the row order holds row %llu at slot %llu, past its %llu rows: it is not a permutation of 0..%llu", (unsigned long long)v, (unsigned long long)i, (unsigned long long)n, (unsigned long long)n);
            if (seen[v >> 6] & (1ull << (v & 63)))
                return fail(OXZ_ERR_DATA, "the row order holds row %llu twice (again at slot %llu): it is not a permutation of 0..%llu", (unsigned long long)v, (unsigned long long)i, (unsigned long long)n);
            seen[v >> 6] |= 1ull << (v & 63);
        }
        return OXZ_OK;
    });
}

int32_t oxz_rows_next_window_ordered(const oxz_row_layout* l, oxz_data_position pos, uint64_t rank, uint64_t seq_len,
                                     uint64_t first_row, const uint32_t* tokens, uint64_t n_tokens, uint64_t perm_epoch,
                                     const uint32_t* perm, uint64_t n_perm, uint64_t* rows, int64_t* inputs, int64_t* targets,
                                     oxz_data_position* next) {
    return oxz::guarded("oxz_rows_next_window_ordered", [&]() -> int32_t {
        if (!perm) return fail(OXZ_ERR_INVALID, "oxz_rows_next_window_ordered: null row order");
        OXZ_TRY(oxz_rows_check(l));
        if (n_perm != l->num_rows)
            return fail(OXZ_ERR_DATA, "the row order holds %llu rows and the layout %llu: pass the permutation of this layout's rows",
                        (unsigned long long)n_perm, (unsigned long long)l->num_rows);
        // the slots, by the stream-order arithmetic; then EpochOrder::row: the row at each slot (src/data/rows.rs:240-256)
        std::vector<uint64_t> slots(l->rank_batch_size);
        oxz_data_position after{};
        OXZ_TRY(oxz_rows_next_window(l, pos, rank, seq_len, 0, nullptr, 0, slots.data(), nullptr, nullptr, &after));
        if (after.epoch != perm_epoch)
            return fail(OXZ_ERR_DATA, "the next batch reads epoch %llu and the row order given is epoch %llu's: pass epoch_permutation(num_rows, seed, %llu)",
                        (unsigned long long)after.epoch, (unsigned long long)perm_epoch, (unsigned long long)after.epoch);
        const uint64_t width = seq_len + 1;
        for (uint64_t k = 0; k < l->rank_batch_size; k++) {
            const uint64_t shard_row = perm[slots[k]];
            if (shard_row >= l->num_rows)
                return fail(OXZ_ERR_DATA, "the row order holds row %llu at slot %llu, past its %llu rows: it is not a permutation", (unsigned long long)shard_row,
                            (unsigned long long)slots[k], (unsigned long long)l->num_rows);
            const uint64_t row = first_row + shard_row;
            if (rows) rows[k] = row;
            if (tokens) {
                if ((row + 1) * width > n_tokens)
                    return fail(OXZ_ERR_DATA, "row %llu lies past the %llu tokens of the stream", (unsigned long long)row, (unsigned long long)n_tokens);
                const uint32_t* src = tokens + row * width;
                for (uint64_t j = 0; j < seq_len; j++) {
                    if (inputs) inputs[k * seq_len + j] = (int64_t)src[j];
                    if (targets) targets[k * seq_len + j] = (int64_t)src[j + 1];
                }
            }
        }
        if (next) *next = after;
        return OXZ_OK;
    });
}

// ---- step weighting: src/dp/weighting.rs:46-61, src/step_loss.rs:79-112 ----

int32_t oxz_step_weighting(uint64_t local_micro_batches, int32_t world, const int64_t counts[2], uint64_t* micro_batches,
                           int64_t* global_scored) {
    return oxz::guarded("oxz_step_weighting", [&]() -> int32_t {
        if (!counts || !micro_batches || !global_scored) return fail(OXZ_ERR_INVALID, "oxz_step_weighting: null argument");
        if (world <= 0) return fail(OXZ_ERR_INVALID, "a data-parallel step needs at least one rank, got world size 0");
        uint64_t m;
        if (__builtin_mul_overflow(local_micro_batches, (uint64_t)world, &m))
            return fail(OXZ_ERR_INVALID, "%llu micro-batches times %d ranks overflows a count", (unsigned long long)local_micro_batches, world);
        if (counts[0] < 0 || counts[1] < 0)
            return fail(OXZ_ERR_NCCL, "a step count summed over %d ranks is %lld. Every rank must pass counts of 0 or more", world,
                        (long long)(counts[0] < 0 ? counts[0] : counts[1]));
        if (counts[1] != 0 && counts[1] != world)
            return fail(OXZ_ERR_INVALID,
                        "%lld of %d data-parallel ranks carry a loss mask in this step. Every rank must mask, or none. "
                        "Build every rank's loader from the same config", (long long)counts[1], world);
        *micro_batches = m;
        *global_scored = counts[1] == 0 ? -1 : counts[0];
        return OXZ_OK;
    });
}

}  // extern "C"
