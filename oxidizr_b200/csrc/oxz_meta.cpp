// The keys of a checkpoint meta (`checkpoint_step_N.meta.json`, CheckpointMeta of src/config.rs:1223-1302) that the
// optimizer path writes and reads around a resume: world_size and global_batch_rows (src/dp/resume.rs:19-55),
// loss_scale (src/loss_scale/resume.rs:14-29), weight_decay_rule and no_decay_patterns
// (src/weight_decay/rule.rs:68-74), data_position, spike_guard and optimizer_file (src/checkpoint_set/snapshot.rs:245-262).
// Host only. The file is JSON as serde_json writes it; keys this module does not know are skipped on load.
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "oxz_internal.h"
#include "oxz_json.h"

using namespace oxz;

namespace {

struct Parsed {
    oxz_resume_meta m{};
    std::vector<std::string> patterns;
    std::vector<double> mixture_weights;  // MixtureRecord::weights
};

int32_t rule_of(const std::string& s) {
    if (s == "decay_all") return OXZ_DECAY_ALL;
    if (s == "skip_1d") return OXZ_SKIP_1D;
    if (s == "skip_all") return OXZ_SKIP_ALL;
    return -1;
}
const char* rule_name(int32_t r) { return r == OXZ_DECAY_ALL ? "decay_all" : r == OXZ_SKIP_1D ? "skip_1d" : "skip_all"; }

// Reads the file; on failure `why` says what went wrong (the caller words the error the way its reference does).
bool parse_file(const char* path, Parsed* out, std::string* why) {
    FILE* f = fopen(path, "rb");
    if (!f) { *why = strerror(errno); return false; }
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof buf, f)) > 0) text.append(buf, n);
    fclose(f);
    JsonReader r{text.data(), text.data() + text.size()};
    oxz_resume_meta& m = out->m;
    m = oxz_resume_meta{};
    m.weight_decay_rule = OXZ_DECAY_ALL;  // WeightDecayRule::LEGACY for a meta without the key
    bool has_step = false;
    auto copy = [&](char* dst, size_t cap, const std::string& s) {
        if (s.size() >= cap) { r.ok = false; *why = "a file name in the meta is longer than " + std::to_string(cap - 1) + " bytes"; return; }
        memcpy(dst, s.c_str(), s.size() + 1);
    };
    r.object([&](const std::string& key) {
        if (r.word("null")) return;  // Option::None written explicitly
        if (key == "step") { has_step = r.u64(&m.step); }
        else if (key == "world_size") { m.has_world_size = r.u64(&m.world_size) ? 1 : 0; }
        else if (key == "global_batch_rows") { m.has_global_batch_rows = r.u64(&m.global_batch_rows) ? 1 : 0; }
        else if (key == "weight_decay_rule") {
            const int32_t rule = rule_of(r.str());
            if (rule < 0) { r.ok = false; *why = "unknown weight_decay_rule"; }
            else { m.weight_decay_rule = rule; m.has_weight_decay_rule = 1; }
        } else if (key == "no_decay_patterns") {
            if (!r.eat('[')) { r.ok = false; return; }
            if (!r.eat(']')) {
                do { out->patterns.push_back(r.str()); } while (r.ok && r.eat(','));
                if (!r.eat(']')) r.ok = false;
            }
        } else if (key == "loss_scale") {
            bool a = false, b = false;
            r.object([&](const std::string& k) {
                if (k == "scale") a = r.f64(&m.loss_scale.scale);
                else if (k == "consecutive_ok") b = r.u64(&m.loss_scale.consecutive_ok);
                else r.skip();
            });
            if (r.ok && !(a && b)) { r.ok = false; *why = "loss_scale needs `scale` and `consecutive_ok`"; }
            m.has_loss_scale = 1;
        } else if (key == "data_position") {
            bool a = false, b = false;
            r.object([&](const std::string& k) {
                if (k == "epoch") a = r.u64(&m.data_position.epoch);
                else if (k == "row") b = r.u64(&m.data_position.row);
                else r.skip();
            });
            if (r.ok && !(a && b)) { r.ok = false; *why = "data_position needs `epoch` and `row`"; }
            m.has_data_position = 1;
        } else if (key == "spike_guard") {
            r.object([&](const std::string& k) {
                if (k == "mean") r.f64(&m.spike_guard.mean);
                else if (k == "variance") r.f64(&m.spike_guard.variance);
                else if (k == "observed") r.u64(&m.spike_guard.observed);
                else if (k == "detected") r.u64(&m.spike_guard.detected);
                else if (k == "skipped") r.u64(&m.spike_guard.skipped);
                else r.skip();
            });
            m.has_spike_guard = 1;
        } else if (key == "mixture") {
            bool a = false, b = false;
            r.object([&](const std::string& k) {
                if (k == "weights") {
                    if (!r.eat('[')) { r.ok = false; return; }
                    if (!r.eat(']')) {
                        do { double w = 0.0; r.f64(&w); out->mixture_weights.push_back(w); } while (r.ok && r.eat(','));
                        if (!r.eat(']')) r.ok = false;
                    }
                    a = r.ok;
                } else if (k == "rows_per_epoch") b = r.u64(&m.mixture_rows_per_epoch);
                else r.skip();
            });
            if (r.ok && !(a && b)) { r.ok = false; *why = "mixture needs `weights` and `rows_per_epoch`"; }
            m.has_mixture = 1;
        } else if (key == "optimizer_file") { copy(m.optimizer_file, sizeof m.optimizer_file, r.str()); }
        else if (key == "checkpoint_file") { copy(m.checkpoint_file, sizeof m.checkpoint_file, r.str()); }
        else r.skip();
    });
    r.ws();
    if (r.ok && r.p != r.e) r.ok = false;
    if (r.ok && !has_step) { r.ok = false; *why = "missing field `step`"; }
    if (!r.ok) {
        if (why->empty()) *why = "the file is not valid JSON near byte " + std::to_string((size_t)(r.p - text.data()));
        return false;
    }
    m.n_no_decay_patterns = (uint32_t)out->patterns.size();
    m.n_mixture_weights = (uint32_t)out->mixture_weights.size();
    return true;
}

std::string esc(const std::string& s) {
    std::string out;
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') { out += '\\'; out += (char)c; }
        else if (c == '\n') out += "\\n";
        else if (c == '\t') out += "\\t";
        else if (c == '\r') out += "\\r";
        else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); out += b; }
        else out += (char)c;
    }
    return out;
}

// The shortest decimal text that reads back to the same f64 bits.
std::string f64_text(double v) {
    char b[40];
    for (int prec = 1; prec <= 17; prec++) {
        snprintf(b, sizeof b, "%.*g", prec, v);
        if (strtod(b, nullptr) == v) break;
    }
    std::string s = b;
    if (s.find_first_of(".eEn") == std::string::npos) s += ".0";  // serde_json keeps a float a float
    return s;
}

}  // namespace

extern "C" {

int32_t oxz_meta_load(const char* path, oxz_resume_meta* out) {
    return oxz::guarded("oxz_meta_load", [&]() -> int32_t {
        if (!path || !out) return fail(OXZ_ERR_INVALID, "oxz_meta_load: null argument");
        Parsed p;
        std::string why;
        if (!parse_file(path, &p, &why))
            return fail(OXZ_ERR_INVALID, "checkpoint meta '%s' was not read: %s. Restore the file to resume from it.", path, why.c_str());
        *out = p.m;
        return OXZ_OK;
    });
}

int32_t oxz_meta_no_decay_pattern(const char* path, uint32_t index, char* buf, uint64_t cap) {
    return oxz::guarded("oxz_meta_no_decay_pattern", [&]() -> int32_t {
        if (!path || !buf || cap == 0) return fail(OXZ_ERR_INVALID, "oxz_meta_no_decay_pattern: null argument");
        Parsed p;
        std::string why;
        if (!parse_file(path, &p, &why))
            return fail(OXZ_ERR_INVALID, "checkpoint meta '%s' was not read: %s. Restore the file to resume from it.", path, why.c_str());
        if (index >= p.patterns.size())
            return fail(OXZ_ERR_INVALID, "oxz_meta_no_decay_pattern: pattern %u of %zu", index, p.patterns.size());
        if (p.patterns[index].size() >= cap)
            return fail(OXZ_ERR_INVALID, "oxz_meta_no_decay_pattern: the pattern needs %zu bytes, the buffer has %llu",
                        p.patterns[index].size() + 1, (unsigned long long)cap);
        memcpy(buf, p.patterns[index].c_str(), p.patterns[index].size() + 1);
        return OXZ_OK;
    });
}

int32_t oxz_meta_mixture_weights(const char* path, double* weights, uint32_t cap, uint32_t* n_weights) {
    return oxz::guarded("oxz_meta_mixture_weights", [&]() -> int32_t {
        if (!path || !n_weights) return fail(OXZ_ERR_INVALID, "oxz_meta_mixture_weights: null argument");
        Parsed p;
        std::string why;
        if (!parse_file(path, &p, &why))
            return fail(OXZ_ERR_INVALID, "checkpoint meta '%s' was not read: %s. Restore the file to resume from it.", path, why.c_str());
        *n_weights = (uint32_t)p.mixture_weights.size();
        for (uint32_t i = 0; weights && i < cap && i < *n_weights; i++) weights[i] = p.mixture_weights[i];
        return OXZ_OK;
    });
}

int32_t oxz_meta_save(const char* path, const oxz_resume_meta* m, const char* const* no_decay_patterns,
                      const double* mixture_weights) {
    return oxz::guarded("oxz_meta_save", [&]() -> int32_t {
        if (!path || !m || (m->n_no_decay_patterns && !no_decay_patterns) || (m->has_mixture && m->n_mixture_weights && !mixture_weights))
            return fail(OXZ_ERR_INVALID, "oxz_meta_save: null argument");
        if (m->has_weight_decay_rule && (m->weight_decay_rule < OXZ_DECAY_ALL || m->weight_decay_rule > OXZ_SKIP_ALL))
            return fail(OXZ_ERR_INVALID, "oxz_meta_save: unknown weight decay rule %d", m->weight_decay_rule);
        if (m->has_loss_scale && !(std::isfinite(m->loss_scale.scale) && m->loss_scale.scale > 0.0))
            return fail(OXZ_ERR_INVALID, "oxz_meta_save: loss scale %g must be finite and positive", m->loss_scale.scale);
        // Field order and Option handling follow CheckpointMeta's serde derive: required keys first, None left out.
        // The keys outside the optimizer path (timestamp, hashes, data sources) are written empty.
        std::string j = "{\n";
        j += "  \"step\": " + std::to_string(m->step) + ",\n";
        j += "  \"timestamp\": \"\",\n  \"model_config_hash\": \"\",\n  \"data_file_path\": \"\",\n  \"data_file_hash\": \"\",\n";
        j += "  \"checkpoint_file\": \"" + esc(m->checkpoint_file) + "\"";
        if (m->has_data_position)
            j += ",\n  \"data_position\": {\n    \"epoch\": " + std::to_string(m->data_position.epoch) + ",\n    \"row\": " +
                 std::to_string(m->data_position.row) + "\n  }";
        if (m->optimizer_file[0]) j += ",\n  \"optimizer_file\": \"" + esc(m->optimizer_file) + "\"";
        if (m->has_weight_decay_rule) j += std::string(",\n  \"weight_decay_rule\": \"") + rule_name(m->weight_decay_rule) + "\"";
        if (m->n_no_decay_patterns) {
            j += ",\n  \"no_decay_patterns\": [";
            for (uint32_t i = 0; i < m->n_no_decay_patterns; i++) {
                if (!no_decay_patterns[i]) return fail(OXZ_ERR_INVALID, "oxz_meta_save: pattern %u is null", i);
                j += std::string(i ? "," : "") + "\n    \"" + esc(no_decay_patterns[i]) + "\"";
            }
            j += "\n  ]";
        }
        if (m->has_loss_scale)
            j += ",\n  \"loss_scale\": {\n    \"scale\": " + f64_text(m->loss_scale.scale) + ",\n    \"consecutive_ok\": " +
                 std::to_string(m->loss_scale.consecutive_ok) + "\n  }";
        if (m->has_world_size) j += ",\n  \"world_size\": " + std::to_string(m->world_size);
        if (m->has_global_batch_rows) j += ",\n  \"global_batch_rows\": " + std::to_string(m->global_batch_rows);
        if (m->has_spike_guard)
            j += ",\n  \"spike_guard\": {\n    \"mean\": " + f64_text(m->spike_guard.mean) + ",\n    \"variance\": " +
                 f64_text(m->spike_guard.variance) + ",\n    \"observed\": " + std::to_string(m->spike_guard.observed) +
                 ",\n    \"detected\": " + std::to_string(m->spike_guard.detected) + ",\n    \"skipped\": " +
                 std::to_string(m->spike_guard.skipped) + "\n  }";
        if (m->has_mixture) {
            j += ",\n  \"mixture\": {\n    \"weights\": [";
            for (uint32_t i = 0; i < m->n_mixture_weights; i++) j += std::string(i ? "," : "") + "\n      " + f64_text(mixture_weights[i]);
            j += std::string(m->n_mixture_weights ? "\n    " : "") + "],\n    \"rows_per_epoch\": " + std::to_string(m->mixture_rows_per_epoch) + "\n  }";
        }
        j += "\n}";
        // atomic like CheckpointMeta::save_to (src/config.rs:1386-1394): write beside, then rename
        const std::string tmp = std::string(path) + ".tmp";
        FILE* f = fopen(tmp.c_str(), "wb");
        const char* next = "Check that the directory is writable.";
        if (!f) return fail(OXZ_ERR_INVALID, "failed to write checkpoint meta '%s': %s. %s", path, strerror(errno), next);
        const bool wrote = fwrite(j.data(), 1, j.size(), f) == j.size();
        if (fclose(f) != 0 || !wrote || rename(tmp.c_str(), path) != 0) {
            const int32_t st = fail(OXZ_ERR_INVALID, "failed to write checkpoint meta '%s': %s. %s", path, strerror(errno), next);
            remove(tmp.c_str());
            return st;
        }
        return OXZ_OK;
    });
}

int32_t oxz_check_resume_world(const char* meta_path, uint64_t start_step, uint64_t world, uint64_t global_batch_rows,
                               char* warning, uint64_t cap) {
    return oxz::guarded("oxz_check_resume_world", [&]() -> int32_t {
        if (warning && cap) warning[0] = '\0';
        if (!meta_path || start_step == 0) return OXZ_OK;  // a fresh run and a resume without a meta check nothing
        Parsed p;
        std::string why;
        if (!parse_file(meta_path, &p, &why))
            return fail(OXZ_ERR_INVALID, "checkpoint meta '%s' was not read: %s. Restore the file to resume with its world size.",
                        meta_path, why.c_str());
        const uint64_t saved = p.m.has_world_size ? p.m.world_size : 1;  // an old meta reads as one rank
        if (saved != world)
            return fail(OXZ_ERR_INVALID,
                        "checkpoint meta '%s' records world size %llu, and this run has world size %llu. Resume with %llu "
                        "GPU id(s) in `--gpus`, or start a fresh run.",
                        meta_path, (unsigned long long)saved, (unsigned long long)world, (unsigned long long)saved);
        if (p.m.has_global_batch_rows && p.m.global_batch_rows != global_batch_rows && warning && cap)
            snprintf(warning, cap,
                     "Warning: checkpoint meta '%s' records global batches of %llu rows, and this run's global batch is %llu "
                     "rows. The data stream resumes at the saved row, but the resume does not match an uninterrupted run.",
                     meta_path, (unsigned long long)p.m.global_batch_rows, (unsigned long long)global_batch_rows);
        return OXZ_OK;
    });
}

// f64 the way Rust's `{}` prints it for the common cases: the shortest text that reads back, no trailing ".0"
static std::string display_f64(double v) {
    std::string t = f64_text(v);
    if (t.size() > 2 && t.compare(t.size() - 2, 2, ".0") == 0) t.resize(t.size() - 2);
    return t;
}
static std::string debug_weights(const std::vector<double>& w) {  // `{:?}` of a Vec<f64>
    std::string t = "[";
    for (size_t i = 0; i < w.size(); i++) t += (i ? ", " : "") + f64_text(w[i]);
    return t + "]";
}

int32_t oxz_check_mixture_resume(const char* meta_path, uint64_t start_step, int32_t has_current, const double* weights,
                                 uint32_t n_weights, uint64_t rows_per_epoch) {
    return oxz::guarded("oxz_check_mixture_resume", [&]() -> int32_t {
        if (has_current && n_weights && !weights) return fail(OXZ_ERR_INVALID, "oxz_check_mixture_resume: null argument");
        if (!meta_path || start_step == 0) return OXZ_OK;
        Parsed p;
        std::string why;
        if (!parse_file(meta_path, &p, &why))
            return fail(OXZ_ERR_DATA, "checkpoint meta '%s' was not read: %s. Restore the file to resume with its data mixture.",
                        meta_path, why.c_str());
        const bool saved = p.m.has_mixture != 0;
        const std::vector<double> current(weights, weights + (has_current ? n_weights : 0));
        std::string reason;
        if (!saved && !has_current) return OXZ_OK;
        if (saved && !has_current)
            reason = "the checkpoint trained on trainer.data.sources weights " + debug_weights(p.mixture_weights) + ", and this run sets no weights.";
        else if (!saved && has_current)
            reason = "the checkpoint trained without trainer.data.sources weights, and this run sets weights " + debug_weights(current) + ".";
        else if (p.mixture_weights.size() != current.size())
            reason = "the checkpoint trained on " + std::to_string(p.mixture_weights.size()) + " weighted trainer.data.sources, and this run sets " +
                     std::to_string(current.size()) + ".";
        else {
            for (size_t i = 0; i < current.size() && reason.empty(); i++)
                if (memcmp(&p.mixture_weights[i], &current[i], 8) != 0)  // compared by bits
                    reason = "trainer.data.sources[" + std::to_string(i) + "].weight was " + display_f64(p.mixture_weights[i]) +
                             ", and this run sets " + display_f64(current[i]) + ".";
            if (reason.empty() && p.m.mixture_rows_per_epoch != rows_per_epoch)
                reason = "trainer.data.rows_per_epoch was " + std::to_string(p.m.mixture_rows_per_epoch) + ", and this run reads " +
                         std::to_string(rows_per_epoch) + " rows per epoch.";
        }
        if (reason.empty()) return OXZ_OK;
        return fail(OXZ_ERR_DATA, "checkpoint meta '%s': %s The mixture decides which rows the saved data position counts. Resume with the original config, or start a fresh run.",
                    meta_path, reason.c_str());
    });
}

int32_t oxz_read_loss_scale_state(const char* meta_path, uint64_t start_step, int32_t* has_state, oxz_scaler_state* state) {
    return oxz::guarded("oxz_read_loss_scale_state", [&]() -> int32_t {
        if (!has_state || !state) return fail(OXZ_ERR_INVALID, "oxz_read_loss_scale_state: null argument");
        *has_state = 0;
        if (!meta_path || start_step == 0) return OXZ_OK;
        Parsed p;
        std::string why;
        if (!parse_file(meta_path, &p, &why))
            return fail(OXZ_ERR_INVALID, "checkpoint meta '%s' was not read: %s. Restore the file to resume with its loss scale.",
                        meta_path, why.c_str());
        if (p.m.has_loss_scale) {
            *has_state = 1;
            *state = p.m.loss_scale;
        }
        return OXZ_OK;
    });
}

}  // extern "C"
