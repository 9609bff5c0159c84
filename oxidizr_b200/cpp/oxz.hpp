// Host-side mirror of the reference's interface for the data-parallel optimizer step, in C++17 over the C ABI of
// liboxz_dpstep.so. The reference is compiled code (Rust); this header is what its safe wrapper over the FFI crate
// would look like, with the reference's names and error behaviour: LossScaler (src/loss_scale/scaler.rs),
// WeightDecaySpec / DecayPlan (src/weight_decay/), SpikeGuard (src/metrics/spike.rs), LrPlan (src/schedule.rs),
// RowLayout (src/data/rows.rs), the communicator and run_ranks (src/dp/launch.rs), and the post-accumulation half of
// LitTrainer::step_once (src/trainer.rs:515-695). Every decision and all arithmetic happens inside the library.
#pragma once

#include <cmath>
#include <cstdint>
#include <functional>
#include <limits>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/oxz_dpstep.h"

namespace oxidizr {

// boostr::error::Error as oxidizr sees it: the variant follows the status.
struct Error : std::runtime_error {
    enum class Kind { Training, Distributed, Data };
    int32_t status;
    Kind kind;
    Error(int32_t s, const std::string& reason)
        : std::runtime_error(reason), status(s),
          kind(s == OXZ_ERR_NCCL || s == OXZ_ERR_ABORTED || s == OXZ_ERR_TIMEOUT ? Kind::Distributed
               : s == OXZ_ERR_DATA ? Kind::Data : Kind::Training) {}
};

inline void check(int32_t status) {
    if (status != OXZ_OK) throw Error(status, oxz_last_error());
}

constexpr double NONE = std::numeric_limits<double>::quiet_NaN();  // an unset Option<f64>

// ---- loss scale (src/loss_scale/config.rs:28-41, scaler.rs:13-51)
struct LossScaleConfig {
    double initial = 65536.0, growth_factor = 2.0, backoff_factor = 0.5;
    uint64_t growth_interval = 2000;
    oxz_scaler_config c() const { return {initial, growth_factor, backoff_factor, growth_interval}; }
    void check_fields() const { auto v = c(); check(oxz_scaler_check(&v)); }
};
struct GradScalerState {
    double scale = 0.0;
    uint64_t consecutive_ok = 0;
    bool operator==(const GradScalerState& o) const { return scale == o.scale && consecutive_ok == o.consecutive_ok; }
};
class LossScaler {
  public:
    explicit LossScaler(LossScaleConfig config = {}) : cfg_(config.c()) { check(oxz_scaler_init(&cfg_, &st_)); }
    double scale() const { return st_.scale; }
    GradScalerState state() const { return {st_.scale, st_.consecutive_ok}; }
    void restore(GradScalerState s) { oxz_scaler_state saved{s.scale, s.consecutive_ok}; check(oxz_scaler_restore(&saved, &st_)); }
    void record_step(bool overflow, bool spike_skip = false) { check(oxz_scaler_record_step(&cfg_, &st_, overflow, spike_skip)); }
  private:
    oxz_scaler_config cfg_;
    oxz_scaler_state st_{};
};

// ---- weight decay (src/weight_decay/rule.rs:10-118, plan.rs:10-122)
enum class WeightDecayRule { DecayAll = OXZ_DECAY_ALL, Skip1d = OXZ_SKIP_1D, SkipAll = OXZ_SKIP_ALL };
struct WeightDecaySpec {
    WeightDecayRule rule = WeightDecayRule::Skip1d;
    std::vector<std::string> no_decay_patterns;
    std::vector<const char*> ptrs() const { std::vector<const char*> p; for (auto& s : no_decay_patterns) p.push_back(s.c_str()); return p; }
    void check_spec() const { auto p = ptrs(); check(oxz_decay_check((int32_t)rule, p.data(), (uint32_t)p.size())); }
    bool excludes(const std::string& name, size_t rank) const {
        auto p = ptrs();
        int32_t ex = 0;
        check(oxz_decay_excludes((int32_t)rule, p.data(), (uint32_t)p.size(), name.c_str(), (uint32_t)rank, &ex));
        return ex != 0;
    }
};
struct TensorInfo {
    uint64_t id;
    std::string name;  // checkpoint name
    std::vector<uint64_t> shape;
    uint64_t elements() const { uint64_t n = 1; for (auto d : shape) n *= d; return n; }
};
class DecayPlan {
  public:
    DecayPlan(WeightDecaySpec spec, const std::vector<TensorInfo>& tensors) : spec_(std::move(spec)) {
        spec_.check_spec();
        std::vector<uint64_t> seen;
        for (const auto& t : tensors) {
            bool dup = false;
            for (auto id : seen) dup |= id == t.id;
            if (dup) continue;  // a repeated id counts once, under its first entry
            seen.push_back(t.id);
            tensors_.push_back(t);
            const bool ex = spec_.excludes(t.name, t.shape.size());
            no_decay_.push_back(ex ? 1 : 0);
            if (ex) no_decay_elements_ += t.elements();
            else { decay_tensors_++; decay_elements_ += t.elements(); }
        }
    }
    const std::vector<uint8_t>& no_decay() const { return no_decay_; }
    const std::vector<TensorInfo>& tensors() const { return tensors_; }
    size_t decay_tensors() const { return decay_tensors_; }
    uint64_t decay_elements() const { return decay_elements_; }
    uint64_t no_decay_elements() const { return no_decay_elements_; }
  private:
    WeightDecaySpec spec_;
    std::vector<TensorInfo> tensors_;
    std::vector<uint8_t> no_decay_;
    size_t decay_tensors_ = 0;
    uint64_t decay_elements_ = 0, no_decay_elements_ = 0;
};

// ---- spike guard (src/metrics/config.rs:69-115, spike.rs:72-168, state.rs:79-86)
struct SpikeGuardConfig {
    uint64_t window = 100;
    double z_threshold = 6.0;
    uint64_t min_steps = 50;
    bool warn_only = false;
};
class SpikeGuard {
  public:
    explicit SpikeGuard(SpikeGuardConfig c) : cfg_{c.window, c.z_threshold, c.min_steps, c.warn_only, 0} {
        oxz_spike_state probe{};
        int32_t skip = 0;
        check(oxz_spike_judge(&cfg_, &probe, 0, NONE, &skip, nullptr));
    }
    bool judge(uint64_t index, double loss) {
        int32_t skip = 0, flagged = 0;
        check(oxz_spike_judge(&cfg_, &st_, index, loss, &skip, &flagged));
        last_flagged = flagged != 0;
        return skip != 0;
    }
    const oxz_spike_state& state() const { return st_; }
    bool last_flagged = false;
  private:
    oxz_spike_config cfg_;
    oxz_spike_state st_{};
};

// ---- learning rate (src/schedule.rs:135-202)
class LrPlan {
  public:
    LrPlan(double base_lr, oxz_lr_schedule schedule, uint64_t warmup_steps, uint64_t total_steps, double min_lr_ratio,
           std::optional<uint64_t> decay_steps = std::nullopt, std::optional<double> decay_ratio = std::nullopt,
           oxz_decay_shape shape = OXZ_SHAPE_LINEAR)
        : p_{base_lr, min_lr_ratio, warmup_steps, total_steps, 0, (int32_t)schedule, (int32_t)shape} {
        if (schedule == OXZ_LR_WSD)
            p_.decay_steps = decay_steps ? *decay_steps : (uint64_t)std::ceil((double)total_steps * decay_ratio.value_or(0.1));
        lr_at(0);
    }
    double lr_at(uint64_t step) const { double lr = 0; check(oxz_lr_at(&p_, step, &lr)); return lr; }
  private:
    oxz_lr_plan p_;
};

// ---- rows (src/data/rows.rs:29-208)
struct DataPosition {
    uint64_t epoch = 0, row = 0;
    bool operator==(const DataPosition& o) const { return epoch == o.epoch && row == o.row; }
};
class RowLayout {
  public:
    static RowLayout for_world(uint64_t num_rows, uint64_t rank_batch_size, uint64_t world_size) {
        RowLayout l;
        l.l_ = {num_rows, rank_batch_size, world_size};
        check(oxz_rows_check(&l.l_));
        return l;
    }
    static RowLayout create(uint64_t num_rows, uint64_t batch_size) { return for_world(num_rows, batch_size, 1); }
    uint64_t num_rows() const { return l_.num_rows; }
    uint64_t batch_size() const { return l_.rank_batch_size * l_.world_size; }
    uint64_t batches_per_epoch() const { return l_.num_rows / batch_size(); }
    uint64_t total_steps(uint64_t grad_accum, uint64_t num_epochs) const { return batches_per_epoch() * num_epochs / (grad_accum ? grad_accum : 1); }
    DataPosition advance(DataPosition pos, uint64_t batches) const {
        oxz_data_position out{};
        check(oxz_rows_advance(&l_, {pos.epoch, pos.row}, batches, &out));
        return {out.epoch, out.row};
    }
    DataPosition batch_start(DataPosition pos) const { return pos.row + batch_size() > l_.num_rows ? DataPosition{pos.epoch + 1, 0} : pos; }
    // One rank's rows of the next global batch. With `order` = (epoch, that epoch's permutation) the row at each slot is
    // order.second[slot], as EpochOrder::row does under RowOrder::Shuffled (src/data/rows.rs:240-256); the permutation is
    // the caller's epoch_permutation(num_rows, seed, epoch) (src/data/rows.rs:258-263). Returns the position after the batch.
    DataPosition next_window(DataPosition pos, uint64_t rank, std::vector<uint64_t>& rows,
                             const std::pair<uint64_t, std::vector<uint32_t>>* order = nullptr) const {
        rows.resize(l_.rank_batch_size);
        oxz_data_position next{};
        if (order) check(oxz_rows_next_window_ordered(&l_, {pos.epoch, pos.row}, rank, 1, 0, nullptr, 0, order->first, order->second.data(),
                                                      order->second.size(), rows.data(), nullptr, nullptr, &next));
        else check(oxz_rows_next_window(&l_, {pos.epoch, pos.row}, rank, 1, 0, nullptr, 0, rows.data(), nullptr, nullptr, &next));
        return {next.epoch, next.row};
    }
    uint64_t batch_epoch(DataPosition pos) const { uint64_t e = 0; check(oxz_rows_batch_epoch(&l_, {pos.epoch, pos.row}, &e)); return e; }
    DataPosition position_after_steps(uint64_t steps, uint64_t grad_accum) const { return advance({}, steps * grad_accum); }
    const oxz_row_layout& raw() const { return l_; }
  private:
    oxz_row_layout l_{};
};

// ---- the checkpoint meta's data-parallel and loss-scale keys on resume (src/dp/resume.rs:19-55, src/loss_scale/resume.rs:14-29)
struct CheckpointMeta {
    oxz_resume_meta raw{};
    std::vector<std::string> no_decay_patterns;
    std::vector<double> mixture_weights;  // with raw.mixture_rows_per_epoch: MixtureRecord
    static CheckpointMeta load(const std::string& path) {
        CheckpointMeta m;
        check(oxz_meta_load(path.c_str(), &m.raw));
        for (uint32_t i = 0; i < m.raw.n_no_decay_patterns; i++) {
            char buf[4096];
            check(oxz_meta_no_decay_pattern(path.c_str(), i, buf, sizeof buf));
            m.no_decay_patterns.emplace_back(buf);
        }
        m.mixture_weights.resize(m.raw.n_mixture_weights);
        uint32_t n = 0;
        check(oxz_meta_mixture_weights(path.c_str(), m.mixture_weights.data(), m.raw.n_mixture_weights, &n));
        return m;
    }
    void save_to(const std::string& path) {
        std::vector<const char*> p;
        for (const auto& s : no_decay_patterns) p.push_back(s.c_str());
        raw.n_no_decay_patterns = (uint32_t)p.size();
        raw.has_mixture = mixture_weights.empty() ? raw.has_mixture : 1;
        raw.n_mixture_weights = (uint32_t)mixture_weights.size();
        check(oxz_meta_save(path.c_str(), &raw, p.empty() ? nullptr : p.data(), mixture_weights.empty() ? nullptr : mixture_weights.data()));
    }
};
// Returns the warning (empty: none); throws when the meta records another world size.
inline std::string check_resume_world(const char* meta_path, uint64_t start_step, uint64_t world, uint64_t global_batch_rows) {
    char warning[1024];
    check(oxz_check_resume_world(meta_path, start_step, world, global_batch_rows, warning, sizeof warning));
    return warning;
}
inline bool read_loss_scale_state(const char* meta_path, uint64_t start_step, GradScalerState* out) {
    int32_t has = 0;
    oxz_scaler_state st{};
    check(oxz_read_loss_scale_state(meta_path, start_step, &has, &st));
    if (has) *out = GradScalerState{st.scale, st.consecutive_ok};
    return has != 0;
}

// ---- communicator (src/dp/launch.rs:19-109)
class Communicator {
  public:
    explicit Communicator(oxz_comm* h = nullptr) : h_(h) {}
    Communicator(Communicator&& o) noexcept : h_(o.h_) { o.h_ = nullptr; }
    Communicator& operator=(Communicator&& o) noexcept { std::swap(h_, o.h_); return *this; }
    Communicator(const Communicator&) = delete;
    ~Communicator() { if (h_) oxz_comm_destroy(h_); }
    static std::vector<Communicator> local_group(int32_t n, const std::vector<int32_t>* devices = nullptr, double timeout = 30.0) {
        std::vector<oxz_comm*> raw(n);
        check(oxz_comm_init_local(n, devices ? devices->data() : nullptr, timeout, raw.data()));
        std::vector<Communicator> out;
        for (auto* c : raw) out.emplace_back(c);
        return out;
    }
    static std::vector<Communicator> nccl(const std::vector<int32_t>& devices) {
        std::vector<oxz_comm*> raw(devices.size());
        check(oxz_comm_init_all((int32_t)devices.size(), devices.data(), raw.data()));
        std::vector<Communicator> out;
        for (auto* c : raw) out.emplace_back(c);
        return out;
    }
    oxz_comm* handle() const { return h_; }
    int32_t world_size() const { int32_t w = 1; if (h_) check(oxz_comm_world_size(h_, &w)); return w; }
    int32_t rank() const { int32_t r = 0; if (h_) check(oxz_comm_rank(h_, &r)); return r; }
    void abort() const { check(oxz_comm_abort(h_)); }
    void barrier() const { check(oxz_barrier(h_)); }
    std::pair<int64_t, int64_t> sum_counts(int64_t scored, int64_t masks) const {
        int64_t v[2] = {scored, masks};
        check(oxz_allreduce_i64x2(h_, v));
        return {v[0], v[1]};
    }
    double sum_f64(double x) const { check(oxz_allreduce_f64(h_, &x, 1)); return x; }
  private:
    oxz_comm* h_;
};

// run_ranks (src/dp/launch.rs:183-272): one thread per rank, first failure aborts the group and is the error thrown.
inline void run_ranks(const std::vector<Communicator>& comms, const std::function<void(int32_t rank, int32_t world, const Communicator&)>& body) {
    struct Ctx { const std::vector<Communicator>* comms; const std::function<void(int32_t, int32_t, const Communicator&)>* body; } ctx{&comms, &body};
    std::vector<oxz_comm*> raw;
    for (auto& c : comms) raw.push_back(c.handle());
    auto tramp = [](int32_t rank, int32_t world, void* user) -> int32_t {
        auto* c = static_cast<Ctx*>(user);
        try {
            (*c->body)(rank, world, (*c->comms)[rank]);
            return OXZ_OK;
        } catch (const Error& e) {
            oxz_set_last_error(e.what());
            return e.status;
        } catch (const std::exception& e) {
            oxz_set_last_error((std::string("panic: ") + e.what()).c_str());
            return OXZ_ERR_INVALID;
        }
    };
    int32_t failed = -1;
    check(oxz_run_ranks((int32_t)comms.size(), raw.data(), tramp, &ctx, &failed));
}

// ---- the rank-sliced loader (src/data/construction.rs, ranks.rs:25-41, multi_source.rs:17-52, mixture/loader.rs:16-33,
// host_masks.rs:28-77, prefetch.rs:86-115), stream order
struct Batch {  // src/data/batch.rs:11-26; device pointers, valid until the batch after the next
    const int64_t* inputs = nullptr;
    const int64_t* targets = nullptr;
    const float* loss_mask = nullptr;       // null when masking is off
    const int32_t* segment_ids = nullptr;   // null unless the document mask is on
    const int32_t* cu_seqlens = nullptr;
    const uint64_t* scored = nullptr;       // pinned host: read once the stream has passed the batch
    const uint64_t* n_segments = nullptr;
    std::vector<uint64_t> rows;             // the global rows of the batch
};
class LitDataLoader {
  public:
    static LitDataLoader from_files(const std::vector<std::string>& paths, uint64_t batch_size, uint64_t seq_len, int32_t device = 0) {
        return LitDataLoader(paths, batch_size, seq_len, 0, 1, {}, device);
    }
    LitDataLoader(const std::vector<std::string>& paths, uint64_t batch_size, uint64_t seq_len, uint64_t rank, uint64_t world,
                  const std::vector<std::pair<uint64_t, uint64_t>>& row_ranges, int32_t device = 0)
        : batch_(batch_size) {
        std::vector<const char*> p;
        for (const auto& s : paths) p.push_back(s.c_str());
        std::vector<uint64_t> spans;
        for (const auto& r : row_ranges) { spans.push_back(r.first); spans.push_back(r.second); }
        check(oxz_loader_open_files(p.data(), (uint32_t)p.size(), seq_len, batch_size, rank, world, spans.empty() ? nullptr : spans.data(),
                                    (uint32_t)row_ranges.size(), device, &h_));
    }
    LitDataLoader(LitDataLoader&& o) noexcept : h_(o.h_), batch_(o.batch_) { o.h_ = nullptr; }
    LitDataLoader(const LitDataLoader&) = delete;
    ~LitDataLoader() { if (h_) oxz_loader_close(h_); }
    LitDataLoader& with_mixture(const std::vector<double>& weights, std::optional<uint64_t> rows_per_epoch = std::nullopt) {
        check(oxz_loader_set_mixture(h_, weights.data(), (uint32_t)weights.size(), rows_per_epoch ? 1 : 0, rows_per_epoch.value_or(0)));
        return *this;
    }
    LitDataLoader& with_target_mask(uint32_t target_base, const std::vector<uint32_t>& always_score) {  // TargetMask::PrefixLm
        check(oxz_loader_set_target_mask(h_, 1, target_base, always_score.empty() ? nullptr : always_score.data(), (uint32_t)always_score.size()));
        return *this;
    }
    LitDataLoader& with_document_mask(uint32_t separator_id) { check(oxz_loader_set_document_mask(h_, 1, separator_id)); return *this; }
    LitDataLoader& with_prefetch(uint32_t depth) { check(oxz_loader_set_prefetch(h_, depth)); return *this; }
    // with_row_order(RowOrder::Shuffled{seed}) (src/data/construction.rs:140) with the epoch's permutation made by the
    // caller; the loader keeps two epochs' orders. An empty permutation returns to stream order.
    LitDataLoader& set_row_order(uint64_t epoch, const std::vector<uint32_t>& perm) {
        check(oxz_loader_set_row_order(h_, epoch, perm.empty() ? nullptr : perm.data(), perm.size()));
        return *this;
    }
    uint64_t num_rows() const { uint64_t n = 0; check(oxz_loader_num_rows(h_, &n)); return n; }
    std::vector<uint64_t> source_rows() const {
        uint32_t n = 0;
        check(oxz_loader_source_rows(h_, nullptr, 0, &n));
        std::vector<uint64_t> rows(n);
        check(oxz_loader_source_rows(h_, rows.data(), n, &n));
        return rows;
    }
    DataPosition position() const { oxz_data_position p{}; check(oxz_loader_position(h_, &p)); return {p.epoch, p.row}; }
    void seek(DataPosition pos) { check(oxz_loader_seek(h_, {pos.epoch, pos.row})); }
    std::vector<uint64_t> next_rows() { std::vector<uint64_t> rows(batch_); check(oxz_loader_next_rows(h_, rows.data())); return rows; }
    Batch next_batch(void* stream = nullptr) {
        Batch b;
        b.rows.resize(batch_);
        int64_t *in = nullptr, *tg = nullptr;
        check(oxz_loader_next_batch_async(h_, stream, &in, &tg, b.rows.data()));
        oxz_batch_masks m{};
        check(oxz_loader_batch_masks(h_, &m));
        b.inputs = in;
        b.targets = tg;
        b.loss_mask = m.loss_mask;
        b.segment_ids = m.segment_ids;
        b.cu_seqlens = m.cu_seqlens;
        b.scored = m.scored;
        b.n_segments = m.n_segments;
        return b;
    }
  private:
    oxz_loader* h_ = nullptr;
    uint64_t batch_;
};

// ---- the optimizer state and step
struct StepConfig {  // trainer keys with the reference's defaults (src/config.rs:40-62)
    double lr = 3e-4, beta1 = 0.9, beta2 = 0.95, eps = 1e-6, weight_decay = 0.1, max_grad_norm = 1.0;
    double max_grad_value = NONE, target_grad_norm = NONE, loss_scale = NONE, clip_eps = 1e-6;
    bool spike_skip = false;
    oxz_hyper hyper() const { return {lr, beta1, beta2, eps, weight_decay, max_grad_norm, max_grad_value, target_grad_norm, loss_scale, clip_eps, 0, 0, spike_skip, 0}; }
};

class DpOptimizer {
  public:
    DpOptimizer(const std::vector<uint64_t>& numel, const std::vector<uint8_t>& no_decay, oxz_dtype grad_dtype, oxz_dtype param_dtype,
                const Communicator* comm = nullptr, int32_t device = 0, oxz_sync_mode mode = OXZ_SYNC_P2P, uint64_t bucket_bytes = 0)
        : comm_(comm) {
        const int32_t world = comm ? comm->world_size() : 1;
        oxz_plan_desc d{numel.size(), numel.data(), no_decay.empty() ? nullptr : no_decay.data(), nullptr, grad_dtype, param_dtype,
                        world, comm ? comm->rank() : 0, world == 1 ? OXZ_SYNC_SINGLE : mode, device, bucket_bytes};
        check(oxz_plan_create(&d, &h_));
        numel_ = numel;
    }
    DpOptimizer(const DpOptimizer&) = delete;
    ~DpOptimizer() { if (h_) oxz_plan_destroy(h_); }
    void alloc() { check(oxz_state_alloc(h_, comm_ ? comm_->handle() : nullptr)); }
    oxz_plan_info info() const { oxz_plan_info i{}; check(oxz_plan_query(h_, &i)); return i; }
    void import_tensor(oxz_state_kind kind, uint64_t tensor, const void* host) { if (numel_[tensor]) check(oxz_state_import(h_, kind, tensor, host)); }
    void export_tensor(oxz_state_kind kind, uint64_t tensor, void* host) { if (numel_[tensor]) check(oxz_state_export(h_, kind, tensor, host)); }
    uint64_t timestep() const { uint64_t t = 0; check(oxz_state_timestep(h_, &t)); return t; }
    oxz_step_result step(const StepConfig& cfg, const std::vector<uint8_t>* present = nullptr, double* loss = nullptr) {
        oxz_hyper h = cfg.hyper();
        oxz_step_result r{};
        check(oxz_step(h_, comm_ ? comm_->handle() : nullptr, &h, present ? present->data() : nullptr, loss, loss ? 1 : 0, &r));
        return r;
    }
    // grad_norm_for_tensor for every parameter (src/trainer.rs:933-937), what diagnose_bad_gradients reads after a
    // non-finite norm (src/trainer.rs:990-1020); -1 marks a tensor no rank had a gradient for. Collective.
    std::vector<double> grad_norms_per_tensor(double loss_scale = NONE, double max_grad_value = NONE) {
        std::vector<double> norms(numel_.size());
        check(oxz_grad_norms_per_tensor(h_, comm_ ? comm_->handle() : nullptr, loss_scale, max_grad_value, norms.data()));
        return norms;
    }
    int32_t exchange_kind() const { int32_t k = 0; check(oxz_plan_exchange_kind(h_, &k)); return k; }
    int32_t last_update_kernel() const { int32_t k = 0; check(oxz_plan_last_update_kernel(h_, &k)); return k; }
    oxz_plan* handle() const { return h_; }
  private:
    oxz_plan* h_ = nullptr;
    const Communicator* comm_;
    std::vector<uint64_t> numel_;
};

// The post-accumulation half of LitTrainer::step_once (src/trainer.rs:515-695): returns (loss, grad_norm).
class LitTrainerStep {
  public:
    LitTrainerStep(DpOptimizer& opt, LrPlan lr, std::optional<LossScaleConfig> loss_scale = std::nullopt,
                   std::optional<SpikeGuardConfig> spike = std::nullopt, StepConfig base = {})
        : opt_(opt), lr_(lr), base_(base) {
        if (loss_scale) scaler_.emplace(*loss_scale);
        if (spike) guard_.emplace(*spike);
    }
    std::pair<double, double> training_step(double loss, const std::vector<uint8_t>* present = nullptr) {
        StepConfig cfg = base_;
        cfg.lr = lr_.lr_at(global_step_);
        cfg.loss_scale = scaler_ ? scaler_->scale() : NONE;
        cfg.spike_skip = guard_ ? guard_->judge(global_step_, loss) : false;
        const oxz_step_result r = opt_.step(cfg, present, nullptr);
        if (scaler_) scaler_->record_step(r.overflow != 0, cfg.spike_skip);
        global_step_++;
        return {loss, r.reported_norm};
    }
    uint64_t global_step() const { return global_step_; }
    uint64_t optimizer_timestep() const { return opt_.timestep(); }
    std::optional<GradScalerState> loss_scale_state() const { return scaler_ ? std::optional<GradScalerState>(scaler_->state()) : std::nullopt; }
  private:
    DpOptimizer& opt_;
    LrPlan lr_;
    StepConfig base_;
    std::optional<LossScaler> scaler_;
    std::optional<SpikeGuard> guard_;
    uint64_t global_step_ = 0;
};

}  // namespace oxidizr
