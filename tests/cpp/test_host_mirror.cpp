// Known answers of the reference's own unit tests, replayed in C++ through the host-side mirror (oxz.hpp) over the
// C ABI. Without arguments it runs what needs no GPU; with --gpu it also runs the optimizer step on cuda:0.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <thread>

#include <sys/stat.h>
#include <unistd.h>

#include "../../oxidizr_b200/cpp/oxz.hpp"

using namespace oxidizr;

static int failures = 0;
#define EXPECT(cond)                                                        \
    do {                                                                    \
        if (!(cond)) {                                                      \
            printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);        \
            failures++;                                                     \
        }                                                                   \
    } while (0)
template <class F>
static bool throws(F f, const char* needle) {
    try { f(); } catch (const Error& e) { return strstr(e.what(), needle) != nullptr; }
    return false;
}

// src/loss_scale/scaler.rs:273-289, tests/loss_scale.rs:180-214
static void record_step_halves_on_overflow_and_grows_after_the_interval() {
    LossScaleConfig c; c.initial = 64.0; c.growth_interval = 2;
    LossScaler s(c);
    s.record_step(true);  EXPECT(s.scale() == 32.0);
    s.record_step(false); EXPECT(s.scale() == 32.0);
    s.record_step(false); EXPECT(s.scale() == 64.0);
    LossScaler t(c);
    const GradScalerState want[4] = {{64.0, 1}, {128.0, 0}, {128.0, 1}, {256.0, 0}};
    for (auto& w : want) { t.record_step(false); EXPECT(t.state() == w); }
    LossScaleConfig bad; bad.growth_interval = 0;
    EXPECT(throws([&] { LossScaler x(bad); }, "trainer.loss_scale.growth_interval"));
    EXPECT(throws([&] { t.restore({NONE, 0}); }, "finite and positive"));
    t.restore({512.0, 7}); EXPECT((t.state() == GradScalerState{512.0, 7}));
    // a spike skip with finite gradients leaves the scale untouched (src/trainer.rs:666-670)
    t.record_step(false, true); EXPECT((t.state() == GradScalerState{512.0, 7}));
}

// src/weight_decay/rule.rs:142-196, plan.rs:153-175
static void skip_1d_keeps_norms_biases_and_ssm_tensors_out_of_decay() {
    const std::pair<const char*, size_t> names[10] = {
        {"model.embed_tokens.weight", 2}, {"model.layers.0.input_layernorm.weight", 1}, {"model.layers.0.self_attn.q_proj.weight", 2},
        {"model.layers.0.self_attn.q_proj.bias", 1}, {"model.layers.0.self_attn.q_proj.lora_a", 2}, {"model.layers.1.mamba.a_log", 2},
        {"model.layers.1.mamba.d_param", 1}, {"model.layers.1.mamba.dt_bias", 1}, {"model.layers.1.mamba.b_bias", 2}, {"lm_head.weight", 2}};
    const bool want[10] = {false, true, false, true, false, true, true, true, true, false};
    WeightDecaySpec skip;
    for (int i = 0; i < 10; i++) EXPECT(skip.excludes(names[i].first, names[i].second) == want[i]);
    WeightDecaySpec all{WeightDecayRule::DecayAll, {}}, none{WeightDecayRule::SkipAll, {}};
    for (auto& n : names) { EXPECT(!all.excludes(n.first, n.second)); EXPECT(none.excludes(n.first, n.second)); }
    WeightDecaySpec pat{WeightDecayRule::Skip1d, {"embed_tokens", "lora_"}};
    EXPECT(pat.excludes("model.embed_tokens.weight", 2) && pat.excludes("model.layers.0.self_attn.q_proj.lora_a", 2));
    EXPECT(!pat.excludes("lm_head.weight", 2));
    EXPECT(throws([&] { WeightDecaySpec{WeightDecayRule::DecayAll, {"embed"}}.check_spec(); }, "skip_1d"));
    EXPECT(throws([&] { WeightDecaySpec{WeightDecayRule::Skip1d, {""}}.check_spec(); }, "no_decay_patterns[0]"));
    DecayPlan plan(skip, {{7, "model.embed_tokens.weight", {2, 3}}, {7, "lm_head.weight", {2, 3}}, {9, "model.norm.weight", {3}}});
    EXPECT(plan.no_decay() == (std::vector<uint8_t>{0, 1}));
    EXPECT(plan.decay_tensors() == 1 && plan.decay_elements() == 6 && plan.no_decay_elements() == 3);
}

// src/metrics/spike.rs:204-217, src/metrics/state.rs:122-152
static void the_guard_skips_the_scripted_spike() {
    SpikeGuard g({4, 6.0, 50, false});
    const double first[3] = {1.0, 2.0, 0.5};
    for (int i = 0; i < 3; i++) EXPECT(!g.judge(i, first[i]));
    EXPECT(g.state().observed == 3 && std::fabs(g.state().mean - 1.04) < 1e-12 && std::fabs(g.state().variance - 0.3384) < 1e-12);
    SpikeGuard h({4, 6.0, 2, false});
    const bool want[5] = {false, false, false, true, false};
    for (int i = 0; i < 5; i++) EXPECT(h.judge(i, i == 3 ? 1e3 : 1.0 + 0.1 * (i % 2)) == want[i]);
    EXPECT(h.state().observed == 4 && h.state().detected == 1 && h.state().skipped == 1);
    EXPECT(throws([] { SpikeGuard bad({0, 6.0, 2, false}); }, "window"));
}

// src/schedule.rs:284-428
static void lr_plan_matches_the_closed_form() {
    const double base = 3e-4;
    const uint64_t total = 110;
    for (auto shape : {OXZ_SHAPE_LINEAR, OXZ_SHAPE_COSINE, OXZ_SHAPE_SQRT}) {
        LrPlan p(base, OXZ_LR_WSD, 10, total, 0.1, 20, std::nullopt, shape);
        EXPECT(p.lr_at(0) == base * (1.0 / 10.0) && p.lr_at(9) == base && p.lr_at(90) == base);
        EXPECT(p.lr_at(91) < base && p.lr_at(109) > base * 0.1 && p.lr_at(total) == base * 0.1 && p.lr_at(total + 50) == base * 0.1);
    }
    LrPlan cosine(base, OXZ_LR_COSINE, 10, total, 0.37);
    for (uint64_t s = 11; s <= total + 5; s++) {
        const double progress = std::min((double)(s - 10) / (double)(total - 10), 1.0);
        const double want = base * (0.37 + (1.0 - 0.37) * (0.5 * (1.0 + std::cos(M_PI * progress))));
        EXPECT(cosine.lr_at(s) == want);
    }
    EXPECT(LrPlan(base, OXZ_LR_WSD, 10, total, 0.1).lr_at(99) == base);  // ceil(110 * 0.1) = 11 decay steps
    EXPECT(throws([&] { LrPlan(base, OXZ_LR_WSD, 10, total, 0.1, 101); }, "trainer.decay_steps"));
}

// src/data/rows.rs:293-360
static void advance_matches_one_batch_at_a_time() {
    const uint64_t cases[5][2] = {{10, 3}, {9, 3}, {7, 1}, {5, 5}, {11, 4}};
    for (auto& c : cases) {
        RowLayout l = RowLayout::create(c[0], c[1]);
        for (uint64_t start = 0; start <= c[0]; start++)
            for (uint64_t n = 0; n < 4 * l.batches_per_epoch() + 3; n++) {
                DataPosition pos{2, start};
                for (uint64_t k = 0; k < n; k++) { DataPosition s = l.batch_start(pos); pos = {s.epoch, s.row + l.batch_size()}; }
                EXPECT(l.advance({2, start}, n) == pos);
            }
    }
    RowLayout w = RowLayout::for_world(22, 3, 2);
    EXPECT(w.batch_size() == 6 && w.batches_per_epoch() == 3 && w.total_steps(1, 2) == 6);
    EXPECT((w.advance({}, 4) == DataPosition{1, 6}));
    EXPECT(throws([] { RowLayout::for_world(5, 3, 2); }, "one global batch of 6 rows"));
    EXPECT(throws([] { RowLayout::create(3, 4); }, "fewer than batch_size 4"));
}

// src/data/rows.rs:240-256 and :376-411: under a shuffled order the row at a slot is the epoch's permutation at that
// slot; an epoch reads every row once; the ranks' windows are disjoint; the wrong epoch's order is refused.
static void a_shuffled_epoch_reads_the_callers_permutation() {
    const uint64_t rows = 12;
    RowLayout l = RowLayout::for_world(rows, 2, 2);
    auto perm_of = [&](uint64_t epoch) {
        std::vector<uint32_t> p(rows);
        for (uint64_t i = 0; i < rows; i++) p[i] = (uint32_t)((i * 5 + 3 * epoch + 1) % rows);  // 5 is coprime to 12
        return p;
    };
    DataPosition pos[2] = {{}, {}};
    for (uint64_t epoch = 0; epoch < 2; epoch++) {
        std::vector<int> seen(rows, 0);
        for (int batch = 0; batch < 3; batch++)
            for (uint64_t rank = 0; rank < 2; rank++) {
                EXPECT(l.batch_epoch(pos[rank]) == epoch);
                std::pair<uint64_t, std::vector<uint32_t>> order{epoch, perm_of(epoch)};
                std::vector<uint64_t> got;
                const DataPosition start = l.batch_start(pos[rank]);
                pos[rank] = l.next_window(pos[rank], rank, got, &order);
                for (uint64_t k = 0; k < 2; k++) {
                    EXPECT(got[k] == order.second[start.row + rank * 2 + k]);
                    seen[got[k]]++;
                }
            }
        for (uint64_t r = 0; r < rows; r++) EXPECT(seen[r] == 1);
    }
    std::pair<uint64_t, std::vector<uint32_t>> wrong{5, perm_of(5)};
    std::vector<uint64_t> got;
    EXPECT(throws([&] { l.next_window({}, 0, got, &wrong); }, "reads epoch 0 and the row order given is epoch 5"));
    std::vector<uint32_t> twice = perm_of(0);
    twice[1] = twice[0];
    EXPECT(oxz_rows_check_permutation(twice.data(), twice.size()) == OXZ_ERR_DATA);
    EXPECT(oxz_rows_check_permutation(perm_of(1).data(), rows) == OXZ_OK);
}

// src/dp/resume.rs:76-125
static void the_meta_world_size_gates_a_resume() {
    const std::string dir = std::string("/tmp/oxz-mirror-meta-") + std::to_string((long)getpid());
    mkdir(dir.c_str(), 0700);
    auto meta_file = [&](const char* tag, int world, int rows) {
        CheckpointMeta m;
        m.raw.step = 3;
        snprintf(m.raw.checkpoint_file, sizeof m.raw.checkpoint_file, "w.safetensors");
        if (world) { m.raw.has_world_size = 1; m.raw.world_size = (uint64_t)world; }
        if (rows) { m.raw.has_global_batch_rows = 1; m.raw.global_batch_rows = (uint64_t)rows; }
        const std::string path = dir + "/" + tag + ".meta.json";
        m.save_to(path);
        return path;
    };
    const std::string match = meta_file("match", 2, 8), old = meta_file("old", 0, 0), batch = meta_file("batch", 1, 4);
    EXPECT(check_resume_world(match.c_str(), 3, 2, 8).empty());
    EXPECT(throws([&] { check_resume_world(match.c_str(), 3, 1, 4); }, "world size 2"));
    EXPECT(throws([&] { check_resume_world(match.c_str(), 3, 1, 4); }, "--gpus"));
    EXPECT(check_resume_world(old.c_str(), 3, 1, 4).empty());
    EXPECT(throws([&] { check_resume_world(old.c_str(), 3, 2, 8); }, "world size 1"));
    const std::string warning = check_resume_world(batch.c_str(), 3, 1, 6);
    EXPECT(warning.find("4 rows") != std::string::npos && warning.find("6 rows") != std::string::npos);
    EXPECT(check_resume_world(match.c_str(), 0, 1, 4).empty() && check_resume_world(nullptr, 5, 3, 12).empty());
    GradScalerState st{};
    EXPECT(!read_loss_scale_state(match.c_str(), 3, &st));
    for (const std::string& p : {match, old, batch}) remove(p.c_str());
    rmdir(dir.c_str());
}

// src/data/multi_source.rs:99-161, src/data/mixture/loader.rs:108-171 in stream order, on the host alone
static void the_loader_reads_sources_ranges_and_mixtures_in_order() {
    const std::string dir = std::string("/tmp/oxz-mirror-data-") + std::to_string((long)getpid());
    mkdir(dir.c_str(), 0700);
    const uint64_t seq = 3, width = seq + 1;
    std::vector<std::string> paths;
    uint32_t first = 0;
    const uint64_t rows[3] = {3, 2, 4};
    for (int i = 0; i < 3; i++) {  // every token is its own offset in the concatenation; each file has a 2-token tail
        paths.push_back(dir + "/s" + std::to_string(i) + ".bin");
        FILE* f = fopen(paths.back().c_str(), "wb");
        for (uint32_t t = 0; t < rows[i] * width; t++) { const uint32_t v = first + t; fwrite(&v, 4, 1, f); }
        const uint32_t tail = 0xffffffffu;
        fwrite(&tail, 4, 1, f);
        fwrite(&tail, 4, 1, f);
        fclose(f);
        first += (uint32_t)(rows[i] * width);
    }
    {
        LitDataLoader l = LitDataLoader::from_files(paths, 3, seq, -1);
        EXPECT((l.source_rows() == std::vector<uint64_t>{3, 2, 4}) && l.num_rows() == 9);
        std::vector<uint64_t> seen;
        for (int b = 0; b < 3; b++) for (uint64_t r : l.next_rows()) seen.push_back(r);
        EXPECT((seen == std::vector<uint64_t>{0, 1, 2, 3, 4, 5, 6, 7, 8}));
    }
    {
        LitDataLoader eval(paths, 1, seq, 0, 1, {{2, 3}, {8, 9}}, -1);
        EXPECT((eval.next_rows() == std::vector<uint64_t>{2}) && (eval.next_rows() == std::vector<uint64_t>{8}));
        EXPECT(throws([&] { LitDataLoader(paths, 1, seq, 0, 1, {{0, 5}, {4, 6}}, -1); }, "starts before row 5"));
    }
    {
        LitDataLoader full(paths, 3, seq, 0, 1, {}, -1), resumed(paths, 3, seq, 0, 1, {}, -1);
        full.with_mixture({1.0, 1.0, 2.0}, 12);
        resumed.with_mixture({1.0, 1.0, 2.0}, 12);
        EXPECT(full.num_rows() == 12);
        for (int b = 0; b < 5; b++) full.next_rows();
        resumed.seek(RowLayout::create(12, 3).advance({}, 5));
        for (int b = 0; b < 9; b++) EXPECT(full.next_rows() == resumed.next_rows());
        EXPECT(throws([&] { LitDataLoader(paths, 1, seq, 0, 1, {}, -1).with_mixture({1.0}); }, "1 weight(s)"));
    }
    for (const auto& p : paths) remove(p.c_str());
    rmdir(dir.c_str());
}

// src/dp/reduce.rs:88-121, src/dp/launch.rs:296-366
static void ranks_sum_and_the_first_error_wins() {
    auto comms = Communicator::local_group(2, nullptr, 10.0);
    double got[2] = {0, 0};
    run_ranks(comms, [&](int32_t rank, int32_t, const Communicator& c) { got[rank] = c.sum_f64(rank == 0 ? 0.75 : 0.5); });
    EXPECT(got[0] == 1.25 && got[1] == 1.25);
    auto three = Communicator::local_group(3, nullptr, 30.0);
    bool ok = false;
    try {
        run_ranks(three, [&](int32_t rank, int32_t, const Communicator& c) {
            c.sum_counts(1, 0);
            if (rank == 1) throw Error(OXZ_ERR_DATA, "the loader of this rank ran out of rows");
            c.sum_counts(1, 0);  // the peers block here until the abort
        });
    } catch (const Error& e) {
        ok = strstr(e.what(), "rank 1 of 3 failed first: the loader of this rank ran out of rows") && e.kind == Error::Kind::Data;
    }
    EXPECT(ok);
}

// src/grad_clip.rs:82-143, tests/weight_decay.rs:102-147, tests/loss_scale.rs:118-176 on the device
static void the_step_on_the_gpu() {
    const std::vector<uint64_t> numel = {4, 2};
    DpOptimizer opt(numel, {0, 1}, OXZ_F32, OXZ_F32);
    opt.alloc();
    const float w0[4] = {1.f, -2.f, 3.f, -4.f}, w1[2] = {0.5f, -0.5f};
    const float g0[4] = {100.f, -100.f, 100.f, -100.f}, g1[2] = {0.f, 0.f};
    opt.import_tensor(OXZ_STATE_MASTER, 0, w0); opt.import_tensor(OXZ_STATE_MASTER, 1, w1);
    opt.import_tensor(OXZ_STATE_GRADS, 0, g0);  opt.import_tensor(OXZ_STATE_GRADS, 1, g1);
    StepConfig cfg; cfg.max_grad_value = 3.0; cfg.max_grad_norm = 1.5;
    auto r = opt.step(cfg);  // clamp to 3 gives norm 6, the norm clip scales to 1.5
    EXPECT(std::fabs(r.grad_norm - 6.0) < 1e-5 && r.reported_norm == 1.5 && r.applied == 1 && opt.timestep() == 1);
    float out1[2];
    opt.export_tensor(OXZ_STATE_MASTER, 1, out1);
    EXPECT(out1[0] == 0.5f && out1[1] == -0.5f);  // zero gradient, no-decay group: bit-unchanged
    const float bad[4] = {1.f, INFINITY, 1.f, 1.f};
    opt.import_tensor(OXZ_STATE_GRADS, 0, bad);
    float before[4], after[4];
    opt.export_tensor(OXZ_STATE_MASTER, 0, before);
    r = opt.step(cfg);
    opt.export_tensor(OXZ_STATE_MASTER, 0, after);
    EXPECT(r.overflow == 1 && r.applied == 0 && !std::isfinite(r.grad_norm) && opt.timestep() == 1);
    EXPECT(memcmp(before, after, sizeof before) == 0);
    // diagnose_bad_gradients (src/trainer.rs:990-1020): the per-tensor norms name the tensor that overflowed
    const std::vector<double> per = opt.grad_norms_per_tensor();
    EXPECT(std::isinf(per[0]) && per[1] == 0.0);
    EXPECT(opt.exchange_kind() == OXZ_EXCHANGE_NONE && opt.last_update_kernel() == OXZ_UPDATE_KERNEL_TILE);
    // the trainer's half of the step with a scaler: overflow halves the scale, the step does not count
    LossScaleConfig lc; lc.initial = 1048576.0;
    LitTrainerStep trainer(opt, LrPlan(3e-4, OXZ_LR_CONSTANT, 0, 0, 0.0), lc);
    auto [loss, norm] = trainer.training_step(2.5);
    EXPECT(loss == 2.5 && !std::isfinite(norm) && trainer.optimizer_timestep() == 1 && trainer.global_step() == 1);
    EXPECT((*trainer.loss_scale_state() == GradScalerState{524288.0, 0}));
}

int main(int argc, char** argv) {
    record_step_halves_on_overflow_and_grows_after_the_interval();
    skip_1d_keeps_norms_biases_and_ssm_tensors_out_of_decay();
    the_guard_skips_the_scripted_spike();
    lr_plan_matches_the_closed_form();
    advance_matches_one_batch_at_a_time();
    a_shuffled_epoch_reads_the_callers_permutation();
    ranks_sum_and_the_first_error_wins();
    the_meta_world_size_gates_a_resume();
    the_loader_reads_sources_ranges_and_mixtures_in_order();
    if (argc > 1 && strcmp(argv[1], "--gpu") == 0) the_step_on_the_gpu();
    printf(failures ? "%d FAILED\n" : "all passed (%d failures)\n", failures);
    return failures ? 1 : 0;
}
