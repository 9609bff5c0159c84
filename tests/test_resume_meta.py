"""The checkpoint meta's keys on the optimizer path: the cases of the reference's own unit tests
(src/dp/resume.rs:57-125, src/weight_decay/rule.rs:205-224, src/loss_scale/resume.rs, src/loss_scale/scaler.rs:291-308).
Host only: no GPU."""
import json
import math
import struct

import pytest

import oxidizr_b200 as ox


def meta_file(tmp_path, world, rows, name="checkpoint_step_3.meta.json", **more):
    path = str(tmp_path / name)
    ox.CheckpointMeta(step=3, checkpoint_file="w.safetensors", world_size=world, global_batch_rows=rows, **more).save_to(path)
    return path


def test_a_matching_world_and_batch_pass_without_a_warning(tmp_path):
    assert ox.check_resume_world(meta_file(tmp_path, 2, 8), 3, 2, 8) is None


def test_another_world_size_is_an_error_naming_both_values(tmp_path):
    with pytest.raises(ox.OxzError) as e:
        ox.check_resume_world(meta_file(tmp_path, 2, 8), 3, 1, 4)
    text = str(e.value)
    assert "world size 2" in text and "world size 1" in text and "--gpus" in text


def test_an_old_meta_reads_as_one_rank(tmp_path):
    path = meta_file(tmp_path, None, None)
    assert "world_size" not in json.load(open(path))
    assert ox.check_resume_world(path, 3, 1, 4) is None
    with pytest.raises(ox.OxzError, match="world size 1"):
        ox.check_resume_world(path, 3, 2, 8)


def test_another_global_batch_warns(tmp_path):
    warning = ox.check_resume_world(meta_file(tmp_path, 1, 4), 3, 1, 6)
    assert warning and "4 rows" in warning and "6 rows" in warning


def test_step_zero_and_no_meta_check_nothing(tmp_path):
    assert ox.check_resume_world(meta_file(tmp_path, 2, 8), 0, 1, 4) is None
    assert ox.check_resume_world(None, 5, 3, 12) is None


def test_an_unreadable_meta_is_an_error_that_names_the_file(tmp_path):
    with pytest.raises(ox.OxzError, match="was not read"):
        ox.check_resume_world(str(tmp_path / "missing.meta.json"), 3, 1, 4)
    bad = tmp_path / "bad.meta.json"
    bad.write_text('{"step": 3, "world_size": ')
    with pytest.raises(ox.OxzError, match="bad.meta.json"):
        ox.check_resume_world(str(bad), 3, 1, 4)


def test_a_meta_written_by_serde_reads_back_and_a_legacy_one_means_decay_all(tmp_path):
    # the text of src/weight_decay/rule.rs:209-210: a meta from before the rule existed
    old = tmp_path / "old.meta.json"
    old.write_text('{"step":3,"timestamp":"t","model_config_hash":"h","data_file_path":"",\n'
                   '            "data_file_hash":"","checkpoint_file":"w.safetensors"}')
    meta = ox.CheckpointMeta.load(str(old))
    assert meta.step == 3 and meta.checkpoint_file == "w.safetensors"
    assert meta.weight_decay_rule is None and meta.weight_decay_spec() == ox.WeightDecaySpec("decay_all", [])
    meta.weight_decay_rule, meta.no_decay_patterns = "skip_1d", ["embed"]
    new = str(tmp_path / "new.meta.json")
    meta.save_to(new)
    assert json.load(open(new))["weight_decay_rule"] == "skip_1d"
    assert ox.CheckpointMeta.load(new).weight_decay_spec() == ox.WeightDecaySpec("skip_1d", ["embed"])


def test_every_key_survives_a_round_trip_with_floats_bit_for_bit(tmp_path):
    scale, mean, var = 65536.0 / 3.0, 2.718281828459045e-3, 1.0000000000000002e-300
    meta = ox.CheckpointMeta(step=41, checkpoint_file="checkpoint_step_41.safetensors",
                             optimizer_file="checkpoint_step_41.optimizer.safetensors",
                             data_position=ox.DataPosition(2, 12345), weight_decay_rule="skip_1d",
                             no_decay_patterns=["embed", 'a "quoted" \\ name', "tab\there"],
                             loss_scale=ox.GradScalerState(scale, 7), world_size=8, global_batch_rows=64,
                             spike_guard=ox.SpikeGuardState(mean, var, 99, 3, 2))
    path = str(tmp_path / "m.meta.json")
    meta.save_to(path)
    back = ox.CheckpointMeta.load(path)
    assert back == meta
    bits = lambda x: struct.pack("<d", x)  # noqa: E731
    assert bits(back.loss_scale.scale) == bits(scale) and bits(back.spike_guard.variance) == bits(var)
    # any JSON reader sees the same document, keys the path does not own are present but empty
    doc = json.load(open(path))
    assert doc["world_size"] == 8 and doc["loss_scale"] == {"scale": scale, "consecutive_ok": 7}
    assert doc["data_position"] == {"epoch": 2, "row": 12345} and doc["timestamp"] == ""
    # and a document with keys in another order, nulls, and keys this path does not know still loads
    other = tmp_path / "other.meta.json"
    doc["holdout_rows"] = None
    doc["data_sources"] = [{"weights": [0.5, 0.5], "names": ["a", "b"], "nested": {"x": [1, {"y": "\u00e9"}]}}]
    doc["loss_scale"] = None
    other.write_text(json.dumps(dict(reversed(list(doc.items())))))
    again = ox.CheckpointMeta.load(str(other))
    assert again.loss_scale is None and again.world_size == 8 and again.no_decay_patterns == meta.no_decay_patterns


def test_the_loss_scale_a_resume_reads(tmp_path):
    path = meta_file(tmp_path, 1, 4, loss_scale=ox.GradScalerState(512.0, 7))
    assert ox.read_loss_scale_state(path, 3) == ox.GradScalerState(512.0, 7)
    assert ox.read_loss_scale_state(path, 0) is None          # a run at step 0
    assert ox.read_loss_scale_state(None, 3) is None          # a resume without a meta
    assert ox.read_loss_scale_state(meta_file(tmp_path, 1, 4, name="plain.meta.json"), 3) is None  # no such key
    with pytest.raises(ox.OxzError, match="loss scale"):
        ox.read_loss_scale_state(str(tmp_path / "gone.meta.json"), 3)
    # restore continues from the saved state and refuses a non-finite one (src/loss_scale/scaler.rs:291-308)
    s = ox.LossScaler(ox.LossScaleConfig(initial=65536.0))
    s.restore(ox.read_loss_scale_state(path, 3))
    assert s.state() == ox.GradScalerState(512.0, 7)
    with pytest.raises(ox.OxzError):
        s.restore(ox.GradScalerState(math.nan, 0))
    with pytest.raises(ox.OxzError, match="finite and positive"):
        ox.CheckpointMeta(step=1, loss_scale=ox.GradScalerState(math.nan, 0)).save_to(str(tmp_path / "x.json"))


def test_a_resume_must_run_the_mixture_the_meta_records(tmp_path):
    # src/data/mixture/record.rs:132-187
    saved = ox.MixtureRecord([2.0, 1.0], 12)
    path = str(tmp_path / "checkpoint_step_3.meta.json")
    ox.CheckpointMeta(step=3, checkpoint_file="w.safetensors", mixture=saved).save_to(path)
    assert ox.CheckpointMeta.load(path).mixture == saved
    ox.check_mixture_resume(path, 3, saved)
    with pytest.raises(ox.OxzError) as e:
        ox.check_mixture_resume(path, 3, None)
    assert "checkpoint_step_3.meta.json" in str(e.value) and "sets no weights" in str(e.value)
    assert "Resume with the original config, or start a fresh run." in str(e.value)
    ox.check_mixture_resume(path, 0, None)       # step 0 starts fresh
    ox.check_mixture_resume(None, 3, saved)      # no meta
    a = ox.MixtureRecord([0.7, 0.3], 100)
    pa = str(tmp_path / "a.meta.json")
    ox.CheckpointMeta(step=3, mixture=a).save_to(pa)
    plain = str(tmp_path / "plain.meta.json")
    ox.CheckpointMeta(step=3).save_to(plain)
    ox.check_mixture_resume(plain, 3, None)      # two plain runs match
    for meta, current, msg in [(pa, ox.MixtureRecord([0.7, 0.4], 100), r"trainer.data.sources\[1\].weight was 0.3, and this run sets 0.4"),
                               (pa, ox.MixtureRecord([0.7, 0.3], 90), "trainer.data.rows_per_epoch was 100, and this run reads 90"),
                               (plain, a, r"trained without trainer.data.sources weights, and this run sets weights \[0.7, 0.3\]"),
                               (pa, ox.MixtureRecord([1.0], 100), "2 weighted trainer.data.sources, and this run sets 1")]:
        with pytest.raises(ox.OxzError, match=msg):
            ox.check_mixture_resume(meta, 3, current)
    # the weights are compared by bits: the nearest other double is another mixture
    import math
    ox.check_mixture_resume(pa, 3, ox.MixtureRecord([0.7, 0.3], 100))
    with pytest.raises(ox.OxzError, match="weight was 0.3"):
        ox.check_mixture_resume(pa, 3, ox.MixtureRecord([0.7, math.nextafter(0.3, 1.0)], 100))


def test_trainer_hooks_check_the_group_and_describe_the_resume(tmp_path):
    """src/dp/trainer_hooks.rs:36-107 and src/loss_scale/scaler.rs:123-153, 291-308 through the trainer-step mirror,
    on a plan without device state (host only)."""
    class Plan:  # what LitTrainerStep needs of an optimizer on the host
        world, rank, timestep, comm = 2, 1, 0, None
    comms = ox.Communicator.local_group(2, None, timeout=5.0)
    cfg = ox.TrainerConfig(loss_scale=ox.LossScaleConfig(initial=65536.0), spike_guard=ox.SpikeGuardConfig())
    step = ox.LitTrainerStep(cfg, Plan())
    step.with_communicator(comms[1], ox.RowLayout(64, 4, 2))
    assert (step.world_size(), step.rank(), step.quiet()) == (2, 1, True)
    with pytest.raises(ValueError, match="communicator world size 2 differs from the row layout's 1"):
        step.with_communicator(comms[1], ox.RowLayout(64, 4, 1))
    hits = []
    step.with_abort_hook(lambda: hits.append(1)).abort_collectives()
    assert hits == [1]
    # restore: both present continue; a scaler without a state past step 0 and a state without a scaler only warn
    assert step.restore_loss_scale(ox.GradScalerState(512.0, 7), 3) is None
    assert step.loss_scale_state() == ox.GradScalerState(512.0, 7)
    with pytest.raises(ox.OxzError):
        step.restore_loss_scale(ox.GradScalerState(float("nan"), 0), 3)
    assert "restarts at 512" in step.restore_loss_scale(None, 3) and step.restore_loss_scale(None, 0) is None
    plain = ox.LitTrainerStep(ox.TrainerConfig(), Plan())
    assert "does not train in f16" in plain.restore_loss_scale(ox.GradScalerState(512.0, 7), 3)
    # the keys the path contributes to a checkpoint's meta, and back
    meta = step.checkpoint_meta(3, "checkpoint_step_3.safetensors", "checkpoint_step_3.optimizer.safetensors",
                                ox.WeightDecaySpec("skip_1d", ["embed"]), ox.DataPosition(0, 24))
    path = str(tmp_path / "checkpoint_step_3.meta.json")
    meta.save_to(path)
    back = ox.CheckpointMeta.load(path)
    assert back == meta and back.world_size == 2 and back.global_batch_rows == 8 and back.loss_scale.scale == 512.0
    assert ox.check_resume_world(path, 3, 2, 8) is None and ox.read_loss_scale_state(path, 3) == ox.GradScalerState(512.0, 7)
    for c in comms:
        c.destroy()
