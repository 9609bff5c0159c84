"""The optimizer-state file: the reference's SafeTensors layout (src/checkpoint_set/optimizer_io.rs:1-5), a strict
load, bit-identical resume (tests/exact_resume.rs, tests/data_parallel_run.rs:203-230) and loading at another
world size. The file is parsed here with a few lines of Python, independently of the library's own reader."""
import json
import struct
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

import oxidizr_b200 as ox
from oxidizr_b200 import ffi
from oracle import dpstep as orc
from tests.helpers import bits, seeded_state

pytestmark = pytest.mark.gpu

TENSORS = [ox.TensorInfo("model.embed_tokens.weight", (40, 16)), ox.TensorInfo("model.layers.0.input_layernorm.weight", (16,)),
           ox.TensorInfo("model.layers.0.self_attn.q_proj.weight", (33, 16)), ox.TensorInfo("model.norm.weight", (16,)),
           ox.TensorInfo("lm_head.weight", (40, 16))]
NUMEL = [t.elements for t in TENSORS]
CFG = ox.StepConfig(max_grad_norm=1e9)


def read_safetensors(path):
    with open(path, "rb") as f:
        (hl,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hl))
        data = f.read()
    meta = header.pop("__metadata__", {})
    out = {}
    for name, e in header.items():
        dt = {"F32": np.float32, "F64": np.float64}[e["dtype"]]
        a, b = e["data_offsets"]
        out[name] = np.frombuffer(data[a:b], dtype=dt).reshape(e["shape"])
    return meta, out


def make(world, pd=ox.BF16, seed=41, steps=2, mode=None):
    plan = ox.DecayPlan(ox.WeightDecaySpec("skip_1d"), TENSORS)
    master, m, v, grads = seeded_state(NUMEL, seed, 1e-3, world, ox.BF16)
    comms = ox.Communicator.local_group(world, [0] * world, timeout=60.0) if world > 1 else [None]
    pool = ThreadPoolExecutor(world)

    def build(r):
        opt = ox.DpOptimizer(NUMEL, plan.no_decay, ox.BF16, pd, world=world, rank=r, comm=comms[r], bucket_bytes=1024, sync_mode=mode)
        for i in range(len(NUMEL)):
            opt.import_tensor(ffi.STATE_MASTER, i, master[i])
            opt.import_tensor(ffi.STATE_EXP_AVG, i, m[i])
            opt.import_tensor(ffi.STATE_EXP_AVG_SQ, i, v[i])
            opt.import_tensor(ffi.STATE_WORK, i, orc.narrow(master[i], pd))
            opt.import_tensor(ffi.STATE_GRADS, i, grads[r][i])
        return opt
    opts = list(pool.map(build, range(world)))
    for _ in range(steps):
        list(pool.map(lambda r: opts[r].step(CFG), range(world)))
    return opts, comms, pool, grads


def merged(opts, kind):
    out = []
    for i, n in enumerate(NUMEL):
        acc = np.full(n, np.nan, np.float32)
        for o in opts:
            o.export_tensor(kind, i, acc)
        out.append(acc)
    return out


def close(opts, comms):
    for o in opts:
        o.destroy()
    for c in comms:
        if c is not None:
            c.destroy()


@pytest.mark.parametrize("world", [1, 2, 3])
def test_file_has_the_reference_layout_and_every_bit(world, tmp_path):
    opts, comms, pool, _ = make(world)
    path = str(tmp_path / "ckpt_step_2.optimizer.safetensors")
    list(pool.map(lambda r: opts[r].save_optimizer(path, TENSORS), range(world)))
    meta, tensors = read_safetensors(path)
    assert meta == {"format": "oxidizr-optimizer", "optimizer": "adamw"}
    want_keys = {f"{t.name}.{s}" for t in TENSORS for s in ("exp_avg", "exp_avg_sq", "master")} | {"__step"}
    assert set(tensors) == want_keys
    assert tensors["__step"].dtype == np.float64 and tensors["__step"].tolist() == [2.0]
    for kind, suffix in ((ffi.STATE_EXP_AVG, "exp_avg"), (ffi.STATE_EXP_AVG_SQ, "exp_avg_sq"), (ffi.STATE_MASTER, "master")):
        for t, arr in zip(TENSORS, merged(opts, kind)):
            got = tensors[f"{t.name}.{suffix}"]
            assert got.shape == t.shape and np.array_equal(bits(got.reshape(-1)), bits(arr))
    close(opts, comms)


def test_full_replicas_write_the_file_the_shards_write(tmp_path):
    """With OXZ_SYNC_REPLICATED every rank holds the whole state and rank 0 alone writes it; the bytes must be the
    ones the sharded run gathers, and loading them back must reach every replica."""
    files = []
    for mode in (ox.SYNC_REPLICATED, ox.SYNC_P2P):
        opts, comms, pool, _ = make(2, mode=mode)
        path = str(tmp_path / f"mode{mode}.optimizer.safetensors")
        list(pool.map(lambda r: opts[r].save_optimizer(path, TENSORS), range(2)))
        files.append(open(path, "rb").read())
        close(opts, comms)
    assert files[0] == files[1]
    opts, comms, pool, _ = make(2, mode=ox.SYNC_REPLICATED, seed=7, steps=0)
    path = str(tmp_path / f"mode{ox.SYNC_REPLICATED}.optimizer.safetensors")
    list(pool.map(lambda r: opts[r].load_optimizer(path, TENSORS), range(2)))
    _, tensors = read_safetensors(path)
    for o in opts:
        assert o.timestep == 2
        for i, t in enumerate(TENSORS):
            assert np.array_equal(bits(o.export_tensor(ffi.STATE_EXP_AVG_SQ, i)), bits(tensors[f"{t.name}.exp_avg_sq"].reshape(-1)))
    close(opts, comms)


def test_f32_parameters_keep_no_separate_master(tmp_path):
    opts, comms, pool, _ = make(1, pd=ox.F32)
    path = str(tmp_path / "o.safetensors")
    opts[0].save_optimizer(path, TENSORS)
    _, tensors = read_safetensors(path)
    assert not any(k.endswith(".master") for k in tensors) and f"{TENSORS[0].name}.exp_avg" in tensors
    close(opts, comms)


@pytest.mark.parametrize("save_world,load_world", [(1, 1), (2, 1), (1, 2), (3, 2)])
def test_resume_is_bit_identical_also_across_world_sizes(save_world, load_world, tmp_path):
    # uninterrupted: 2 steps + 2 more. resumed: load after 2 steps into fresh optimizers, then the same 2 steps.
    path = str(tmp_path / "resume.optimizer.safetensors")
    a, ca, pa, _ = make(save_world)
    list(pa.map(lambda r: a[r].save_optimizer(path, TENSORS), range(save_world)))
    for _ in range(2):
        list(pa.map(lambda r: a[r].step(CFG), range(save_world)))
    b, cb, pb, _ = make(load_world, seed=99, steps=0)  # different initial state: the file must replace all of it
    list(pb.map(lambda r: b[r].load_optimizer(path, TENSORS), range(load_world)))
    assert all(o.timestep == 2 for o in b)
    if save_world == load_world:
        grads = seeded_state(NUMEL, 41, 1e-3, load_world, ox.BF16)[3]
        for r in range(load_world):
            for i in range(len(NUMEL)):
                b[r].import_tensor(ffi.STATE_GRADS, i, grads[r][i])
        for _ in range(2):
            list(pb.map(lambda r: b[r].step(CFG), range(load_world)))
        for kind in (ffi.STATE_MASTER, ffi.STATE_EXP_AVG, ffi.STATE_EXP_AVG_SQ):
            for x, y in zip(merged(a, kind), merged(b, kind)):
                assert np.array_equal(bits(x), bits(y))
    else:
        # another world size: the loaded state itself must carry every bit
        a2, ca2, pa2, _ = make(save_world)
        for kind in (ffi.STATE_MASTER, ffi.STATE_EXP_AVG, ffi.STATE_EXP_AVG_SQ):
            for x, y in zip(merged(a2, kind), merged(b, kind)):
                assert np.array_equal(bits(x), bits(y))
        close(a2, ca2)
    close(a, ca)
    close(b, cb)


def test_load_is_strict_and_leaves_the_state_unchanged(tmp_path):
    opts, comms, pool, _ = make(1)
    opt = opts[0]
    path = str(tmp_path / "o.safetensors")
    opt.save_optimizer(path, TENSORS)
    before = merged(opts, ffi.STATE_MASTER)
    renamed = [ox.TensorInfo("model.other.weight", TENSORS[0].shape)] + TENSORS[1:]
    with pytest.raises(ox.OxzError, match="missing key 'model.other.weight.exp_avg'"):
        opt.load_optimizer(path, renamed)
    reshaped = [ox.TensorInfo(TENSORS[0].name, (16, 40))] + TENSORS[1:]
    with pytest.raises(ox.OxzError, match="shape mismatch"):
        opt.load_optimizer(path, reshaped)
    fewer = ox.DpOptimizer(NUMEL[:-1], None, ox.BF16, ox.BF16)
    with pytest.raises(ox.OxzError, match="unknown name 'lm_head.weight"):
        fewer.load_optimizer(path, TENSORS[:-1])
    fewer.destroy()
    with pytest.raises(ox.OxzError, match="open failed"):
        opt.load_optimizer(str(tmp_path / "absent.safetensors"), TENSORS)
    with pytest.raises(ox.OxzError, match="holds 600 elements"):
        opt.save_optimizer(path, [ox.TensorInfo(TENSORS[0].name, (40, 15))] + TENSORS[1:])
    with pytest.raises(ox.OxzError, match="write failed"):
        opt.save_optimizer(str(tmp_path / "no_such_dir" / "o.safetensors"), TENSORS)
    for x, y in zip(before, merged(opts, ffi.STATE_MASTER)):
        assert np.array_equal(bits(x), bits(y))
    assert opt.timestep == 2
    close(opts, comms)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2])
def test_an_unwritable_directory_is_every_ranks_error_and_nobody_hangs(world, tmp_path):
    """tests/data_parallel_run.rs:547-568: the writing rank reports the file error; the other ranks, which only feed the
    gathers, come back instead of waiting for a rank that left early, and they too learn that nothing was written (no
    rank may take a checkpoint that does not exist for saved). An existing file stays as it was."""
    opts, comms, pool, _ = make(world)
    good = str(tmp_path / "kept.optimizer.safetensors")
    list(pool.map(lambda r: opts[r].save_optimizer(good, TENSORS), range(world)))
    kept = open(good, "rb").read()
    bad = str(tmp_path / "no_such_dir" / "o.safetensors")

    def save(r):
        try:
            opts[r].save_optimizer(bad, TENSORS)
            return None
        except ox.OxzError as e:
            return str(e)
    out = list(pool.map(save, range(world)))
    assert out[0] is not None and "write failed" in out[0] and "no_such_dir" in out[0]
    assert all(x is not None and "the writing rank could not write it" in x and "no_such_dir" in x for x in out[1:])
    assert open(good, "rb").read() == kept
    # the group is still usable: the next save succeeds
    list(pool.map(lambda r: opts[r].save_optimizer(good, TENSORS), range(world)))
    close(opts, comms)
