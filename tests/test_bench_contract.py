"""The bench's output contract, on the arm that needs no GPU: one JSON line with the agreed keys."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    # on the small dense set, so the CPU suite stays short; the line's shape is the same for every workload. The
    # launcher-style OMP_NUM_THREADS=1 must not reach the timed loop: the arm sets its own thread count.
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--workload", "nano_dense", "--gpus", "2"],
                         capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert out.returncode == 0, out.stderr
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "impl", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["vs_baseline"] is None and d["config"]["workload"] == "nano_dense"
    assert d["config"]["params"] == 134188544 and "whole set" in d["cpu_baseline"]["sample"]  # nothing is sampled away
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] == d["value"] > 0
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))
    assert d["product_library_mapped"] is False  # the CPU arm runs the checker alone
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_gpu_arm_refuses_to_run_without_a_gpu_instead_of_falling_back():
    import torch
    if torch.cuda.is_available():
        return
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode != 0 and "no CPU fallback" in (out.stderr + out.stdout)


def test_the_roofline_names_the_resource_that_binds_each_kernel():
    sys.path.insert(0, ROOT)
    import bench
    P = 1235814400
    one = bench.kernel_rooflines(P, 1, False, 2, 0.385, 5.394, 6555.5, None, "k_adamw", True, "bf16")
    assert one["bound"] == "hbm" and one["kernel"] == "k_adamw" and abs(one["frac"] - 28 * P / 5.394e-3 / 1e9 / 6555.5) < 1e-9
    assert one["algorithmic_bytes_per_launch"] == 28 * P and one["traffic"] is not None
    four = bench.kernel_rooflines(P, 4, False, 2, 2.772, 2.871, 6555.5, "k_pull_bulk", "k_adamw", False, "bf16")
    assert four["bound"] == "nvlink" and four["kernel"] == "k_adamw" and four["peak"] == 770.0 and four["peak_nominal"] == 900.0
    wire = 3 / 4 * 2 * P  # (W-1)/W x 2 bytes x parameters, per direction and rank
    assert four["algorithmic_bytes_per_launch"] == wire and abs(four["achieved"] - wire / 2.871e-3 / 1e9) < 1e-6
    assert [k["bound"] for k in four["kernels"]] == ["nvlink", "nvlink"] and four["kernels"][0]["kernel"] == "k_pull_bulk"
    two = bench.kernel_rooflines(P, 2, False, 2, 1.846, 3.060, 6555.5, "k_pull_bulk", "k_adamw_wide", False, "bf16")
    assert [k["bound"] for k in two["kernels"]] == ["nvlink", "hbm"] and two["bound"] == "hbm" and two["kernel"] == "k_adamw_wide"


def test_the_unrouted_experts_of_the_moe_set_are_a_fifth_of_its_parameters():
    sys.path.insert(0, ROOT)
    import bench
    from oxidizr_b200 import inventory
    tensors = inventory.moe_1b()
    gone = bench.absent_tensors(tensors)
    assert len(gone) == 12 * 2 * 3 and all(".moe.experts." in tensors[i].name for i in gone)
    assert sum(tensors[i].elements for i in gone) == 12 * 2 * 3 * 2816 * 1024
    assert bench.absent_tensors(inventory.llama_3_2_1b()) == []
