"""The benchmark's reference arm and command line, on CPU.

`bench.py --impl reference` times the reference's CPU path (PyTorch's CPU convolution and convolution_backward) on
the same sweep as the GPU arm and prints one JSON line with the same metric, unit and workload; under a multi-rank
launch only rank 0 runs it.  The GPU arm itself is covered by the GPU tests and by running it."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")

sys.path.insert(0, ROOT)


def _run(args, env_extra=None):
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    env.update(env_extra or {})
    return subprocess.run([sys.executable, BENCH] + args, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)


def test_reference_arm_prints_the_contract_line():
    done = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"])
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [l for l in done.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference"
    assert line["metric"] == "conv2d_fwd_bwd_tflops" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 0
    assert line["dtype"] == "f32" and line["data"] == "synthetic" and line["vs_baseline"] is None
    assert "workload" in line["config"] and "model" not in line["config"]
    # value and ms_per_step describe the same measurement: 483 GFLOP of algorithmic work per step
    flops = line["value"] * 1e12 * line["ms_per_step"] * 1e-3
    assert abs(flops / 482.9e9 - 1) < 0.01, flops
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"] and base["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_runs_on_rank_zero_only():
    done = _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                {"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert done.returncode == 0, done.stderr[-2000:]
    assert not [l for l in done.stdout.splitlines() if l.startswith("{")]


def test_sweep_flops_match_the_formula():
    import bench
    total = 0
    for cin, cout, hw, k, s, p in bench.LAYERS:
        oh = (hw + 2 * p - k) // s + 1
        per_phase = 2 * bench.BATCH * oh * oh * cout * cin * k * k
        assert bench.layer_flops(cin, cout, hw, k, s, p) == per_phase
        total += 2 * 3 * per_phase          # both layouts, three phases
    assert abs(total / 482.9e9 - 1) < 0.01


def test_gpu_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return
    done = _run(["--steps", "1", "--warmup", "0"])
    assert done.returncode != 0
    assert not [l for l in done.stdout.splitlines() if l.startswith("{")]
