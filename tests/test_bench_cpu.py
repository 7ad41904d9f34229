"""The benchmark's reference arm (the CPU restatement of the path, timed on the host cores) and its
command line, as far as they run without a GPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=600, env=e, cwd=ROOT)


def test_reference_arm_prints_one_line_with_the_contract_keys():
    run = _run("--impl", "reference", "--steps", "1", "--warmup", "0", "--cpu-rows", "4")
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [ln for ln in run.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "w4a4_linear_tflops" and d["unit"] == "TFLOP/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] == d["value"] and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]


def test_reference_arm_runs_on_rank_zero_only():
    run = _run("--impl", "reference", "--steps", "1", "--warmup", "0", "--cpu-rows", "4",
               env={"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"})
    assert run.returncode == 0 and run.stdout.strip() == ""


def test_own_arm_refuses_to_run_without_a_gpu():
    import torch

    if torch.cuda.is_available():
        return
    run = _run("--steps", "1", "--warmup", "1")
    assert run.returncode != 0 and "CUDA device" in (run.stderr + run.stdout)
