"""bench.py's reference arm runs on CPU (the reference's own qw_cpu_attn_decode on the host
threads): its JSON line carries the keys the measurement contract asks for, and the arm does
nothing on ranks other than 0.  The GPU arm needs a device and says so."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_bench(args, env=None):
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, capture_output=True, text=True, cwd=ROOT, env=e,
                          timeout=600)


def test_reference_arm_line():
    r = run_bench(["--impl", "reference", "--workload", "c1_9b_decode_4k", "--steps", "2", "--warmup", "1"])
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["steps"] == 2 and line["warmup"] == 1
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] and line["cpu_baseline"]["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"] == "c1_9b_decode_4k" and line["vs_baseline"] is None


def test_reference_arm_only_rank_zero_works():
    r = run_bench(["--impl", "reference", "--workload", "c1_9b_decode_4k", "--steps", "1", "--warmup", "0", "--gpus", "2"],
                  env={"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_gpu_arm_needs_a_device():
    import torch
    if torch.cuda.is_available():
        return
    r = run_bench(["--steps", "1", "--warmup", "1"])
    assert r.returncode != 0 and "CUDA" in (r.stderr + r.stdout)
