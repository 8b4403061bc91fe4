"""The benchmark's reference arm runs on the CPU: check the JSON line it prints."""
import json
import os
import subprocess
import sys


def test_reference_arm_prints_one_json_line(repo_root):
    r = subprocess.run([sys.executable, os.path.join(repo_root, "bench.py"), "--impl", "reference", "--workload", "tiny",
                        "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300, cwd=repo_root)
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "TFLOP/s" and d["higher_is_better"] is True
    assert d["steps"] == 2 and d["warmup"] == 1 and d["value"] > 0 and d["ms_per_step"] > 0
    assert d["config"]["workload"] == "tiny"
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["gpu_launches"] == 0 and d["vs_baseline"] is None


def test_other_ranks_of_the_reference_arm_exit_quietly(repo_root):
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(repo_root, "bench.py"), "--impl", "reference", "--gpus", "2",
                        "--workload", "tiny", "--steps", "1", "--warmup", "0"], capture_output=True, text=True,
                       timeout=120, cwd=repo_root, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""
