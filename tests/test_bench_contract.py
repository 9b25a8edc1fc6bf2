"""The reference arm of bench.py runs on the host alone, so its side of the output contract is checked
here without a GPU: one JSON line with the agreed keys from rank 0, nothing from the other ranks."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(env_extra):
    env = dict(os.environ, BENCH_CPU_SAMPLE_ROWS="64", **env_extra)     # a small sample keeps the CPU suite short
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                           "--warmup", "1", "--gpus", env_extra.get("WORLD_SIZE", "1")],
                          capture_output=True, text=True, env=env, timeout=600)


def test_reference_arm_prints_one_contract_line():
    r = run({"OMP_NUM_THREADS": "1"})                      # as torchrun would set it
    assert r.returncode == 0, r.stderr
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "w8a8_quant_matmul_tops" and d["unit"] == "TOPS"
    assert d["higher_is_better"] is True and d["steps"] == 1 and d["value"] > 0
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["value"] == d["value"]
    assert d["cpu_baseline"]["cores"] == (os.cpu_count() or 1)          # not the single thread of the launcher
    assert d["e2e"] == {"value": d["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"] and "model" not in d["config"]


def test_reference_arm_other_ranks_print_nothing():
    r = run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"})
    assert r.returncode == 0, r.stderr
    assert r.stdout.strip() == ""
