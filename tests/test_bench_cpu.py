"""The benchmark's reference arm (`bench.py --impl reference`) on the CPU: one JSON line with the keys of the
benchmark contract from rank 0, nothing from the other ranks."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(env_extra):
    env = dict(os.environ, **env_extra)
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


def test_reference_arm_prints_one_contract_line_from_rank_zero_only():
    r = _run({"RANK": "0", "WORLD_SIZE": "1"})
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and out["metric"] == "train samples/s" and out["unit"] == "samples/s"
    assert out["higher_is_better"] is True and out["vs_baseline"] is None and out["value"] > 0
    assert out["config"]["workload"].startswith("ResNet-152")
    base = out["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == out["value"] and "batch 8" in base["sample"]
    assert out["e2e"] == {"value": out["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the other ranks of a multi-rank launch do no work and print nothing
    other = _run({"RANK": "1", "WORLD_SIZE": "2"})
    assert other.returncode == 0 and other.stdout.strip() == ""
