"""The parts of bench.py's output contract that need no GPU: the reference arm (the reference's own CPU attention timed
on the host cores) prints one JSON line with the agreed keys on rank 0, and the other ranks of a multi-process launch
exit 0 without work or output."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BENCH = os.path.join(ROOT, "bench.py")


def _run(extra_env, *args):
    env = dict(os.environ)
    env.update(extra_env)
    return subprocess.run([sys.executable, BENCH, *args], cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    r = _run({"RANK": "0", "WORLD_SIZE": "1"}, "--impl", "reference", "--workload", "toy_f32", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["higher_is_better"] is True and d["unit"] == "TFLOP/s"
    assert d["warmup"] >= 3                      # fewer warm-up steps than three are raised to three
    assert d["value"] > 0 and d["ms_per_step"] > 0 and d["vs_baseline"] is None
    assert d["gpu_launches"] == 0
    cfg = d["config"]
    assert cfg["workload"] == "toy_f32" and (cfg["Hq"], cfg["Hkv"], cfg["S"], cfg["D"]) == (4, 4, 64, 16)
    base = d["cpu_baseline"]
    assert base["kind"] in ("reference", "port") and base["cores"] >= 1 and base["value"] == d["value"]
    assert "S=64" in base["sample"]
    e2e = d["e2e"]
    assert e2e["value"] == d["value"] and e2e["unit"] == d["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_reference_arm_on_other_ranks_exits_without_work():
    r = _run({"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"}, "--impl", "reference", "--gpus", "2")
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip() == ""


def test_product_arm_refuses_to_run_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a GPU is present")
    r = _run({"RANK": "0", "WORLD_SIZE": "1"}, "--steps", "1", "--warmup", "1", "--no-cpu-baseline", "--skip-e2e")
    assert r.returncode != 0                     # no CPU fallback for the product path
    assert "{" not in r.stdout                   # and no bench line
