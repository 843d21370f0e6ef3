"""The reference arm of bench.py (CPU only): one JSON line with the agreed keys, and nothing
from the other ranks of a multi-process launch."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CMD = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
       "--warmup", "0", "--rays", "4096", "--init-refine", "3", "--extra-levels", "2"]


def _run(extra_env=None, args=()):
    env = dict(os.environ)
    env.pop("RANK", None)
    env.update(extra_env or {})
    return subprocess.run(CMD + list(args), capture_output=True, text=True, timeout=600, env=env,
                          cwd=ROOT)


def test_reference_arm_prints_one_line_with_the_agreed_keys():
    res = _run()
    assert res.returncode == 0, res.stderr[-2000:]
    rows = [ln for ln in res.stdout.splitlines() if ln.strip()]
    assert len(rows) == 1
    line = json.loads(rows[0])
    assert line["impl"] == "reference" and line["higher_is_better"] is True
    assert line["unit"] == "Mrays/s" and line["value"] > 0 and line["ms_per_step"] > 0
    assert line["metric"].startswith("Mrays/s volume_render fwd+bwd")
    assert line["vs_baseline"] is None and line["data"] == "synthetic"
    assert "workload" in line["config"] and "model" not in line["config"]
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and "rays per step" in base["sample"]
    assert base["value"] == line["value"]
    assert line["e2e"] == {"value": line["value"], "unit": "Mrays/s", "h2d_bytes_per_step": 0,
                           "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_reference_arm_is_silent_on_other_ranks():
    res = _run({"RANK": "1", "WORLD_SIZE": "2", "LOCAL_RANK": "1"}, ["--gpus", "2"])
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_reference_arm_of_the_query_workload():
    env = dict(os.environ)
    env.pop("RANK", None)
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                          "--workload", "query", "--steps", "1", "--warmup", "0", "--points",
                          "8192", "--init-refine", "3"],
                         capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["unit"] == "Mpoints/s" and line["value"] > 0
