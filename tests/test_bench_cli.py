"""The benchmark's reference arm runs without a GPU (it times the C restatement on the host cores): its
line must parse and carry the keys the launch contract names.  CPU only."""
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run_reference_arm(extra_env=None, args=()):
    env = dict(os.environ)
    env.update(extra_env or {})
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--cpu-seconds-reference", "2", *args], capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    return lines, res


def test_reference_arm_line():
    lines, _ = run_reference_arm()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    assert d["metric"].startswith("train windows/sec") and d["unit"] == "windows/s" and d["higher_is_better"] is True
    assert d["value"] > 0 and d["n_gpus"] == 1
    assert d["dtype"] == "f32" and d["data"] == "synthetic" and d["vs_baseline"] is None
    assert "config 1 shapes" in d["config"]["workload"]
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["value"] == d["value"] and cb["cores"] >= 1 and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "windows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_uses_all_cores_under_a_launcher_and_only_rank_0_works():
    """A launcher exports OMP_NUM_THREADS=1; the arm sets the thread count itself.  Ranks other than 0 print
    nothing and exit 0."""
    lines, _ = run_reference_arm({"OMP_NUM_THREADS": "1"})
    d = json.loads(lines[0])
    assert d["cpu_baseline"]["cores"] == (os.cpu_count() or 1)
    lines, _ = run_reference_arm({"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2", "MASTER_ADDR": "127.0.0.1",
                                  "MASTER_PORT": "29999"}, args=("--gpus", "2"))
    assert lines == []
