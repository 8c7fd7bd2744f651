"""bench.py pieces that need no GPU: the parallel plan and the reference arm's one-line answer."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_default_plan_is_one_replica_per_gpu():
    assert bench.parallel_plan(1)["name"] == "tp1"
    for n in (2, 4, 8):
        plan = bench.parallel_plan(n)
        assert (plan["tp"], plan["cp"], plan["dp"], plan["name"]) == (1, 1, n, f"dp{n}")


def test_named_plans_parse_and_must_use_every_gpu():
    plan = bench.parallel_plan(8, "tp4xcp2")
    assert (plan["tp"], plan["cp"], plan["dp"], plan["name"]) == (4, 2, 1, "tp4xcp2")
    assert bench.parse_plan("tp2xdp4") == {"tp": 2, "cp": 1, "dp": 4, "name": "tp2xdp4"}
    with pytest.raises(SystemExit):
        bench.parallel_plan(8, "tp2xcp2")
    with pytest.raises(SystemExit):
        bench.parse_plan("pp2")


def test_reference_arm_prints_one_json_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "1", "--warmup", "3"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference"
    assert "unavailable" in rec or "value" in rec
