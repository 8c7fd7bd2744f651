"""Run registered operator workloads through ``PerformanceProfiler`` and write JSON / CSV.

    python -m rl_kernel_b200.benchmarks.run_profile_suite --out suite.json [--csv suite.csv] [--only NAME ...]
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from rl_kernel_b200.benchmarks.common import PerformanceProfiler, WORKLOAD_REGISTRY


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", nargs="*", default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="")
    ap.add_argument("--csv", default="")
    ap.add_argument("--peaks", default="MEASURED_PEAKS.json", help="JSON with hbm_gbs / bf16_tflops of this box")
    a = ap.parse_args()
    peaks = json.loads(Path(a.peaks).read_text()) if a.peaks and Path(a.peaks).exists() else {}
    prof = PerformanceProfiler(iters=a.iters, peaks=peaks)
    for name in (a.only or sorted(WORKLOAD_REGISTRY)):
        r = prof.run(name)
        print(json.dumps({"name": r.name, "status": r.status, "ms": r.ms, "tflops": r.tflops, "gbs": r.gbs,
                          "tokens_per_s": r.tokens_per_s, "reason": r.reason}), flush=True)
    if a.out:
        prof.to_json(a.out)
    if a.csv:
        prof.to_csv(a.csv)


if __name__ == "__main__":
    main()
