"""Validate an arm directory (parity: validate_run.py of the reference's dense experiment): the run finished, has one
record per requested step, every metric is finite, the read-back shows no fallback, and -- for arms whose modules are all
strict on both sides -- no token's training log-prob differs from its rollout log-prob."""
from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

REQUIRED_FILES = ("arm.json", "rounds.jsonl", "readback.json", "summary.json", "DONE")
REQUIRED_FIELDS = ("step", "tokens_compared", "mismatch_count", "max_abs_dlogp", "reward_mean", "grad_norm", "step_seconds")


def validate_run(run_dir: str | Path) -> dict:
    d = Path(run_dir)
    issues: list[str] = []
    missing = [f for f in REQUIRED_FILES if not (d / f).exists()]
    if missing:
        return {"run_dir": str(d), "valid": False, "issues": [f"missing files: {missing}"]}
    arm = json.loads((d / "arm.json").read_text())
    rounds = [json.loads(line) for line in (d / "rounds.jsonl").read_text().splitlines() if line.strip()]
    if len(rounds) != arm["num_rollout"]:
        issues.append(f"{len(rounds)} step records for {arm['num_rollout']} requested steps")
    if [r.get("step") for r in rounds] != list(range(len(rounds))):
        issues.append("step records are not 0..n-1 in order")
    for r in rounds:
        gone = [k for k in REQUIRED_FIELDS if k not in r]
        if gone:
            issues.append(f"step {r.get('step')}: missing fields {gone}")
            continue
        bad = [k for k in ("max_abs_dlogp", "reward_mean", "grad_norm") if not math.isfinite(float(r[k]))]
        if bad:
            issues.append(f"step {r['step']}: non-finite {bad}")
        if r["tokens_compared"] <= 0:
            issues.append(f"step {r['step']}: no tokens compared")
    strict = all(arm[f"{m}_case"] == "R/R" for m in ("attention", "ffn", "logp"))
    mism = sum(r.get("mismatch_count", 0) for r in rounds)
    if (strict or arm["logp_case"] == "R/P") and mism:
        issues.append(f"{mism} strict-path mismatches: training and rollout log-probs must be bit-equal")
    rb = json.loads((d / "readback.json").read_text())
    if rb.get("fallbacks"):
        issues.append(f"operator fallbacks recorded: {rb['fallbacks']}")
    if arm["logp_case"] == "R/P" and not any("library_mismatch_count" in r for r in rounds):
        issues.append("the library log-prob arm recorded no library rescoring")
    return {"run_dir": str(d), "valid": not issues, "issues": issues, "group": arm["group"], "seed": arm["seed"], "steps": len(rounds),
            "strict_mismatches": mism, "library_mismatches": sum(r.get("library_mismatch_count", 0) for r in rounds),
            "max_abs_dlogp": max((r.get("max_abs_dlogp", 0.0) for r in rounds), default=0.0)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("run_dir", nargs="+")
    a = ap.parse_args(argv)
    reports = [validate_run(d) for d in a.run_dir]
    print(json.dumps(reports, indent=1))
    return 0 if all(r["valid"] for r in reports) else 2


if __name__ == "__main__":
    sys.exit(main())
