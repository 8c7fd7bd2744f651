"""Drive a phase of the experiment matrix: one arm directory per (group, seed); finished arms are skipped, unavailable arms
are recorded with their reason (parity: run.py of the reference's dense experiment)."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from rl_kernel_b200.integrations.orchestrators.vime.experiments.dense.run_arm import ArmUnavailable, load_matrix, resolve_arm, run_arm


def plan_phase(matrix: dict, phase: str, groups: list[str] | None = None) -> list[dict]:
    ph = matrix["phases"][phase]
    names = groups or sorted(ph.get("groups") or matrix["groups"])
    arms = []
    for g in names:
        for seed in ph["seeds"]:
            arm = {"phase": phase, "group": g, "seed": seed, "dir": f"{phase}/{g}/seed{seed}"}
            try:
                resolve_arm(matrix, phase, g)
            except ArmUnavailable as exc:
                arm["unavailable"] = str(exc)
            arms.append(arm)
    return arms


def run_phase(root: str | Path, phase: str, *, preset: str = "tiny", groups: list[str] | None = None, num_rollout: int | None = None,
              dry_run: bool = False) -> dict:
    matrix = load_matrix()
    arms = plan_phase(matrix, phase, groups)
    root = Path(root)
    out = {"phase": phase, "preset": preset, "arms": {}}
    for arm in arms:
        key = arm["dir"]
        if "unavailable" in arm:
            out["arms"][key] = {"status": "unavailable", "reason": arm["unavailable"]}
        elif dry_run:
            out["arms"][key] = {"status": "planned"}
        else:
            s = run_arm(root / key, phase=phase, group=arm["group"], seed=arm["seed"], preset=preset, num_rollout=num_rollout)
            out["arms"][key] = {"status": "done", "strict_mismatches": s["strict_mismatches"], "library_mismatches": s["library_mismatches"],
                                "tokens": s["tokens"]}
    if not dry_run:
        root.mkdir(parents=True, exist_ok=True)
        (root / f"{phase}.json").write_text(json.dumps(out, indent=1, sort_keys=True))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("root")
    ap.add_argument("--phase", default="short")
    ap.add_argument("--preset", default="tiny")
    ap.add_argument("--group", action="append", default=None)
    ap.add_argument("--num-rollout", type=int, default=None)
    ap.add_argument("--dry-run", action="store_true")
    a = ap.parse_args(argv)
    out = run_phase(a.root, a.phase, preset=a.preset, groups=a.group, num_rollout=a.num_rollout, dry_run=a.dry_run)
    print(json.dumps(out, indent=1))
    bad = [k for k, v in out["arms"].items() if v.get("strict_mismatches")]
    return 2 if bad else 0


if __name__ == "__main__":
    sys.exit(main())
