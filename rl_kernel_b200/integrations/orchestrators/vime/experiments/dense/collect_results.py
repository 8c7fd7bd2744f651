"""Collect the arms under an experiment root into one table: JSON, CSV and a Markdown summary (parity: collect_results.py
of the reference's dense experiment)."""
from __future__ import annotations

import argparse
import csv
import json
import statistics
import sys
from pathlib import Path

from rl_kernel_b200.integrations.orchestrators.vime.experiments.dense.validate_run import validate_run

COLUMNS = ("phase", "group", "seed", "steps", "valid", "strict_mismatches", "library_mismatches", "max_abs_dlogp", "mean_step_seconds",
           "final_reward_mean", "final_grad_norm")


def collect(root: str | Path) -> list[dict]:
    rows = []
    for done in sorted(Path(root).glob("*/*/*/DONE")):
        d = done.parent
        v = validate_run(d)
        arm = json.loads((d / "arm.json").read_text())
        rounds = [json.loads(line) for line in (d / "rounds.jsonl").read_text().splitlines() if line.strip()]
        rows.append({"phase": arm["phase"], "group": arm["group"], "seed": arm["seed"], "steps": len(rounds), "valid": v["valid"],
                     "strict_mismatches": v.get("strict_mismatches"), "library_mismatches": v.get("library_mismatches"),
                     "max_abs_dlogp": v.get("max_abs_dlogp"),
                     "mean_step_seconds": statistics.fmean(r["step_seconds"] for r in rounds[1:] or rounds) if rounds else None,
                     "final_reward_mean": rounds[-1]["reward_mean"] if rounds else None,
                     "final_grad_norm": rounds[-1]["grad_norm"] if rounds else None, "issues": v["issues"]})
    return rows


def write_tables(rows: list[dict], out_dir: str | Path) -> dict[str, Path]:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "results.json").write_text(json.dumps(rows, indent=1))
    with open(out / "results.csv", "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=COLUMNS, extrasaction="ignore")
        w.writeheader()
        w.writerows(rows)
    lines = ["| " + " | ".join(COLUMNS) + " |", "|" + "---|" * len(COLUMNS)]
    for r in rows:
        lines.append("| " + " | ".join(f"{r[c]:.4g}" if isinstance(r[c], float) else str(r[c]) for c in COLUMNS) + " |")
    (out / "results.md").write_text("\n".join(lines) + "\n")
    return {"json": out / "results.json", "csv": out / "results.csv", "markdown": out / "results.md"}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("root")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    rows = collect(a.root)
    paths = write_tables(rows, a.out or Path(a.root) / "collected")
    print(json.dumps({"arms": len(rows), "invalid": [f"{r['phase']}/{r['group']}/seed{r['seed']}" for r in rows if not r["valid"]],
                      **{k: str(v) for k, v in paths.items()}}))
    return 0 if rows and all(r["valid"] for r in rows) else 2


if __name__ == "__main__":
    sys.exit(main())
