"""Drift report bundle: JSON summary plus a Chrome Trace Event file that lays the cases out on a
timeline with their mismatch counts (headless; the reference's optional Qt viewer is not built:
unavailable on this box).  Parity: rl_engine/validation/reports/drift_report.py."""
from __future__ import annotations

import json
from pathlib import Path


def write_drift_report(summary: dict, out_dir: str | Path) -> dict[str, Path]:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    events = []
    for i, (name, c) in enumerate(sorted(summary.get("cases", {}).items())):
        events.append({"name": name, "cat": "case", "ph": "X", "ts": i * 1000, "dur": 900, "pid": 1, "tid": 1,
                       "args": {k: c.get(k) for k in ("mismatch_count", "max_abs", "mean_abs", "first_mismatch", "reused")}})
        events.append({"name": "mismatch_count", "ph": "C", "ts": i * 1000, "pid": 1, "args": {"count": c.get("mismatch_count", 0)}})
    paths = {"summary": out / "drift_summary.json", "trace": out / "drift_trace.json", "table": out / "drift_table.md"}
    paths["summary"].write_text(json.dumps(summary, indent=1, sort_keys=True))
    paths["trace"].write_text(json.dumps({"traceEvents": events, "displayTimeUnit": "ms"}))
    rows = ["| case | mismatches | max abs | reused |", "|---|---|---|---|"]
    for name, c in sorted(summary.get("cases", {}).items()):
        rows.append(f"| {name} | {c.get('mismatch_count')} | {c.get('max_abs', 0):.3e} | {c.get('reused')} |")
    paths["table"].write_text("\n".join(rows) + "\n")
    return paths
