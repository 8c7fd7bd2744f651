"""Terminal / static-HTML viewer for drift bundles (parity: ``rlk-drift-view``, rl_engine/validation/reports/viewer.py:
31-288; the reference's viewer is a Qt window, this one needs no display).

A bundle is a run directory: ``summary.json`` of the cross-config runner, ``paired_summary.json`` of a paired alignment
run with its ``paired/<case>/<n>/`` attempts, or ``rounds.jsonl`` of a training run.  The viewer lists the cases with
their status, shows the worst tokens of a case from its stored tensors and can write the whole view as one HTML file."""
from __future__ import annotations

import argparse
import html
import json
import sys
from pathlib import Path
from typing import Any

import torch


def load_bundle(path: str | Path) -> dict[str, Any]:
    root = Path(path)
    if root.is_file() and root.suffix == ".zip":
        from rl_kernel_b200.validation.reports.drift_report import load_drift_bundle

        rep = load_drift_bundle(root)["report"]
        return {"root": str(root), "kind": "drift_bundle", "events": [], "summary": {k: rep.get(k) for k in ("experiment_id", "overall", "bitwise")},
                "cases": {c["case_id"]: {"status": c.get("status"), "mismatch_count": c.get("mismatch_count"), "active_token_count": c.get("active_token_count"),
                                         "changed_paths": []} for c in rep.get("cases", [])}}
    if root.is_file():
        root = root.parent
    bundle: dict[str, Any] = {"root": str(root), "events": [], "cases": {}}
    for name in ("paired_summary.json", "summary.json"):
        f = root / name
        if f.exists():
            data = json.loads(f.read_text())
            bundle["kind"] = name.removesuffix(".json")
            bundle["summary"] = {k: v for k, v in data.items() if k != "cases"}
            bundle["cases"] = data.get("cases", {})
            break
    rounds = root / "rounds.jsonl"
    if rounds.exists():
        bundle.setdefault("kind", "training_rounds")
        bundle["events"] = [json.loads(line) for line in rounds.read_text().splitlines() if line.strip()]
    if "kind" not in bundle:
        raise FileNotFoundError(f"{root} holds no summary.json, paired_summary.json or rounds.jsonl")
    return bundle


def format_event(event: dict[str, Any]) -> str:
    step = event.get("step", "?")
    return (f"step {step:>5}  mismatches {event.get('mismatch_count', 0):>6} / {event.get('tokens_compared', 0):<8} "
            f"max|dlogp| {event.get('max_abs_dlogp', 0.0):.3e}  loss {event.get('loss', float('nan')):.5f}")


def format_case(case_id: str, row: dict[str, Any]) -> str:
    status = row.get("status") or ("blocked" if "blocked" in row else ("pass" if row.get("mismatch_count") == 0 else "fail"))
    mark = {"pass": "ok ", "fail": "RED", "not_executable": "n/a", "blocked": "n/a"}.get(status, status[:3])
    changed = ",".join(row.get("changed_paths", [])) or "-"
    return (f"[{mark}] {case_id:<40} mismatches {row.get('mismatch_count')!s:>6}  active {row.get('active_token_count', row.get('elements', ''))!s:>7}  "
            f"changed {changed}{'  (reused)' if row.get('reused') else ''}")


def worst_tokens(bundle: dict[str, Any], case_id: str, top: int = 10) -> list[dict[str, Any]]:
    """The ``top`` largest |training - rollout| of a paired case, from its newest sealed attempt."""
    case_dir = Path(bundle["root"]) / "paired" / case_id
    attempts = sorted((p for p in case_dir.iterdir() if p.is_dir()), key=lambda p: int(p.name)) if case_dir.exists() else []
    if not attempts:
        return []
    t = torch.load(attempts[-1] / "tensors.pt", weights_only=True)
    a, b, mask = t["rollout_logprobs"], t["training_logprobs"], t["active_mask"].bool()
    diff = (b - a).abs().masked_fill(~mask, -1.0)
    order = diff.reshape(-1).argsort(descending=True)[:top]
    cols = diff.shape[-1]
    return [{"row": int(i) // cols, "position": int(i) % cols, "rollout": float(a.reshape(-1)[i]), "training": float(b.reshape(-1)[i]),
             "abs_diff": float(diff.reshape(-1)[i])} for i in order if diff.reshape(-1)[i] >= 0]


def render_text(bundle: dict[str, Any], *, case: str | None = None, top: int = 10) -> str:
    lines = [f"bundle {bundle['root']}  ({bundle['kind']})"]
    for k, v in bundle.get("summary", {}).items():
        if isinstance(v, (str, int, float, bool)) or v is None:
            lines.append(f"  {k}: {v}")
    for cid, row in bundle["cases"].items():
        if case is None or cid == case:
            lines.append(format_case(cid, row))
    if case is not None:
        for w in worst_tokens(bundle, case, top):
            lines.append(f"    row {w['row']:>3} pos {w['position']:>5}  rollout {w['rollout']:+.6f}  training {w['training']:+.6f}  |d| {w['abs_diff']:.3e}")
    lines += [format_event(e) for e in bundle["events"][-top:]]
    return "\n".join(lines)


def render_html(bundle: dict[str, Any], *, top: int = 10) -> str:
    rows = "".join(f"<tr class='{'ok' if (r.get('mismatch_count') == 0 and 'blocked' not in r) else 'red'}'><td>{html.escape(c)}</td>"
                   f"<td>{html.escape(str(r.get('status', '')))}</td><td>{r.get('mismatch_count')}</td>"
                   f"<td>{html.escape(','.join(r.get('changed_paths', [])))}</td></tr>" for c, r in bundle["cases"].items())
    ev = "".join(f"<li><code>{html.escape(format_event(e))}</code></li>" for e in bundle["events"][-top:])
    return (f"<!doctype html><meta charset='utf-8'><title>drift view</title><style>td{{padding:2px 8px;font-family:monospace}}"
            f".red{{background:#fdd}}.ok{{background:#dfd}}</style><h3>{html.escape(bundle['root'])} ({bundle['kind']})</h3>"
            f"<table><tr><th>case</th><th>status</th><th>mismatches</th><th>changed</th></tr>{rows}</table><ul>{ev}</ul>")


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="rlk-drift-view", description=__doc__.split("\n\n")[0])
    ap.add_argument("bundle", help="run directory (or a file inside it)")
    ap.add_argument("--case", default=None, help="show the worst tokens of this case")
    ap.add_argument("--top", type=int, default=10)
    ap.add_argument("--html", default=None, help="write a static HTML view to this file")
    a = ap.parse_args(argv)
    try:
        bundle = load_bundle(a.bundle)
    except FileNotFoundError as exc:
        print(exc, file=sys.stderr)
        return 2
    if a.html:
        Path(a.html).write_text(render_html(bundle, top=a.top))
    print(render_text(bundle, case=a.case, top=a.top))
    bad = [c for c, r in bundle["cases"].items() if r.get("mismatch_count") not in (0, None)]
    return 1 if bad else 0


__all__ = ["format_case", "format_event", "load_bundle", "main", "render_html", "render_text", "worst_tokens"]

if __name__ == "__main__":
    sys.exit(main())
