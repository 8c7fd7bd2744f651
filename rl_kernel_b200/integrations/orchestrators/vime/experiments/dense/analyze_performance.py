"""Stage timing and token-normalised throughput of finished arms, per group and between groups (parity:
analyze_performance.py of the reference's dense experiment; plots are written as plain SVG so that no plotting
library is needed).

Input: run directories that hold a ``rounds.jsonl`` (one JSON record per step with ``step_seconds``, ``tokens_compared``
and, when the trainer reports it, ``phase_ms``).  ``rlk run`` and the dense arms both write that file.  Output:
``performance.json`` (summary), ``performance_rows.csv`` (one row per step) and ``performance_*.svg``.

The comparison between two groups is descriptive: a bootstrap interval of the difference of mean step times (seeded, so
two invocations print the same numbers) and the ratio of the medians; warm-up steps are dropped first.
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import random
import statistics
import sys
from pathlib import Path
from typing import Any, Iterable, Sequence

PHASES = ("rollout", "ref_score", "train_fwd_bwd", "optimizer")


def load_rounds(run_dir: str | Path) -> list[dict[str, Any]]:
    p = Path(run_dir)
    p = p / "rounds.jsonl" if p.is_dir() else p
    return [json.loads(line) for line in p.read_text().splitlines() if line.strip()]


def describe(values: Sequence[float]) -> dict[str, float]:
    """count / mean / std / min / p05 / median / p95 / max of the finite entries."""
    v = sorted(float(x) for x in values if x is not None and math.isfinite(float(x)))
    if not v:
        return {"count": 0}

    def q(p: float) -> float:
        k = (len(v) - 1) * p
        lo, hi = math.floor(k), math.ceil(k)
        return v[lo] + (v[hi] - v[lo]) * (k - lo)

    return {"count": len(v), "mean": statistics.fmean(v), "std": statistics.pstdev(v) if len(v) > 1 else 0.0, "min": v[0], "p05": q(0.05),
            "median": q(0.5), "p95": q(0.95), "max": v[-1]}


def moving_average(values: Sequence[float], window: int = 10) -> list[float]:
    out, acc = [], 0.0
    for i, x in enumerate(values):
        acc += x
        if i >= window:
            acc -= values[i - window]
        out.append(acc / min(i + 1, window))
    return out


def regression(x: Sequence[float], y: Sequence[float], at: float | None = None) -> dict[str, float]:
    """Least-squares line y = a + b x with r^2, and its value at ``at`` (step time against tokens: b is seconds per token,
    a the fixed cost of a step)."""
    n = len(x)
    if n < 2 or len(y) != n:
        return {"n": n}
    mx, my = statistics.fmean(x), statistics.fmean(y)
    sxx = sum((a - mx) ** 2 for a in x)
    if sxx == 0:
        return {"n": n, "intercept": my, "slope": 0.0, "r2": 0.0, **({"at": at, "value": my} if at is not None else {})}
    b = sum((a - mx) * (c - my) for a, c in zip(x, y)) / sxx
    a0 = my - b * mx
    ss_tot = sum((c - my) ** 2 for c in y)
    ss_res = sum((c - (a0 + b * a)) ** 2 for a, c in zip(x, y))
    out = {"n": n, "intercept": a0, "slope": b, "r2": 1.0 - ss_res / ss_tot if ss_tot else 1.0}
    if at is not None:
        out.update(at=at, value=a0 + b * at)
    return out


def bootstrap_mean_difference(a: Sequence[float], b: Sequence[float], *, samples: int = 2000, seed: int = 20260812) -> dict[str, float]:
    """mean(a) - mean(b) with a percentile interval from resampling both groups with replacement."""
    if not a or not b:
        return {"n_a": len(a), "n_b": len(b)}
    rng = random.Random(seed)
    diffs = sorted(statistics.fmean(rng.choices(a, k=len(a))) - statistics.fmean(rng.choices(b, k=len(b))) for _ in range(samples))
    return {"n_a": len(a), "n_b": len(b), "difference": statistics.fmean(a) - statistics.fmean(b), "ci_low": diffs[int(0.025 * samples)],
            "ci_high": diffs[int(0.975 * samples) - 1], "samples": samples, "seed": seed}


def build_rows(group: str, rounds: Iterable[dict[str, Any]], *, tokens_per_step: int | None = None, warmup: int = 1) -> list[dict[str, Any]]:
    rows = []
    for r in rounds:
        tokens = tokens_per_step or r.get("tokens_per_step") or r.get("tokens_compared")
        sec = float(r["step_seconds"])
        row = {"group": group, "step": int(r["step"]), "warmup": int(r["step"]) < warmup, "step_seconds": sec, "tokens": tokens,
               "tokens_per_second": (tokens / sec) if tokens and sec > 0 else None, "mismatch_count": r.get("mismatch_count")}
        ph = r.get("phase_ms") or {}
        for k in PHASES:
            row[f"{k}_ms"] = ph.get(k)
        known = sum(v for v in (ph.get(k) for k in PHASES) if v is not None)
        row["other_ms"] = sec * 1e3 - known if ph else None
        rows.append(row)
    return rows


def summarize(group_rows: dict[str, list[dict[str, Any]]]) -> dict[str, Any]:
    out: dict[str, Any] = {"groups": {}, "comparisons": []}
    steady = {g: [r for r in rows if not r["warmup"]] for g, rows in group_rows.items()}
    for g, rows in steady.items():
        sec = [r["step_seconds"] for r in rows]
        tok = [r["tokens"] for r in rows if r["tokens"]]
        entry = {"steps": len(rows), "step_seconds": describe(sec), "tokens_per_second": describe([r["tokens_per_second"] for r in rows]),
                 "mismatching_tokens": sum(r["mismatch_count"] or 0 for r in rows),
                 "phases_ms": {k: describe([r[f"{k}_ms"] for r in rows]) for k in (*PHASES, "other")},
                 "drift_over_run": regression([r["step"] for r in rows], sec)}
        total = sum(entry["phases_ms"][k].get("mean", 0.0) for k in (*PHASES, "other"))
        entry["phase_share"] = {k: (entry["phases_ms"][k].get("mean", 0.0) / total if total else None) for k in (*PHASES, "other")}
        if len(set(tok)) > 1:
            entry["seconds_against_tokens"] = regression(tok, [r["step_seconds"] for r in rows if r["tokens"]], at=statistics.fmean(tok))
        out["groups"][g] = entry
    names = sorted(steady)
    for i, a in enumerate(names):
        for b in names[i + 1:]:
            sa, sb = [r["step_seconds"] for r in steady[a]], [r["step_seconds"] for r in steady[b]]
            if not sa or not sb:
                continue
            out["comparisons"].append({"a": a, "b": b, "mean_step_seconds_difference": bootstrap_mean_difference(sa, sb),
                                       "median_ratio_a_over_b": statistics.median(sa) / statistics.median(sb),
                                       "phase_mean_difference_ms": {k: (out["groups"][a]["phases_ms"][k].get("mean", 0.0)
                                                                        - out["groups"][b]["phases_ms"][k].get("mean", 0.0)) for k in PHASES}})
    return out


def write_csv(path: Path, rows: list[dict[str, Any]]) -> None:
    cols = list(rows[0]) if rows else []
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=cols)
        w.writeheader()
        w.writerows(rows)


def analyze(runs: dict[str, str | Path], out_dir: str | Path, *, tokens_per_step: int | None = None, warmup: int = 1, plots: bool = True) -> dict:
    from rl_kernel_b200.integrations.orchestrators.vime.experiments.dense.plot_results import bar_chart, line_chart

    group_rows = {g: build_rows(g, load_rounds(d), tokens_per_step=tokens_per_step, warmup=warmup) for g, d in runs.items()}
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    summary = summarize(group_rows)
    summary["inputs"] = {g: str(d) for g, d in runs.items()}
    (out / "performance.json").write_text(json.dumps(summary, indent=1))
    write_csv(out / "performance_rows.csv", [r for rows in group_rows.values() for r in rows])
    if plots:
        series = {g: [(r["step"], r["step_seconds"]) for r in rows] for g, rows in group_rows.items()}
        (out / "performance_step_seconds.svg").write_text(line_chart(series, title="seconds per step", x_label="step", y_label="s"))
        smooth = {g: list(zip([r["step"] for r in rows], moving_average([r["tokens_per_second"] or 0.0 for r in rows])))
                  for g, rows in group_rows.items()}
        (out / "performance_tokens_per_second.svg").write_text(line_chart(smooth, title="tokens / s (moving average of 10)", x_label="step",
                                                                          y_label="tokens/s"))
        shares = {g: {k: summary["groups"][g]["phases_ms"][k].get("mean", 0.0) for k in (*PHASES, "other")} for g in summary["groups"]}
        (out / "performance_phases.svg").write_text(bar_chart(shares, title="mean milliseconds per phase", y_label="ms"))
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("runs", nargs="+", help="group=run_dir (or just run_dir: the directory name is the group)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokens-per-step", type=int, default=None, help="override the per-record token count (e.g. prompt + response tokens)")
    ap.add_argument("--warmup", type=int, default=1, help="leading steps left out of the statistics")
    ap.add_argument("--no-plots", action="store_true")
    a = ap.parse_args(argv)
    runs = {}
    for item in a.runs:
        g, _, d = item.partition("=")
        runs[g if d else Path(item).name] = d or item
    s = analyze(runs, a.out, tokens_per_step=a.tokens_per_step, warmup=a.warmup, plots=not a.no_plots)
    print(json.dumps({g: {"steps": e["steps"], "median_step_seconds": e["step_seconds"].get("median"),
                          "median_tokens_per_second": e["tokens_per_second"].get("median")} for g, e in s["groups"].items()}, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
