"""Plots of collected results as stand-alone SVG files (parity: plot_results.py of the reference's dense experiment, which
draws with matplotlib; these are drawn by hand so that the experiment needs no plotting library).

``python -m ...plot_results results.csv --out plots/`` writes one figure per metric family from the table that
``collect_results`` produced for step records (``rounds.csv``) or from ``performance_rows.csv``:
consistency (mismatching tokens, largest log-prob difference), learning (reward, KL), optimisation (gradient norm, loss)
and performance (seconds per step)."""
from __future__ import annotations

import argparse
import csv
import json
import math
import sys
from pathlib import Path
from typing import Any

PALETTE = ("#2F67D8", "#E53935", "#2E9E5B", "#8E44AD", "#F39C12", "#16A085", "#7F8C8D")
W, H, ML, MR, MT, MB = 760, 360, 70, 150, 40, 50


def _esc(s: str) -> str:
    return str(s).replace("&", "&amp;").replace("<", "&lt;").replace(">", "&gt;")


def _ticks(lo: float, hi: float, n: int = 5) -> list[float]:
    if not math.isfinite(lo) or not math.isfinite(hi) or hi <= lo:
        return [lo]
    raw = (hi - lo) / n
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m * mag for m in (1, 2, 5, 10) if m * mag >= raw), default=raw)
    first = math.ceil(lo / step) * step
    return [first + i * step for i in range(int((hi - first) / step) + 1)]


def _frame(title: str, x_label: str, y_label: str, body: list[str], legend: list[tuple[str, str]]) -> str:
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" viewBox="0 0 {W} {H}" font-family="sans-serif" font-size="11">',
           f'<rect width="{W}" height="{H}" fill="white"/>', f'<text x="{ML}" y="22" font-size="14">{_esc(title)}</text>',
           f'<text x="{(ML + W - MR) / 2}" y="{H - 10}" text-anchor="middle">{_esc(x_label)}</text>',
           f'<text x="14" y="{(MT + H - MB) / 2}" text-anchor="middle" transform="rotate(-90 14 {(MT + H - MB) / 2})">{_esc(y_label)}</text>',
           f'<rect x="{ML}" y="{MT}" width="{W - ML - MR}" height="{H - MT - MB}" fill="none" stroke="#444"/>', *body]
    for i, (name, colour) in enumerate(legend):
        y = MT + 14 * i + 8
        out += [f'<rect x="{W - MR + 12}" y="{y - 8}" width="10" height="10" fill="{colour}"/>',
                f'<text x="{W - MR + 28}" y="{y + 1}">{_esc(name)}</text>']
    return "\n".join(out + ["</svg>"]) + "\n"


def line_chart(series: dict[str, list[tuple[float, float]]], *, title: str, x_label: str = "", y_label: str = "", symlog: bool = False) -> str:
    """``series``: name -> [(x, y)].  ``symlog`` draws sign(y) * log10(1 + |y|), for counts that are mostly zero."""
    def ty(v: float) -> float:
        return math.copysign(math.log10(1 + abs(v)), v) if symlog else v

    pts = {k: [(float(x), ty(float(y))) for x, y in v if y is not None and math.isfinite(float(y))] for k, v in series.items()}
    xs = [x for v in pts.values() for x, _ in v] or [0.0, 1.0]
    ys = [y for v in pts.values() for _, y in v] or [0.0, 1.0]
    x0, x1, y0, y1 = min(xs), max(xs), min(ys), max(ys)
    if x1 == x0:
        x1 = x0 + 1
    if y1 == y0:
        y0, y1 = y0 - 0.5, y1 + 0.5
    pad = 0.05 * (y1 - y0)
    y0, y1 = y0 - pad, y1 + pad
    sx = lambda x: ML + (x - x0) / (x1 - x0) * (W - ML - MR)          # noqa: E731
    sy = lambda y: H - MB - (y - y0) / (y1 - y0) * (H - MT - MB)      # noqa: E731
    body = []
    for t in _ticks(y0, y1):
        label = f"{(math.copysign(10 ** abs(t) - 1, t) if symlog else t):.4g}"
        body += [f'<line x1="{ML}" x2="{W - MR}" y1="{sy(t):.1f}" y2="{sy(t):.1f}" stroke="#D7DCE2"/>',
                 f'<text x="{ML - 6}" y="{sy(t) + 4:.1f}" text-anchor="end">{label}</text>']
    for t in _ticks(x0, x1):
        body.append(f'<text x="{sx(t):.1f}" y="{H - MB + 16}" text-anchor="middle">{t:.4g}</text>')
    legend = []
    for i, (name, v) in enumerate(pts.items()):
        colour = PALETTE[i % len(PALETTE)]
        legend.append((name, colour))
        if len(v) == 1:
            body.append(f'<circle cx="{sx(v[0][0]):.1f}" cy="{sy(v[0][1]):.1f}" r="3" fill="{colour}"/>')
        elif v:
            body.append(f'<polyline fill="none" stroke="{colour}" stroke-width="1.5" points="' + " ".join(f"{sx(x):.1f},{sy(y):.1f}" for x, y in v) + '"/>')
    return _frame(title, x_label, y_label, body, legend)


def bar_chart(groups: dict[str, dict[str, float]], *, title: str, y_label: str = "") -> str:
    """Stacked bars: group -> {part: value}; the same parts take the same colours in every bar."""
    parts = list(dict.fromkeys(k for g in groups.values() for k in g))
    top = max((sum(max(0.0, v or 0.0) for v in g.values()) for g in groups.values()), default=1.0) or 1.0
    sy = lambda y: H - MB - y / (top * 1.05) * (H - MT - MB)          # noqa: E731
    body = []
    for t in _ticks(0.0, top * 1.05):
        body += [f'<line x1="{ML}" x2="{W - MR}" y1="{sy(t):.1f}" y2="{sy(t):.1f}" stroke="#D7DCE2"/>',
                 f'<text x="{ML - 6}" y="{sy(t) + 4:.1f}" text-anchor="end">{t:.4g}</text>']
    slot = (W - ML - MR) / max(1, len(groups))
    for i, (name, g) in enumerate(groups.items()):
        x, acc = ML + i * slot + slot * 0.2, 0.0
        for j, p in enumerate(parts):
            v = max(0.0, g.get(p) or 0.0)
            body.append(f'<rect x="{x:.1f}" y="{sy(acc + v):.1f}" width="{slot * 0.6:.1f}" height="{sy(acc) - sy(acc + v):.1f}" '
                        f'fill="{PALETTE[j % len(PALETTE)]}"/>')
            acc += v
        body.append(f'<text x="{x + slot * 0.3:.1f}" y="{H - MB + 16}" text-anchor="middle">{_esc(name)}</text>')
    return _frame(title, "", y_label, body, [(p, PALETTE[j % len(PALETTE)]) for j, p in enumerate(parts)])


def _parse(value: str) -> Any:
    if value in ("", "None"):
        return None
    if value in ("True", "False"):
        return value == "True"
    try:
        return int(value)
    except ValueError:
        try:
            return float(value)
        except ValueError:
            return value


def load_rows(path: str | Path, phase: str | None = None) -> list[dict[str, Any]]:
    p = Path(path)
    if p.suffix == ".json":
        rows = json.loads(p.read_text())
    else:
        with open(p, newline="") as f:
            rows = [{k: _parse(v) for k, v in r.items()} for r in csv.DictReader(f)]
    return [r for r in rows if phase is None or r.get("phase") == phase]


def series_by_group(rows: list[dict[str, Any]], metric: str, x: str = "step") -> dict[str, list[tuple[float, float]]]:
    out: dict[str, list[tuple[float, float]]] = {}
    for r in rows:
        if r.get(metric) is None or r.get(x) is None:
            continue
        key = str(r.get("group", "run")) + (f"/seed{r['seed']}" if r.get("seed") is not None else "")
        out.setdefault(key, []).append((float(r[x]), float(r[metric])))
    return {k: sorted(v) for k, v in out.items()}


FIGURES = {"consistency": (("mismatch_count", True), ("max_abs_dlogp", True)), "learning": (("reward_mean", False), ("kl", False)),
           "optimization": (("grad_norm", False), ("loss", False)), "performance": (("step_seconds", False), ("tokens_per_second", False))}


def write_figures(rows: list[dict[str, Any]], out_dir: str | Path) -> list[Path]:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    written = []
    for family, metrics in FIGURES.items():
        for metric, symlog in metrics:
            s = series_by_group(rows, metric)
            if not s:
                continue
            p = out / f"{family}_{metric}.svg"
            p.write_text(line_chart(s, title=f"{family}: {metric}", x_label="step", y_label=metric, symlog=symlog))
            written.append(p)
    return written


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("table", help="CSV or JSON with one row per step (columns: group, seed, step, metrics...)")
    ap.add_argument("--out", required=True)
    ap.add_argument("--phase", default=None)
    a = ap.parse_args(argv)
    files = write_figures(load_rows(a.table, a.phase), a.out)
    print(json.dumps([str(f) for f in files]))
    return 0 if files else 2


if __name__ == "__main__":
    sys.exit(main())
