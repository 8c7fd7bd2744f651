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


# ================================================================================================ reports from sealed attempts
# (parity: build_cross_config_attempt_report / build_drift_report / build_drift_trace / write_drift_bundle / load_drift_bundle /
#  render_drift_report of rl_engine/validation/reports/drift_report.py:53-730.  The reporter is downstream of execution: it
#  validates a sealed attempt, then renders the recorded comparison, token deltas and provenance; it never re-runs a model.)
import html as _html
import io as _io
import zipfile as _zipfile
from typing import Any as _Any, Mapping as _Mapping

import torch as _torch

REPORT_SCHEMA_VERSION = 2
_STATUS_LABELS = {"pass": "PASS", "warning": "WARN", "failure": "FAIL", "info": "INFO"}
_STATUS_COLORS = {"pass": "#39d98a", "warning": "#f4b942", "failure": "#ff5c77", "info": "#70a7ff"}


def _level(status: str) -> str:
    return {"pass": "pass", "fail": "failure", "not_executable": "warning", "zero_active_tokens": "warning"}.get(status, "failure" if "invalid" in status else "info")


def _worst_tokens(tensors: _Mapping[str, _torch.Tensor], top: int = 8) -> list[dict]:
    a, b, mask = tensors["rollout_logprobs"].float(), tensors["training_logprobs"].float(), tensors["active_mask"].bool()
    diff = (b - a).abs().masked_fill(~mask, -1.0).reshape(-1)
    cols = a.shape[-1]
    out = []
    for i in diff.argsort(descending=True)[:top].tolist():
        if diff[i] < 0:
            break
        out.append({"row": i // cols, "position": i % cols, "rollout": float(a.reshape(-1)[i]), "training": float(b.reshape(-1)[i]),
                    "abs_diff": float(diff[i]), "bitwise_equal": bool(a.reshape(-1)[i].view(_torch.int32) == b.reshape(-1)[i].view(_torch.int32))})
    return out


def build_cross_config_attempt_report(attempt_dir: str | Path, *, top: int = 8) -> dict:
    """Report of one sealed paired attempt (``paired/<case>/<n>/``).  An attempt whose seal does not verify is reported as a
    failure with that reason and nothing of its content is trusted."""
    from rl_kernel_b200.validation.cross_config._resume import comparison_matches, load_tensor_bundle, read_json_object, verify_seal

    d = Path(attempt_dir)
    rep: dict[str, _Any] = {"schema_version": REPORT_SCHEMA_VERSION, "attempt": str(d), "case_id": d.parent.name, "attempt_index": d.name}
    if not verify_seal(d):
        rep.update(status="failure", level="failure", reason="the attempt is not sealed or its seal does not verify")
        return rep
    request, result = read_json_object(d / "request.json"), read_json_object(d / "result.json")
    tensors = load_tensor_bundle(d / "tensors.pt")
    sides = {s: read_json_object(d / f"{s}.json") for s in ("rollout", "training") if (d / f"{s}.json").exists()}
    mask = tensors["active_mask"].bool()
    delta = (tensors["training_logprobs"].float() - tensors["rollout_logprobs"].float())[mask]
    rep.update(status=result["status"], level=_level(result["status"]), passed=result["passed"], comparable=result["comparable"],
               active_token_count=result["active_token_count"], mismatch_count=result["mismatch_count"], fixed_threshold=result.get("fixed_threshold"),
               contract_fingerprint=result.get("contract_fingerprint"), diagnostics=result.get("diagnostics", {}),
               identity_errors=result.get("identity_errors", []), artifact_errors=result.get("artifact_errors", []),
               requested=request.get("requested", {}), operators=request.get("operators", {}), execution_fingerprint=request.get("execution_fingerprint"),
               recomputed_comparison_matches=comparison_matches(result, tensors), worst_tokens=_worst_tokens(tensors, top),
               delta_histogram=_torch.histc(delta.abs().clamp(max=1.0), bins=10, min=0.0, max=1.0).tolist() if delta.numel() else [],
               sides={s: {"scorer": v.get("scorer"), "status": v.get("status"), "sha256": v.get("sha256"),
                          "actual": v.get("provenance", {}).get("actual"), "materialized": v.get("provenance", {}).get("materialized"),
                          "implementation_fingerprint": v.get("provenance", {}).get("implementation_fingerprint")} for s, v in sides.items()})
    return rep


def build_drift_report(run_dir: str | Path, *, top: int = 8) -> dict:
    """All cases of a paired run directory (newest attempt of each), plus the run-level summary if present."""
    root = Path(run_dir)
    paired = root / "paired"
    cases = []
    if paired.exists():
        for case_dir in sorted(p for p in paired.iterdir() if p.is_dir()):
            attempts = sorted((p for p in case_dir.iterdir() if p.is_dir() and p.name.isdigit()), key=lambda p: int(p.name))
            if attempts:
                cases.append(build_cross_config_attempt_report(attempts[-1], top=top))
    summary = json.loads((root / "paired_summary.json").read_text()) if (root / "paired_summary.json").exists() else {}
    levels = [c["level"] for c in cases]
    overall = "failure" if "failure" in levels else "warning" if "warning" in levels else "pass" if cases else "info"
    return {"schema_version": REPORT_SCHEMA_VERSION, "run_dir": str(root), "experiment_id": summary.get("experiment_id", root.name), "overall": overall,
            "bitwise": summary.get("bitwise"), "cases": cases, "not_executable": summary.get("not_executable", []),
            "environment": summary.get("environment", {}), "model_state": summary.get("model_state", {})}


def build_drift_trace(report: _Mapping[str, _Any]) -> dict:
    """Chrome Trace Event view: one slice per case (colour by status), a counter track of mismatches, and one instant event per
    worst token."""
    events = [{"name": "process_name", "ph": "M", "pid": 1, "args": {"name": f"drift: {report.get('experiment_id')}"}}]
    cname = {"pass": "good", "warning": "bad", "failure": "terrible", "info": "generic_work"}
    for i, c in enumerate(report.get("cases", [])):
        ts = i * 1000
        events.append({"name": c["case_id"], "cat": "case", "ph": "X", "ts": ts, "dur": 900, "pid": 1, "tid": 1, "cname": cname.get(c["level"], "generic_work"),
                       "args": {k: c.get(k) for k in ("status", "mismatch_count", "active_token_count", "fixed_threshold", "requested")}})
        events.append({"name": "mismatch_count", "ph": "C", "ts": ts, "pid": 1, "args": {"count": c.get("mismatch_count") or 0}})
        for j, w in enumerate(c.get("worst_tokens", [])[:4]):
            events.append({"name": f"row {w['row']} pos {w['position']}", "cat": "token", "ph": "i", "s": "t", "ts": ts + 100 + j * 150, "pid": 1, "tid": 2,
                           "args": w})
    return {"traceEvents": events, "displayTimeUnit": "ms", "otherData": {"schema_version": REPORT_SCHEMA_VERSION, "overall": report.get("overall")}}


def write_drift_trace(report: _Mapping[str, _Any], path: str | Path) -> Path:
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    p.write_text(json.dumps(build_drift_trace(report)))
    return p


def render_drift_report(report: _Mapping[str, _Any]) -> str:
    """One self-contained HTML page (no scripts, no external resources)."""
    esc = lambda v: _html.escape(str(v))  # noqa: E731
    badge = lambda level: f"<span style='background:{_STATUS_COLORS.get(level, '#999')};padding:1px 8px;border-radius:8px'>{_STATUS_LABELS.get(level, level)}</span>"  # noqa: E731
    parts = [f"<!doctype html><meta charset='utf-8'><title>drift report {esc(report.get('experiment_id'))}</title>",
             "<style>body{font-family:sans-serif;margin:24px}td,th{padding:2px 10px;font-family:monospace;text-align:left}table{border-collapse:collapse}"
             "tr:nth-child(even){background:#f4f4f4}</style>",
             f"<h2>{esc(report.get('experiment_id'))} {badge(report.get('overall', 'info'))}</h2><p>{esc(report.get('run_dir'))} &middot; judged "
             f"{'bitwise' if report.get('bitwise') else 'under the fixed threshold of the contract'}</p>",
             "<table><tr><th>case</th><th>status</th><th>mismatches</th><th>active</th><th>max |d|</th><th>requested</th></tr>"]
    for c in report.get("cases", []):
        parts.append(f"<tr><td>{esc(c['case_id'])}</td><td>{badge(c['level'])}</td><td>{esc(c.get('mismatch_count'))}</td><td>{esc(c.get('active_token_count'))}</td>"
                     f"<td>{esc(c.get('diagnostics', {}).get('max_abs_diff', '-'))}</td><td>{esc(json.dumps(c.get('requested', {})))}</td></tr>")
    parts.append("</table>")
    for c in report.get("cases", []):
        if not c.get("worst_tokens") or c["level"] == "pass":
            continue
        parts.append(f"<h3>{esc(c['case_id'])}: largest token differences</h3><table><tr><th>row</th><th>position</th><th>rollout</th><th>training</th><th>|d|</th></tr>")
        parts += [f"<tr><td>{w['row']}</td><td>{w['position']}</td><td>{w['rollout']:+.6f}</td><td>{w['training']:+.6f}</td><td>{w['abs_diff']:.3e}</td></tr>"
                  for w in c["worst_tokens"]]
        parts.append("</table>")
    if report.get("not_executable"):
        parts.append(f"<p>not executable on this runtime: {esc(', '.join(report['not_executable']))}</p>")
    env = report.get("environment", {})
    parts.append("<h3>environment</h3><table>" + "".join(f"<tr><td>{esc(k)}</td><td>{esc(v)}</td></tr>" for k, v in env.items() if not isinstance(v, dict)) + "</table>")
    return "".join(parts)


def write_drift_bundle(report: _Mapping[str, _Any], path: str | Path) -> Path:
    """A zip with report.json, trace.json and report.html: what ``rlk-drift-view`` and a trace viewer open."""
    p = Path(path)
    p.parent.mkdir(parents=True, exist_ok=True)
    with _zipfile.ZipFile(p, "w", _zipfile.ZIP_DEFLATED) as z:
        z.writestr("report.json", json.dumps(report, indent=1, sort_keys=True, default=str))
        z.writestr("trace.json", json.dumps(build_drift_trace(report)))
        z.writestr("report.html", render_drift_report(report))
    return p


def load_drift_bundle(path: str | Path) -> dict:
    with _zipfile.ZipFile(path) as z:
        names = set(z.namelist())
        if not {"report.json", "trace.json"} <= names:
            raise ValueError(f"{path} is not a drift bundle (has {sorted(names)})")
        report = json.loads(z.read("report.json"))
        if report.get("schema_version") != REPORT_SCHEMA_VERSION:
            raise ValueError(f"bundle schema {report.get('schema_version')} is not {REPORT_SCHEMA_VERSION}")
        return {"report": report, "trace": json.loads(z.read("trace.json")), "html": z.read("report.html").decode() if "report.html" in names else None}
