"""The four judgments of an operator: forward accuracy, forward invariance, gradient accuracy,
gradient invariance (parity: rl_engine/validation/operators/four_judgment_matrix.py:21-50).
Accuracy compares with the fp32 gold inside the precision profile's tolerance; invariance is
raw-bit equality per logical token across the batch configurations of the workload manifest."""
from __future__ import annotations

import torch

from rl_kernel_b200.contracts.diagnostics.matrices import DiagnosticMatrix
from rl_kernel_b200.validation.operators.forward_invariance import run_forward_invariance
from rl_kernel_b200.validation.operators.gradient_invariance import run_gradient_invariance
from rl_kernel_b200.validation.operators.operator_specs import OP_SPECS

JUDGMENTS = ("forward_accuracy", "forward_invariance", "gradient_accuracy", "gradient_invariance")


def judge_operator(op_name: str, device="cpu", dtype=torch.float32, seed: int = 0, candidate: str = "auto") -> dict[str, tuple[str, str]]:
    spec = OP_SPECS[op_name]
    out: dict[str, tuple[str, str]] = {}
    if spec.grad_input_names:
        rep = run_gradient_invariance(op_name, candidate=candidate, device=device, dtype=dtype, seed=seed)
    else:
        rep = run_forward_invariance(op_name, candidate=candidate, device=device, dtype=dtype, seed=seed)
    out["forward_accuracy"] = ("pass" if rep.accuracy_ok else "fail", f"max_err={rep.accuracy_err:.3e}")
    bad = [k for k, c in rep.configs.items() if not c.ok]
    out["forward_invariance"] = ("pass" if not bad else "fail",
                                 ",".join(f"{k}({rep.configs[k].mismatched}/{rep.configs[k].tokens})" for k in bad))
    if spec.grad_input_names:
        out["gradient_accuracy"] = ("pass" if rep.grad_accuracy_ok else "fail", f"max_rel_err={rep.grad_accuracy_err:.3e}")
        badg = [f"{k}:d{n}" for k, per in rep.grad_configs.items() for n, c in per.items() if not c.ok]
        out["gradient_invariance"] = ("pass" if not badg else "fail", ",".join(badg))
    else:
        out["gradient_accuracy"] = out["gradient_invariance"] = ("pass", "no differentiable inputs")
    return out


def four_judgment_matrix(op_names=None, device="cpu", dtype=torch.float32, candidate: str = "auto") -> DiagnosticMatrix:
    names = list(op_names or OP_SPECS)
    m = DiagnosticMatrix("four_judgments", names, list(JUDGMENTS))
    for n in names:
        try:
            res = judge_operator(n, device, dtype, candidate=candidate)
            for j, (status, detail) in res.items():
                m.set(n, j, status, detail)
        except Exception as exc:  # noqa: BLE001 - a crashing operator is a red cell, not a crashed report
            for j in JUDGMENTS:
                m.set(n, j, "blocked", f"{type(exc).__name__}: {exc}")
    return m


# ------------------------------------------------------------------------------------------------ coverage grid
# Which (backend profile, required operator, tier, judgment) cells exist, which representative case of the manifest stands
# for each, and whether it is covered -- decided without running a kernel, then filled in from executed judgments
# (parity: MatrixCell / MatrixReport / build_classified_matrix, rl_engine/validation/operators/four_judgment_matrix.py:55-265).
from dataclasses import dataclass, field  # noqa: E402
from typing import Any, Mapping, Sequence  # noqa: E402

from rl_kernel_b200.config.workload import load_manifest  # noqa: E402
from rl_kernel_b200.validation.operators.gradient_adapters import ADAPTER_SPECS, PROFILE_CANDIDATE, resolve_profile_candidate  # noqa: E402

TIERS = ("short", "primary")
CELL_STATUSES = ("green", "red", "pending_execution", "N/A")
REQUIRED_OPS = ("embedding", "rms_norm", "qk_norm", "det_gemm", "rope", "attention", "swiglu", "lm_head", "linear_logp", "pack")


@dataclass(frozen=True)
class MatrixCell:
    profile: str
    op_name: str
    judgment: str
    tier: str
    case_id: str | None
    status: str
    detail: str
    candidate: str | None = None
    expected_kernel_config_id: str | None = None
    evidence_kind: str | None = None

    def to_dict(self) -> dict[str, Any]:
        return dict(self.__dict__)


@dataclass
class MatrixReport:
    cells: tuple[MatrixCell, ...]
    counts: dict[str, int] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return {"cells": [c.to_dict() for c in self.cells], "counts": dict(self.counts)}

    @property
    def green(self) -> bool:
        return all(c.status in ("green", "N/A") for c in self.cells)


def _cases_for(manifest, *, op_name: str, profile: str) -> dict[str, dict]:
    """tier -> the first representative case of ``op_name`` under ``profile`` whose fixture belongs to that tier."""
    out: dict[str, dict] = {}
    for c in manifest.representative_cases:
        if c.get("operator_spec") == op_name and profile in c.get("profile_ids", ()):
            tier = str(c.get("fixture_id", "")).split("_")[0]
            out.setdefault(tier, c)
    return out


def classify_adapter_cell(op_name: str, profile: str, manifest=None) -> tuple[str, str, str | None]:
    """(status, detail, candidate) of an operator under a profile before anything has run."""
    a = ADAPTER_SPECS[op_name]
    r = resolve_profile_candidate(a, profile, manifest)
    cand = r["expected_backend_id"]
    if a.requirement == "layout_supported":
        return "N/A", "layout_supported: profile-independent layout helper, judged by the forward / gradient invariance runs", cand
    if a.requirement == "optional_fused" and r["status"] == "optional":
        return "N/A", "optional_fused with no required chain node", None
    if r["status"] in ("missing_candidate", "untracked_missing_node"):
        return "red", f"required and {r['status']}: a required cell that cannot be judged is red, not N/A", cand
    if r["status"] == "declared" and cand:
        return "pending_execution", "declared; becomes green or red when its judgments are executed on a host of this profile", cand
    return "red", f"unclassified status {r['status']!r}", cand


def build_classified_matrix(manifest=None, *, profiles: Sequence[str] | None = None,
                            executed: Mapping[tuple[str, str], Mapping[str, tuple[str, str]]] | None = None) -> MatrixReport:
    """The grid of profiles x required operators x tiers x judgments.  ``executed[(profile, op)]`` = the result of
    ``judge_operator`` on a host of that profile ({judgment: (status, detail)}); cells without it stay
    ``pending_execution``.  A required operator without a representative case for a tier is red: untested is not N/A."""
    m = manifest or load_manifest()
    profs = tuple(profiles or m.backend_profiles)
    unknown = [p for p in profs if p not in m.backend_profiles]
    if unknown:
        raise ValueError(f"unknown backend profiles {unknown}")
    cells: list[MatrixCell] = []
    for profile in profs:
        family = m.backend_profiles[profile]["backend_family"]
        for op in REQUIRED_OPS:
            status, detail, cand = classify_adapter_cell(op, profile, m)
            cases = _cases_for(m, op_name=op, profile=profile)
            ran = (executed or {}).get((profile, op))
            for tier in TIERS:
                case = cases.get(tier)
                cid = None if case is None else str(case["case_id"])
                st_, dt_ = status, detail
                if status != "N/A":
                    if case is None and not (op == "pack" or tier == "short" and "primary" in cases):
                        st_, dt_ = "red", "required untested: the manifest has no representative case for this tier"
                    elif case is not None and cand is not None and str(case.get("expected_backend_id")) not in (family, PROFILE_CANDIDATE.get(family, family)):
                        st_, dt_ = "red", "the case's candidate is not this profile's: borrowing another path's evidence is not allowed"
                for j in JUDGMENTS:
                    s2, d2 = st_, dt_
                    if ran is not None and st_ == "pending_execution":
                        res = ran.get(j)
                        if res is not None:
                            s2, d2 = ("green" if res[0] == "pass" else "red"), res[1] or res[0]
                    cells.append(MatrixCell(profile, op, j, tier, cid, s2, d2, cand, None if case is None else str(case.get("expected_kernel_config_id")),
                                            "representative_accuracy" if j.endswith("accuracy") else "logical_config_invariance"))
    counts: dict[str, int] = {}
    for c in cells:
        counts[c.status] = counts.get(c.status, 0) + 1
    return MatrixReport(tuple(cells), counts)


def undefined_cells(report: MatrixReport) -> tuple[MatrixCell, ...]:
    return tuple(c for c in report.cells if c.status not in CELL_STATUSES)


def hidden_required_na(report: MatrixReport) -> tuple[MatrixCell, ...]:
    """Required operators must not be N/A without one of the explicit reasons."""
    ok = ("layout_supported", "profile-independent", "optional_fused")
    return tuple(c for c in report.cells if c.status == "N/A" and c.op_name != "pack" and not any(m in (c.detail or "") for m in ok))


def executed_results(profile: str, op_names: Sequence[str] | None = None, *, device="cpu", dtype=torch.float32, candidate: str = "auto"
                     ) -> dict[tuple[str, str], dict[str, tuple[str, str]]]:
    """Run the four judgments of the required operators on this host and key them for ``build_classified_matrix``."""
    out = {}
    for op in (op_names or REQUIRED_OPS):
        try:
            out[(profile, op)] = judge_operator(op, device, dtype, candidate=candidate)
        except Exception as exc:  # noqa: BLE001 - a crashing operator makes red cells
            out[(profile, op)] = {j: ("fail", f"{type(exc).__name__}: {exc}") for j in JUDGMENTS}
    return out
