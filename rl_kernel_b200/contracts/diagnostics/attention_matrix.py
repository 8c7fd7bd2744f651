"""The fixed one-at-a-time replay matrix for attention drift (parity: rl_engine/contracts/diagnostics/
attention_matrix.py:23-210): row A0 is the strict replay baseline, A1..A7 apply the representative probe of one
root-cause axis each (the topology axis is a comparability gate: its row must be rejected, not measured), C0..C2 are
invariant controls that must show an exact-zero drift.  Never a Cartesian product."""
from __future__ import annotations

from dataclasses import dataclass
from types import MappingProxyType
from typing import Any

from rl_kernel_b200.contracts.diagnostics.attention_axes import ATTENTION_DEBUG_AXES, ATTENTION_INVARIANT_CONTROLS
from rl_kernel_b200.contracts.operators.attention import AttentionContractError

ATTENTION_DEBUG_MATRIX_SCHEMA_VERSION = "rlkernel.attention.debug_matrix.v1"
_EXPECTED = {"baseline": "baseline", "root_cause": "diagnostic", "comparability_gate": "rejected", "invariant_control": "exact_zero"}
GATE_AXIS = "topology_head_ownership"


@dataclass(frozen=True)
class AttentionDebugMatrixRow:
    row_id: str
    label: str
    category: str
    probe: str | None = None
    root_cause_axis: str | None = None
    expected: str = "diagnostic"

    def __post_init__(self) -> None:
        if not self.row_id.strip() or not self.label.strip():
            raise ValueError("matrix rows need an id and a label")
        if self.category not in _EXPECTED:
            raise ValueError(f"unknown matrix category {self.category!r}")
        if self.expected != _EXPECTED[self.category]:
            raise ValueError(f"{self.category} rows use expected={_EXPECTED[self.category]!r}")
        if self.category == "baseline":
            if self.probe is not None or self.root_cause_axis is not None:
                raise ValueError("the baseline row names no probe and no axis")
        elif not self.probe or not self.probe.strip():
            raise ValueError("non-baseline rows need a probe")
        if self.category in ("root_cause", "comparability_gate") and not self.root_cause_axis:
            raise ValueError("root-cause and gate rows need root_cause_axis")

    def to_dict(self) -> dict[str, Any]:
        return {"id": self.row_id, "label": self.label, "category": self.category, "probe": self.probe,
                "root_cause_axis": self.root_cause_axis, "expected": self.expected}


def _rows() -> tuple[AttentionDebugMatrixRow, ...]:
    rows = [AttentionDebugMatrixRow("A0", "Strict replay baseline", "baseline", expected="baseline")]
    for i, ax in enumerate(ATTENTION_DEBUG_AXES, start=1):
        gate = ax.axis_id == GATE_AXIS
        rows.append(AttentionDebugMatrixRow(f"A{i}", ax.label, "comparability_gate" if gate else "root_cause", ax.representative_subprobe,
                                            ax.axis_id, "rejected" if gate else "diagnostic"))
    rows += [AttentionDebugMatrixRow(f"C{i}", "Invariant control", "invariant_control", p, expected="exact_zero")
             for i, p in enumerate(ATTENTION_INVARIANT_CONTROLS)]
    return tuple(rows)


ATTENTION_DEBUG_MATRIX = _rows()
_BY_ID = MappingProxyType({r.row_id: r for r in ATTENTION_DEBUG_MATRIX})


def validate_attention_debug_matrix() -> None:
    if len(_BY_ID) != len(ATTENTION_DEBUG_MATRIX):
        raise RuntimeError("matrix row ids must be unique")
    if [r.row_id for r in ATTENTION_DEBUG_MATRIX if r.category == "baseline"] != ["A0"]:
        raise RuntimeError("the matrix has exactly one baseline, A0")
    diag = [r for r in ATTENTION_DEBUG_MATRIX if r.category in ("root_cause", "comparability_gate")]
    axes = {a.axis_id: a for a in ATTENTION_DEBUG_AXES}
    if sorted(r.root_cause_axis for r in diag) != sorted(axes):
        raise RuntimeError("every root-cause axis has exactly one row")
    if [r.root_cause_axis for r in diag if r.category == "comparability_gate"] != [GATE_AXIS]:
        raise RuntimeError("only topology / head ownership is a comparability gate")
    if any(r.probe != axes[r.root_cause_axis].representative_subprobe for r in diag):
        raise RuntimeError("a row applies its axis' representative probe")
    if {r.probe for r in ATTENTION_DEBUG_MATRIX if r.category == "invariant_control"} != set(ATTENTION_INVARIANT_CONTROLS):
        raise RuntimeError("invariant-control coverage is incomplete")


validate_attention_debug_matrix()


def attention_debug_matrix() -> dict[str, Any]:
    return {"schema_version": ATTENTION_DEBUG_MATRIX_SCHEMA_VERSION, "method": "fixed_replay_one_at_a_time", "baseline_row": "A0",
            "cartesian_product": False,
            "replay_identity": "same checkpoint, token IDs, selected-token IDs, masks, positions, cache metadata, and pre-update model state",
            "row_baseline": "each diagnostic row is compared with its own phase-local A0 baseline",
            "metrics": ["train_rollout_logprob_abs_diff", "mismatch_kl", "mismatch_k3_kl", "out_max_abs", "lse_max_abs", "dq_max_abs",
                        "dk_max_abs", "dv_max_abs"],
            "rows": [r.to_dict() for r in ATTENTION_DEBUG_MATRIX],
            "topology_gate": ["checkpoint/model/token identity", "TP head ownership", "CP sequence ownership", "actual Split-KV plan"]}


def attention_debug_matrix_row(row_id: str) -> AttentionDebugMatrixRow:
    if not isinstance(row_id, str) or not row_id.strip():
        raise AttentionContractError("matrix row id must be a non-empty string")
    try:
        return _BY_ID[row_id.strip()]
    except KeyError:
        raise AttentionContractError(f"unknown attention debug matrix row {row_id!r}") from None


__all__ = ["ATTENTION_DEBUG_MATRIX", "ATTENTION_DEBUG_MATRIX_SCHEMA_VERSION", "AttentionDebugMatrixRow", "GATE_AXIS",
           "attention_debug_matrix", "attention_debug_matrix_row", "validate_attention_debug_matrix"]
