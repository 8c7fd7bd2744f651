"""Plan rows shared by planning and every runtime adapter (parity: rl_engine/validation/cross_config/
execution_plan.py:21-77): each planned case bound to its resolved operator selection."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from rl_kernel_b200.validation.cross_config.config import AlignmentExperimentConfig, OperatorSelection, bind_operator_selection
from rl_kernel_b200.validation.cross_config.planner import Planner, PlanningIssue
from rl_kernel_b200.validation.cross_config.schema import ExperimentCase


@dataclass(frozen=True)
class ExecutionPlanEntry:
    case: ExperimentCase
    operators: OperatorSelection
    schema_version: str = "cross_config.execution_plan_entry.v1"

    def to_dict(self) -> dict[str, Any]:
        return {"schema_version": self.schema_version, "case": self.case.to_dict(), "operators": self.operators.to_dict()}


@dataclass(frozen=True)
class ExecutionPlan:
    experiment: Mapping[str, Any]
    entries: tuple[ExecutionPlanEntry, ...]
    issues: tuple[PlanningIssue, ...] = ()
    schema_version: str = "cross_config.execution_plan.v1"

    def rows(self) -> tuple[dict[str, Any], ...]:
        return tuple(e.to_dict() for e in self.entries)


def build_execution_plan(config: AlignmentExperimentConfig, planner: Planner | None = None) -> ExecutionPlan:
    planned = config.plan(planner)
    entries = []
    for case in planned.cases:
        ops = config.operators_for(case)
        entries.append(ExecutionPlanEntry(bind_operator_selection(case, ops), ops))
    return ExecutionPlan(config.to_dict(), tuple(entries), planned.issues)


__all__ = ["ExecutionPlan", "ExecutionPlanEntry", "build_execution_plan"]
