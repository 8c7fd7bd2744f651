"""Experiment planner (parity: rl_engine/validation/cross_config/planner.py:25-573).

``Planner.plan(definition)`` turns a baseline and its interventions into a bounded, deterministic list
of cases: the baseline, one case per non-baseline value of every intervened knob, and -- under the
pairwise strategy -- the products of the named path pairs.  Knob paths are a closed set with
per-path normalisers; anything else is a structured ``PlanningIssue``.  Constraints (capability
checks supplied by a runtime) produce non-fatal issues attached to the plan.
"""
from __future__ import annotations

import copy
import hashlib
import itertools
import json
from dataclasses import dataclass
from typing import Any, Callable, Mapping, Optional, Sequence

from rl_kernel_b200.contracts.numerical import tolerance_contract_fingerprint
from rl_kernel_b200.validation.cross_config.schema import (ExperimentCase, ExperimentDefinition, IsolationScope, KnobDescriptor,
                                                           PlanningStrategy)

MAX_PLAN_CASES = 256
Normalizer = Callable[[Any], Any]
Constraint = Callable[[Mapping[str, Any], tuple[str, ...]], Sequence["PlanningIssue"]]


@dataclass(frozen=True)
class PlanningIssue:
    code: str
    reason: str
    path: Optional[str] = None
    value: Any = None

    def to_dict(self) -> dict[str, Any]:
        return {"code": self.code, "reason": self.reason, "path": self.path, "value": _plain(self.value)}


class PlanningError(ValueError):
    def __init__(self, issues: Sequence[PlanningIssue]):
        self.issues = tuple(issues)
        super().__init__("; ".join(f"{i.code}{f'[{i.path}]' if i.path else ''}: {i.reason}" for i in self.issues))


@dataclass(frozen=True)
class ExperimentPlan:
    definition: ExperimentDefinition
    cases: tuple[ExperimentCase, ...]
    issues: tuple[PlanningIssue, ...] = ()

    def to_dict(self) -> dict[str, Any]:
        return {"schema_version": "cross_config.experiment_plan.v1", "experiment_id": self.definition.experiment_id,
                "cases": [c.to_dict() for c in self.cases], "issues": [i.to_dict() for i in self.issues]}

    @property
    def baseline(self) -> ExperimentCase:
        return self.cases[0]


# ---------------------------------------------------------------------------------------------- normalisers
def _positive_int(v: Any) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ValueError("must be a positive integer")
    return v


def _strict_bool(v: Any) -> bool:
    if not isinstance(v, bool):
        raise ValueError("must be a bool")
    return v


_DTYPE_NAMES = {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp16": "float16", "half": "float16", "float16": "float16",
                "fp32": "float32", "float": "float32", "float32": "float32"}


def _normalize_dtype(v: Any) -> str:
    name = str(v).removeprefix("torch.").lower()
    if name not in _DTYPE_NAMES:
        raise ValueError(f"must be one of {sorted(set(_DTYPE_NAMES.values()))}")
    return _DTYPE_NAMES[name]


def _normalize_choice(*choices: str) -> Normalizer:
    def norm(v: Any) -> str:
        s = str(v).strip().lower()
        if s not in choices:
            raise ValueError(f"must be one of {list(choices)}")
        return s

    return norm


def normalize_backend_id(v: Any) -> str:
    """The public selected-log-prob backend shortcut: ``auto`` / ``default`` mean the runtime's own scorer, ``pytorch`` /
    ``reference`` the PyTorch reference operator, ``b200`` the sm_100a fused LM head."""
    if not isinstance(v, str) or not v.strip():
        raise ValueError("must be a non-empty backend ID")
    s = v.strip().lower().replace("-", "_")
    return {"auto": "native", "default": "native", "pytorch": "rlkernel.reference_logp", "reference": "rlkernel.reference_logp",
            "b200": "rlkernel.b200_linear_logp", "sm100": "rlkernel.b200_linear_logp"}.get(s, s)


V1_KNOB_DESCRIPTORS: tuple[KnobDescriptor, ...] = (
    KnobDescriptor("batch.size", IsolationScope.REQUEST, ("rollout", "training")),
    KnobDescriptor("rollout.tensor_parallel_size", IsolationScope.PROCESS, ("rollout",)),
    KnobDescriptor("rollout.context_parallel_size", IsolationScope.PROCESS, ("rollout",)),
    KnobDescriptor("rollout.dtype", IsolationScope.ENGINE_CONSTRUCTION, ("rollout",)),
    KnobDescriptor("rollout.enable_prefix_caching", IsolationScope.ENGINE_CONSTRUCTION, ("rollout",)),
    KnobDescriptor("rollout.enforce_eager", IsolationScope.ENGINE_CONSTRUCTION, ("rollout",)),
    KnobDescriptor("training.attention_backend", IsolationScope.ENGINE_CONSTRUCTION, ("training",),
                   allowed_values=("flash_attention_2", "sdpa", "eager", "model_default")),
    KnobDescriptor("training.compute_dtype", IsolationScope.ENGINE_CONSTRUCTION, ("training",)),
    KnobDescriptor("logp.backend", IsolationScope.ENGINE_CONSTRUCTION, ("rollout", "training"), derived=True),
    KnobDescriptor("training.sharding", IsolationScope.PROCESS, ("training",), allowed_values=("unsharded", "fsdp")),
)
V1_KNOBS: Mapping[str, KnobDescriptor] = {d.path: d for d in V1_KNOB_DESCRIPTORS}
_NORMALIZERS: Mapping[str, Normalizer] = {
    "batch.size": _positive_int, "rollout.tensor_parallel_size": _positive_int, "rollout.context_parallel_size": _positive_int,
    "rollout.dtype": _normalize_dtype, "rollout.enable_prefix_caching": _strict_bool, "rollout.enforce_eager": _strict_bool,
    "training.attention_backend": _normalize_choice("flash_attention_2", "sdpa", "eager", "model_default"),
    "training.compute_dtype": _normalize_dtype, "logp.backend": normalize_backend_id,
    "training.sharding": _normalize_choice("unsharded", "fsdp"),
}


# ---------------------------------------------------------------------------------------------- nested-path helpers
def _flatten(value: Mapping[str, Any], prefix: str = "") -> dict[str, Any]:
    out: dict[str, Any] = {}
    for k, v in value.items():
        path = f"{prefix}.{k}" if prefix else str(k)
        if isinstance(v, Mapping):
            out.update(_flatten(v, path))
        else:
            out[path] = v
    return out


def _get_path(value: Mapping[str, Any], path: str) -> Any:
    cur: Any = value
    for part in path.split("."):
        if not isinstance(cur, Mapping) or part not in cur:
            return None
        cur = cur[part]
    return cur


def _set_path(value: dict[str, Any], path: str, child: Any) -> None:
    parts = path.split(".")
    cur = value
    for part in parts[:-1]:
        cur = cur.setdefault(part, {})
    cur[parts[-1]] = child


def _plain(v: Any) -> Any:
    if isinstance(v, Mapping):
        return {str(k): _plain(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    return v


def _deep_copy_mapping(value: Mapping[str, Any]) -> dict[str, Any]:
    return copy.deepcopy(_plain(value))


def _fingerprint(value: Mapping[str, Any]) -> str:
    return hashlib.sha256(json.dumps(_plain(value), sort_keys=True, separators=(",", ":")).encode()).hexdigest()


class Planner:
    """Bounded plans from a closed knob set; knows nothing of runtimes or operators."""

    def __init__(self, *, knobs: Mapping[str, KnobDescriptor] = V1_KNOBS, normalizers: Mapping[str, Normalizer] = _NORMALIZERS,
                 constraints: Sequence[Constraint] = ()):
        self.knobs, self.normalizers, self.constraints = dict(knobs), dict(normalizers), tuple(constraints)

    # -- values
    def _normalize_value(self, path: str, value: Any) -> Any:
        knob = self.knobs[path]
        norm = self.normalizers.get(path)
        v = norm(value) if norm is not None else value
        if knob.allowed_values and v not in knob.allowed_values:
            raise ValueError(f"must be one of {list(knob.allowed_values)}")
        return v

    def normalize_requested(self, requested: Mapping[str, Any]) -> dict[str, Any]:
        issues, flat = [], {}
        for path, value in _flatten(requested).items():
            if path not in self.knobs:
                issues.append(PlanningIssue("UNSUPPORTED_PATH", "path is not a user-settable knob", path, value))
                continue
            try:
                flat[path] = self._normalize_value(path, value)
            except (TypeError, ValueError) as exc:
                issues.append(PlanningIssue("UNSUPPORTED_VALUE", str(exc), path, value))
        if issues:
            raise PlanningError(issues)
        out: dict[str, Any] = {}
        for path in sorted(flat):
            _set_path(out, path, flat[path])
        return out

    # -- definition
    def _validate_definition(self, d: ExperimentDefinition) -> list[PlanningIssue]:
        issues: list[PlanningIssue] = []
        seen: set[str] = set()
        for iv in d.interventions:
            if iv.path not in self.knobs:
                issues.append(PlanningIssue("UNSUPPORTED_PATH", "intervention path is not a knob", iv.path))
            elif self.knobs[iv.path].derived:
                issues.append(PlanningIssue("DERIVED_KNOB", "a derived knob follows other knobs and cannot be intervened on", iv.path))
            if iv.path in seen:
                issues.append(PlanningIssue("DUPLICATE_INTERVENTION", "a path may be intervened on once", iv.path))
            seen.add(iv.path)
        if d.strategy is PlanningStrategy.PAIRWISE:
            if not d.pairwise_paths:
                issues.append(PlanningIssue("PAIRWISE_WITHOUT_PAIRS", "the pairwise strategy needs pairwise_paths"))
            for a, b in d.pairwise_paths:
                for p in (a, b):
                    if p not in seen:
                        issues.append(PlanningIssue("PAIR_WITHOUT_INTERVENTION", "a paired path needs its own intervention", p))
                if a == b:
                    issues.append(PlanningIssue("DEGENERATE_PAIR", "a pair joins two different paths", a))
        elif d.pairwise_paths:
            issues.append(PlanningIssue("PAIRS_WITHOUT_STRATEGY", "pairwise_paths need strategy='pairwise'"))
        return issues

    def _case_id(self, d: ExperimentDefinition, requested: Mapping[str, Any], *, contract_fingerprint: str,
                 scenario_fingerprint: str) -> str:
        return _fingerprint({"experiment_id": d.experiment_id, "identity": d.identity.to_dict(), "requested": requested,
                             "contract": contract_fingerprint, "scenario": scenario_fingerprint})[:20]

    def isolation_scope(self, changed_paths: Sequence[str]) -> IsolationScope:
        """The most expensive lifecycle among the changed knobs: what must be rebuilt to move between two cases."""
        scopes = [self.knobs[p].lifecycle for p in changed_paths if p in self.knobs]
        return max(scopes, key=lambda s: s.rank) if scopes else IsolationScope.REQUEST

    def plan(self, definition: ExperimentDefinition) -> ExperimentPlan:
        issues = self._validate_definition(definition)
        if issues:
            raise PlanningError(issues)
        baseline = self.normalize_requested(definition.baseline)
        wanted: list[tuple[dict[str, Any], tuple[str, ...]]] = [(baseline, ())]

        def add(req: dict[str, Any], changed: tuple[str, ...]) -> None:
            if len(wanted) >= MAX_PLAN_CASES:
                raise PlanningError((PlanningIssue("PLAN_TOO_LARGE", f"a plan may contain at most {MAX_PLAN_CASES} cases",
                                                   value=MAX_PLAN_CASES),))
            wanted.append((req, changed))

        values: dict[str, tuple[Any, ...]] = {}
        for iv in definition.interventions:
            try:
                values[iv.path] = tuple(self._normalize_value(iv.path, v) for v in iv.values)
            except (TypeError, ValueError) as exc:
                raise PlanningError((PlanningIssue("UNSUPPORTED_VALUE", str(exc), iv.path, list(iv.values)),)) from exc
            base_v = _get_path(baseline, iv.path)
            for v in values[iv.path]:
                if v != base_v:
                    req = _deep_copy_mapping(baseline)
                    _set_path(req, iv.path, v)
                    add(req, (iv.path,))
        if definition.strategy is PlanningStrategy.PAIRWISE:
            for a, b in definition.pairwise_paths:
                for va, vb in itertools.product(values[a], values[b]):
                    if va == _get_path(baseline, a) or vb == _get_path(baseline, b):
                        continue
                    req = _deep_copy_mapping(baseline)
                    _set_path(req, a, va)
                    _set_path(req, b, vb)
                    add(req, tuple(sorted((a, b))))
        cfp = tolerance_contract_fingerprint()
        sfp = _fingerprint({"scenario_id": definition.scenario_id, "scenario": definition.scenario})
        cases, seen, findings = [], set(), []
        for req, changed in wanted:
            for c in self.constraints:
                findings.extend(c(req, changed))
            cid = self._case_id(definition, req, contract_fingerprint=cfp, scenario_fingerprint=sfp)
            if cid in seen:
                continue
            seen.add(cid)
            cases.append(ExperimentCase(cid, definition.experiment_id, definition.scenario_id, definition.identity, req, {}, changed,
                                        cfp, sfp))
        return ExperimentPlan(definition, tuple(cases), tuple(findings))


__all__ = ["Constraint", "ExperimentPlan", "MAX_PLAN_CASES", "Normalizer", "Planner", "PlanningError", "PlanningIssue", "V1_KNOBS",
           "V1_KNOB_DESCRIPTORS", "normalize_backend_id"]
