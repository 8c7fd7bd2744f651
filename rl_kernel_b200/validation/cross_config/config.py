"""Strict experiment configuration for cross-configuration drift runs: unknown fields are errors,
knobs come from an allow-list (parity: rl_engine/validation/cross_config/config.py and
docs/contracts/cross_config_logprob_drift_contract.md:112-131)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from pathlib import Path

KNOB_ALLOWLIST = {
    "tp_size": (1, 2, 4, 8), "cp_size": (1, 2, 4, 8), "batch_size": None, "chunk_size": None,
    "padding": ("none", "left", "right"), "decode_from": None, "operator_override": None, "dtype": ("float32", "bfloat16"),
}


@dataclass(frozen=True)
class CaseConfig:
    name: str
    knobs: dict = field(default_factory=dict)

    def __post_init__(self):
        for k, v in self.knobs.items():
            if k not in KNOB_ALLOWLIST:
                raise ValueError(f"case {self.name!r}: knob {k!r} is not in the allow-list {sorted(KNOB_ALLOWLIST)}")
            allowed = KNOB_ALLOWLIST[k]
            if allowed is not None and v not in allowed:
                raise ValueError(f"case {self.name!r}: knob {k}={v!r} not in {allowed}")


@dataclass(frozen=True)
class ExperimentConfig:
    experiment_id: str
    reference_case: str
    cases: tuple[CaseConfig, ...]
    seed: int = 20260812
    num_sequences: int = 4
    seq_len: int = 24
    model: dict = field(default_factory=dict)
    backend: str = "reference"            # reference (CPU batch-invariant model) | engine (sm_100a Qwen3Engine) | auto

    def __post_init__(self):
        if self.backend not in ("reference", "engine", "auto"):
            raise ValueError(f"backend {self.backend!r} is not one of reference / engine / auto")
        names = [c.name for c in self.cases]
        if len(set(names)) != len(names):
            raise ValueError("case names must be unique")
        if self.reference_case not in names:
            raise ValueError(f"reference_case {self.reference_case!r} is not one of the cases")

    @classmethod
    def from_dict(cls, d: dict) -> "ExperimentConfig":
        known = {f.name for f in fields(cls)}
        unknown = set(d) - known
        if unknown:
            raise ValueError(f"unknown experiment fields: {sorted(unknown)}")
        cases = []
        for c in d.get("cases", []):
            extra = set(c) - {"name", "knobs"}
            if extra:
                raise ValueError(f"unknown case fields: {sorted(extra)}")
            cases.append(CaseConfig(c["name"], dict(c.get("knobs", {}))))
        return cls(**{**d, "cases": tuple(cases)})

    @classmethod
    def load(cls, path: str | Path) -> "ExperimentConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))


# ================================================================================================ alignment experiments
# (parity: OperatorSelection / ExperimentConfig.plan / load_config / bind_operator_selection,
#  rl_engine/validation/cross_config/config.py:59-268)
import hashlib as _hashlib
from typing import Any as _Any, Mapping as _Mapping

from rl_kernel_b200.validation.cross_config._json import strict_json_loads as _strict_loads
from rl_kernel_b200.validation.cross_config.planner import ExperimentPlan, Planner, _get_path, _plain, normalize_backend_id
from rl_kernel_b200.validation.cross_config.schema import (ExperimentCase, ExperimentDefinition, InterventionSpec, PlanningStrategy,
                                                           SemanticIdentitySpec, freeze as _freeze)

ALIGNMENT_CONFIG_SCHEMA = "cross_config.experiment_config.v1"
_TOP_KEYS = frozenset({"schema_version", "experiment_id", "scenario_id", "contract_source", "contract_version", "strategy",
                       "strict_fallback", "identity", "baseline", "interventions", "pairwise_paths", "operators", "scenario"})
_IDENTITY_KEYS = frozenset(f.name for f in fields(SemanticIdentitySpec) if f.name != "schema_version")
_THRESHOLD_WORDS = ("threshold", "atol", "rtol", "tolerance")


@dataclass(frozen=True)
class OperatorSelection:
    """The selected-log-prob implementation of each side.  ``logp.backend`` in the baseline is the both-sides shortcut;
    this explicit form exists for runs whose two sides use different implementations on purpose."""
    rollout_backend: str
    training_backend: str
    rollout_options: _Mapping[str, _Any] = field(default_factory=dict)
    training_options: _Mapping[str, _Any] = field(default_factory=dict)

    def __post_init__(self):
        object.__setattr__(self, "rollout_backend", normalize_backend_id(self.rollout_backend))
        object.__setattr__(self, "training_backend", normalize_backend_id(self.training_backend))
        object.__setattr__(self, "rollout_options", _freeze(self.rollout_options))
        object.__setattr__(self, "training_options", _freeze(self.training_options))

    def backend_for(self, target: str) -> str:
        return {"rollout": self.rollout_backend, "training": self.training_backend}[target]

    def options_for(self, target: str) -> _Mapping[str, _Any]:
        return {"rollout": self.rollout_options, "training": self.training_options}[target]

    def to_dict(self) -> dict:
        return {"selected_logprob": {t: {"backend": self.backend_for(t), "options": _plain(self.options_for(t))}
                                     for t in ("rollout", "training")}}


def _case_backend(requested: _Mapping[str, _Any]) -> str:
    return normalize_backend_id(_get_path(requested, "logp.backend") or "native")


@dataclass(frozen=True)
class AlignmentExperimentConfig:
    definition: ExperimentDefinition
    source_path: Path | None = None
    operators: OperatorSelection | None = None
    schema_version: str = ALIGNMENT_CONFIG_SCHEMA

    def to_dict(self) -> dict:
        d = self.definition.to_dict()
        d["schema_version"] = self.schema_version
        if self.operators is not None:
            d["operators"] = self.operators.to_dict()
        return d

    def plan(self, planner: Planner | None = None) -> ExperimentPlan:
        return (planner or Planner()).plan(self.definition)

    def operators_for(self, case: ExperimentCase) -> OperatorSelection:
        backend = _case_backend(case.requested)
        if self.operators is None:
            return OperatorSelection(backend, backend)
        if self.operators.rollout_backend != backend:
            raise ValueError(f"operators.selected_logprob.rollout must match the planned logp.backend: "
                             f"{self.operators.rollout_backend!r} != {backend!r}")
        return self.operators


def _reject_threshold_keys(v, prefix: str = "") -> None:
    """A config cannot carry its own tolerance: the contract is the only source of thresholds."""
    if isinstance(v, dict):
        for k, x in v.items():
            if any(w in str(k).lower() for w in _THRESHOLD_WORDS):
                raise ValueError(f"config key {prefix + str(k)!r} looks like a tolerance override; thresholds come from the contract")
            _reject_threshold_keys(x, f"{prefix}{k}.")
    elif isinstance(v, list):
        for i, x in enumerate(v):
            _reject_threshold_keys(x, f"{prefix}{i}.")


def load_config(path: str | Path) -> AlignmentExperimentConfig:
    src = Path(path)
    try:
        raw = _strict_loads(src.read_text(encoding="utf-8"))
    except (OSError, ValueError) as exc:
        raise ValueError(f"failed to load cross-configuration config {src}: {exc}") from exc
    return config_from_dict(raw, source_path=src)


def config_from_dict(raw, *, source_path: Path | None = None) -> AlignmentExperimentConfig:
    if not isinstance(raw, dict):
        raise ValueError("cross-configuration config must contain a JSON object")
    if set(raw) - _TOP_KEYS:
        raise ValueError(f"unknown config keys: {sorted(set(raw) - _TOP_KEYS)}")
    _reject_threshold_keys(raw)
    if raw.get("schema_version") != ALIGNMENT_CONFIG_SCHEMA:
        raise ValueError(f"unsupported config schema {raw.get('schema_version')!r}; expected {ALIGNMENT_CONFIG_SCHEMA!r}")
    ident = raw.get("identity")
    if not isinstance(ident, dict) or set(ident) - _IDENTITY_KEYS:
        raise ValueError(f"identity must be an object with keys from {sorted(_IDENTITY_KEYS)}")
    ivs = []
    for item in raw.get("interventions", []):
        if not isinstance(item, dict) or set(item) != {"path", "values"} or not isinstance(item["values"], list):
            raise ValueError("an intervention is {path, values[]}")
        ivs.append(InterventionSpec(item["path"], tuple(item["values"])))
    if not isinstance(raw.get("strict_fallback", True), bool):
        raise ValueError("strict_fallback must be a JSON boolean")
    ident = dict(ident)
    for k in ("token_ids", "selected_token_ids", "active_mask", "attention_mask", "position_ids"):
        if k in ident:
            ident[k] = tuple(tuple(r) for r in ident[k])
    definition = ExperimentDefinition(raw.get("experiment_id", ""), raw.get("scenario_id", ""), SemanticIdentitySpec(**ident),
                                      raw.get("baseline") or {}, tuple(ivs), raw.get("scenario") or {},
                                      PlanningStrategy(raw.get("strategy", "one_at_a_time")), raw.get("strict_fallback", True),
                                      tuple(tuple(p) for p in raw.get("pairwise_paths", [])), raw.get("contract_source", "ws1"),
                                      raw.get("contract_version", "current"))
    ops = None
    if raw.get("operators") is not None:
        sel = raw["operators"].get("selected_logprob") if isinstance(raw["operators"], dict) else None
        if not isinstance(sel, dict) or set(sel) != {"rollout", "training"}:
            raise ValueError("operators must be {selected_logprob: {rollout: {...}, training: {...}}}")
        ops = OperatorSelection(sel["rollout"]["backend"], sel["training"]["backend"], sel["rollout"].get("options", {}),
                                sel["training"].get("options", {}))
        if any(i.path == "logp.backend" for i in ivs):
            raise ValueError("explicit operators cannot be combined with logp.backend interventions")
        if ops.rollout_backend != _case_backend(definition.baseline):
            raise ValueError("operators.selected_logprob.rollout must match baseline logp.backend")
    return AlignmentExperimentConfig(definition, source_path, ops)


def bind_operator_selection(case: ExperimentCase, selection: OperatorSelection) -> ExperimentCase:
    """Extend a planned case's identity with the concrete operators: the bound case id is what artifacts and resume key on."""
    if selection.rollout_backend != _case_backend(case.requested):
        raise ValueError("rollout operator must match the planned logp.backend")
    binding = selection.to_dict()
    op_fp = _hashlib.sha256(json.dumps({"base_case_id": case.case_id, "scenario": case.scenario_fingerprint, "operators": binding},
                                       sort_keys=True, separators=(",", ":")).encode()).hexdigest()
    cid = _hashlib.sha256(f"{case.case_id}:{op_fp}".encode()).hexdigest()[:24]
    return ExperimentCase(f"cross-config-{cid}", case.experiment_id, case.scenario_id, case.identity, case.requested,
                          {"base_case_id": case.case_id, "operators": binding, "operator_fingerprint": op_fp}, case.changed_paths,
                          case.contract_fingerprint, _hashlib.sha256(f"{case.scenario_fingerprint}:{op_fp}".encode()).hexdigest())
