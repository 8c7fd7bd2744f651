"""Data model of the cross-configuration alignment experiments (parity: rl_engine/validation/cross_config/
schema.py:19-583).

An experiment fixes a *semantic identity* (checkpoint, tokenizer policy, the token matrix, which
tokens are scored), a baseline configuration and a set of single-knob interventions.  The planner
turns it into cases; an adapter materialises a case on a runtime and records what it really ran
(provenance); both sides -- rollout and training -- score the identity's tokens; a comparator
judges the pair under the tolerance contract.  Every record here is immutable, validated on
construction and serialises to canonical JSON.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, fields, is_dataclass
from enum import Enum
from types import MappingProxyType
from typing import Any, Mapping, Optional, Sequence

import torch


class ScoreSide(str, Enum):
    ROLLOUT = "rollout"
    TRAINING = "training"


class IsolationScope(str, Enum):
    """What has to be rebuilt before a knob's new value takes effect; ordered from cheapest to most expensive."""
    REQUEST = "request"
    ENGINE_CONSTRUCTION = "engine_construction"
    DISTRIBUTED_CONTEXT = "distributed_context"
    PROCESS = "process"

    @property
    def rank(self) -> int:
        return list(IsolationScope).index(self)


class PlanningStrategy(str, Enum):
    ONE_AT_A_TIME = "one_at_a_time"
    PAIRWISE = "pairwise"


class MaterializationStatus(str, Enum):
    UNSUPPORTED = "unsupported"
    APPLIED = "applied"
    FALLBACK = "fallback"
    UNOBSERVABLE = "unobservable"
    ERROR = "error"


class AlignmentStatus(str, Enum):
    PASS = "pass"
    FAIL = "fail"
    INVALID_IDENTITY = "invalid_identity"
    INVALID_ARTIFACT = "invalid_artifact"
    ZERO_ACTIVE_TOKENS = "zero_active_tokens"


def serialize_value(v: Any) -> Any:
    if isinstance(v, SerializableModel):
        return v.to_dict()
    if isinstance(v, Enum):
        return v.value
    if isinstance(v, torch.Tensor):
        t = v.detach().cpu()
        return {"dtype": str(t.dtype).removeprefix("torch."), "shape": list(t.shape), "values": t.tolist()}
    if isinstance(v, torch.dtype):
        return str(v).removeprefix("torch.")
    if isinstance(v, Mapping):
        return {str(k): serialize_value(x) for k, x in sorted(v.items(), key=lambda kv: str(kv[0]))}
    if isinstance(v, (tuple, list)):
        return [serialize_value(x) for x in v]
    if is_dataclass(v) and not isinstance(v, type):
        return {f.name: serialize_value(getattr(v, f.name)) for f in fields(v)}
    if isinstance(v, float) and not math.isfinite(v):
        raise ValueError("non-finite floats do not serialise")
    return v


class SerializableModel:
    def to_dict(self) -> dict[str, Any]:
        return {f.name: serialize_value(getattr(self, f.name)) for f in fields(self)}        # type: ignore[arg-type]

    def to_json(self, *, indent: Optional[int] = None) -> str:
        return json.dumps(self.to_dict(), indent=indent, sort_keys=True, allow_nan=False)


def freeze(v: Any) -> Any:
    if isinstance(v, Mapping):
        return MappingProxyType({str(k): freeze(x) for k, x in v.items()})
    if isinstance(v, (list, tuple)):
        return tuple(freeze(x) for x in v)
    return v


def _coerce(value: Any, enum_type):
    return value if isinstance(value, enum_type) else enum_type(value)


def _matrix(value: Sequence[Sequence[Any]], kind, name: str) -> tuple[tuple[Any, ...], ...]:
    rows = []
    for row in value:
        out = []
        for x in row:
            if kind is int and (isinstance(x, bool) or not isinstance(x, int)):
                raise ValueError(f"{name} must hold integers")
            if kind is bool and not isinstance(x, bool):
                raise ValueError(f"{name} must hold booleans")
            out.append(x)
        rows.append(tuple(out))
    if rows and any(len(r) != len(rows[0]) for r in rows):
        raise ValueError(f"{name} must be rectangular")
    return tuple(rows)


def _shape(m) -> tuple[int, int]:
    return (len(m), len(m[0]) if m else 0)


def _snapshot(t: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError("expected a tensor")
    t = t.detach().cpu().clone()
    return t.to(dtype) if dtype is not None else t


def _set(obj, name, value) -> None:
    object.__setattr__(obj, name, value)


@dataclass(frozen=True)
class SemanticIdentitySpec(SerializableModel):
    """The logical inputs that must agree before two scores may be compared numerically."""
    checkpoint_id: str
    model_version: str
    tokenizer_policy: str
    token_ids: tuple[tuple[int, ...], ...]
    selected_token_ids: tuple[tuple[int, ...], ...]
    active_mask: tuple[tuple[bool, ...], ...]
    pre_update_state: str
    tokenizer_id: str = ""
    attention_mask: tuple[tuple[bool, ...], ...] = ()
    position_ids: tuple[tuple[int, ...], ...] = ()
    cache_metadata: Mapping[str, Any] = field(default_factory=dict)
    packing_metadata: Mapping[str, Any] = field(default_factory=dict)
    schema_version: str = "cross_config.semantic_identity.v1"

    def __post_init__(self) -> None:
        if self.schema_version != "cross_config.semantic_identity.v1":
            raise ValueError("unsupported SemanticIdentitySpec schema_version")
        for name in ("checkpoint_id", "model_version", "tokenizer_policy", "pre_update_state"):
            if not getattr(self, name):
                raise ValueError(f"{name} must not be empty")
        _set(self, "token_ids", _matrix(self.token_ids, int, "token_ids"))
        _set(self, "selected_token_ids", _matrix(self.selected_token_ids, int, "selected_token_ids"))
        _set(self, "active_mask", _matrix(self.active_mask, bool, "active_mask"))
        if not self.token_ids or not self.token_ids[0]:
            raise ValueError("token_ids must contain at least one token")
        if not self.attention_mask:
            _set(self, "attention_mask", tuple(tuple(True for _ in r) for r in self.token_ids))
        _set(self, "attention_mask", _matrix(self.attention_mask, bool, "attention_mask"))
        _set(self, "position_ids", _matrix(self.position_ids, int, "position_ids"))
        _set(self, "cache_metadata", freeze(self.cache_metadata))
        _set(self, "packing_metadata", freeze(self.packing_metadata))
        want = _shape(self.token_ids)
        for name in ("selected_token_ids", "active_mask", "attention_mask"):
            if _shape(getattr(self, name)) != want:
                raise ValueError(f"{name} must have the shape of token_ids {want}")
        if self.position_ids and _shape(self.position_ids) != want:
            raise ValueError(f"position_ids must have the shape of token_ids {want}")

    @classmethod
    def from_tensors(cls, *, checkpoint_id: str, model_version: str, token_ids: torch.Tensor, selected_token_ids: torch.Tensor,
                     active_mask: torch.Tensor, tokenizer_policy: str = "ids-only", pre_update_state: str = "pre_update", **kw
                     ) -> "SemanticIdentitySpec":
        return cls(checkpoint_id, model_version, tokenizer_policy, tuple(map(tuple, token_ids.tolist())),
                   tuple(map(tuple, selected_token_ids.tolist())), tuple(map(tuple, active_mask.bool().tolist())), pre_update_state,
                   **kw)

    @property
    def active_token_count(self) -> int:
        return sum(sum(r) for r in self.active_mask)


@dataclass(frozen=True)
class ScorerSpec(SerializableModel):
    side: ScoreSide
    backend_id: str
    dtype: str
    device: str = "cpu"
    world_size: int = 1
    topology: Mapping[str, Any] = field(default_factory=dict)
    construction_options: Mapping[str, Any] = field(default_factory=dict)
    operator_overrides: Mapping[str, str] = field(default_factory=dict)
    schema_version: str = "cross_config.scorer.v1"

    def __post_init__(self) -> None:
        _set(self, "side", _coerce(self.side, ScoreSide))
        if not self.backend_id or not self.dtype:
            raise ValueError("backend_id and dtype must not be empty")
        if self.world_size < 1:
            raise ValueError("world_size must be >= 1")
        for name in ("topology", "construction_options", "operator_overrides"):
            _set(self, name, freeze(getattr(self, name)))


@dataclass(frozen=True)
class KnobDescriptor(SerializableModel):
    path: str
    lifecycle: IsolationScope
    targets: tuple[str, ...]
    allowed_values: tuple[Any, ...] = ()
    derived: bool = False
    critical: bool = True
    schema_version: str = "cross_config.knob_descriptor.v1"

    def __post_init__(self) -> None:
        _set(self, "lifecycle", _coerce(self.lifecycle, IsolationScope))
        _set(self, "targets", tuple(str(t) for t in self.targets))
        _set(self, "allowed_values", freeze(self.allowed_values))
        if not self.path or not self.targets:
            raise ValueError("path and targets must not be empty")
        if set(self.targets) - {"rollout", "training"}:
            raise ValueError("targets are rollout and / or training")


@dataclass(frozen=True)
class InterventionSpec(SerializableModel):
    path: str
    values: tuple[Any, ...]
    schema_version: str = "cross_config.intervention.v1"

    def __post_init__(self) -> None:
        if not self.path:
            raise ValueError("path must not be empty")
        _set(self, "values", freeze(self.values))
        if not self.values:
            raise ValueError("values must not be empty")


@dataclass(frozen=True)
class ExperimentDefinition(SerializableModel):
    experiment_id: str
    scenario_id: str
    identity: SemanticIdentitySpec
    baseline: Mapping[str, Any]
    interventions: tuple[InterventionSpec, ...] = ()
    scenario: Mapping[str, Any] = field(default_factory=dict)
    strategy: PlanningStrategy = PlanningStrategy.ONE_AT_A_TIME
    strict_fallback: bool = True
    pairwise_paths: tuple[tuple[str, str], ...] = ()
    contract_source: str = "ws1"
    contract_version: str = "current"
    schema_version: str = "cross_config.experiment_definition.v1"

    def __post_init__(self) -> None:
        if not self.experiment_id or not self.scenario_id:
            raise ValueError("experiment_id and scenario_id must not be empty")
        if self.contract_source != "ws1" or self.contract_version != "current":
            raise ValueError("alignment experiments are judged under contract_source='ws1', contract_version='current'")
        _set(self, "baseline", freeze(self.baseline))
        _set(self, "scenario", freeze(self.scenario))
        _set(self, "interventions", tuple(self.interventions))
        _set(self, "strategy", _coerce(self.strategy, PlanningStrategy))
        pairs = []
        for pair in self.pairwise_paths:
            if len(pair) != 2:
                raise ValueError("each pairwise_paths entry must contain exactly two paths")
            pairs.append((str(pair[0]), str(pair[1])))
        _set(self, "pairwise_paths", tuple(pairs))


@dataclass(frozen=True)
class ExperimentCase(SerializableModel):
    case_id: str
    experiment_id: str
    scenario_id: str
    identity: SemanticIdentitySpec
    requested: Mapping[str, Any]
    execution_binding: Mapping[str, Any] = field(default_factory=dict)
    changed_paths: tuple[str, ...] = ()
    contract_fingerprint: str = ""
    scenario_fingerprint: str = ""
    schema_version: str = "cross_config.experiment_case.v1"

    def __post_init__(self) -> None:
        if not self.case_id or not self.experiment_id or not self.scenario_id:
            raise ValueError("case_id, experiment_id and scenario_id must not be empty")
        _set(self, "requested", freeze(self.requested))
        _set(self, "execution_binding", freeze(self.execution_binding))
        _set(self, "changed_paths", tuple(str(p) for p in self.changed_paths))

    @property
    def is_baseline(self) -> bool:
        return not self.changed_paths


@dataclass(frozen=True)
class MaterializedCase(SerializableModel):
    case: ExperimentCase
    normalized: Mapping[str, Any]
    materialized: Mapping[str, Any]
    isolation_scope: IsolationScope
    construction_fingerprint: str = ""
    distributed_context_fingerprint: str = ""
    process_fingerprint: str = ""
    status: MaterializationStatus = MaterializationStatus.APPLIED
    evidence: Mapping[str, Any] = field(default_factory=dict)
    schema_version: str = "cross_config.materialized_case.v1"

    def __post_init__(self) -> None:
        for name in ("normalized", "materialized", "evidence"):
            _set(self, name, freeze(getattr(self, name)))
        _set(self, "isolation_scope", _coerce(self.isolation_scope, IsolationScope))
        _set(self, "status", _coerce(self.status, MaterializationStatus))


def _matches(name: str, t: torch.Tensor, m) -> None:
    want = torch.tensor(m, dtype=t.dtype)
    if want.shape != t.shape or not torch.equal(t, want):
        raise ValueError(f"{name} does not match the semantic identity")


@dataclass(frozen=True)
class CanonicalScoringBatch(SerializableModel):
    """The identity's matrices as tensors: what every scorer is handed."""
    identity: SemanticIdentitySpec
    input_ids: torch.Tensor
    selected_token_ids: torch.Tensor
    active_mask: torch.Tensor
    attention_mask: torch.Tensor
    position_ids: Optional[torch.Tensor] = None
    metadata: Mapping[str, Any] = field(default_factory=dict)
    schema_version: str = "cross_config.canonical_scoring_batch.v1"

    def __post_init__(self) -> None:
        _set(self, "input_ids", _snapshot(self.input_ids, torch.long))
        _set(self, "selected_token_ids", _snapshot(self.selected_token_ids, torch.long))
        _set(self, "active_mask", _snapshot(self.active_mask, torch.bool))
        _set(self, "attention_mask", _snapshot(self.attention_mask, torch.bool))
        if self.position_ids is not None:
            _set(self, "position_ids", _snapshot(self.position_ids, torch.long))
        _set(self, "metadata", freeze(self.metadata))
        if self.input_ids.ndim != 2:
            raise ValueError("input_ids must be [batch, seq]")
        _matches("input_ids", self.input_ids, self.identity.token_ids)
        _matches("selected_token_ids", self.selected_token_ids, self.identity.selected_token_ids)
        _matches("active_mask", self.active_mask, self.identity.active_mask)
        _matches("attention_mask", self.attention_mask, self.identity.attention_mask)
        if self.identity.position_ids:
            if self.position_ids is None:
                raise ValueError("the identity fixes position_ids; the batch must carry them")
            _matches("position_ids", self.position_ids, self.identity.position_ids)
        elif self.position_ids is not None:
            raise ValueError("the identity has no position_ids; the batch must not add any")

    @classmethod
    def from_identity(cls, identity: SemanticIdentitySpec, **metadata) -> "CanonicalScoringBatch":
        pos = torch.tensor(identity.position_ids) if identity.position_ids else None
        return cls(identity, torch.tensor(identity.token_ids), torch.tensor(identity.selected_token_ids),
                   torch.tensor(identity.active_mask), torch.tensor(identity.attention_mask), pos, metadata)


@dataclass(frozen=True)
class RuntimeProvenance(SerializableModel):
    """requested -> normalized -> materialized -> actual: what was asked for, what it means, what the adapter set, and
    what the runtime reports back."""
    requested: Mapping[str, Any]
    normalized: Mapping[str, Any]
    materialized: Mapping[str, Any]
    actual: Mapping[str, Any]
    status: MaterializationStatus = MaterializationStatus.APPLIED
    construction_fingerprint: str = ""
    distributed_context_fingerprint: str = ""
    process_fingerprint: str = ""
    implementation_fingerprint: str = ""
    evidence: Mapping[str, Any] = field(default_factory=dict)
    rank: int = 0
    world_size: int = 1
    schema_version: str = "cross_config.runtime_provenance.v1"

    def __post_init__(self) -> None:
        for name in ("requested", "normalized", "materialized", "actual", "evidence"):
            _set(self, name, freeze(getattr(self, name)))
        _set(self, "status", _coerce(self.status, MaterializationStatus))
        if self.rank < 0 or self.world_size < 1 or self.rank >= self.world_size:
            raise ValueError("rank must lie in [0, world_size)")


@dataclass(frozen=True)
class ScoreArtifact(SerializableModel):
    case_id: str
    attempt_id: str
    side: ScoreSide
    identity: SemanticIdentitySpec
    scorer: ScorerSpec
    selected_logprobs: torch.Tensor
    active_mask: torch.Tensor
    provenance: RuntimeProvenance
    schema_version: str = "cross_config.score_artifact.v1"

    def __post_init__(self) -> None:
        _set(self, "side", _coerce(self.side, ScoreSide))
        if not self.case_id or not self.attempt_id:
            raise ValueError("case_id and attempt_id must not be empty")
        if self.scorer.side is not self.side:
            raise ValueError("the scorer belongs to the other side")
        _set(self, "selected_logprobs", _snapshot(self.selected_logprobs))
        _set(self, "active_mask", _snapshot(self.active_mask, torch.bool))
        if self.selected_logprobs.shape != self.active_mask.shape:
            raise ValueError("selected_logprobs and active_mask must have one shape")


@dataclass(frozen=True)
class TokenComparisonArtifact(SerializableModel):
    rollout_logprobs: torch.Tensor
    training_logprobs: torch.Tensor
    active_mask: torch.Tensor
    absolute_diff: torch.Tensor
    mismatch_mask: torch.Tensor
    fixed_threshold: float
    schema_version: str = "cross_config.token_comparison.v1"

    def __post_init__(self) -> None:
        for name in ("rollout_logprobs", "training_logprobs", "absolute_diff"):
            _set(self, name, _snapshot(getattr(self, name)))
        _set(self, "active_mask", _snapshot(self.active_mask, torch.bool))
        _set(self, "mismatch_mask", _snapshot(self.mismatch_mask, torch.bool))
        shape = self.rollout_logprobs.shape
        for name in ("training_logprobs", "active_mask", "absolute_diff", "mismatch_mask"):
            if getattr(self, name).shape != shape:
                raise ValueError(f"{name} must have the shape of rollout_logprobs")
        if not math.isfinite(self.fixed_threshold) or self.fixed_threshold < 0.0:
            raise ValueError("fixed_threshold must be finite and non-negative")


@dataclass(frozen=True)
class AlignmentResult(SerializableModel):
    case_id: str
    attempt_id: str
    status: AlignmentStatus
    comparable: bool
    passed: bool
    active_token_count: int
    mismatch_count: int
    contract_fingerprint: str
    fixed_threshold: Optional[float] = None
    identity_errors: tuple[str, ...] = ()
    artifact_errors: tuple[str, ...] = ()
    diagnostics: Mapping[str, Any] = field(default_factory=dict)
    token_artifact: Optional[TokenComparisonArtifact] = None
    schema_version: str = "cross_config.alignment_result.v1"

    def __post_init__(self) -> None:
        _set(self, "status", _coerce(self.status, AlignmentStatus))
        _set(self, "identity_errors", tuple(self.identity_errors))
        _set(self, "artifact_errors", tuple(self.artifact_errors))
        _set(self, "diagnostics", freeze(self.diagnostics))
        if self.passed and self.status is not AlignmentStatus.PASS:
            raise ValueError("passed is only true with status PASS")
        if self.comparable and self.status not in (AlignmentStatus.PASS, AlignmentStatus.FAIL):
            raise ValueError("a comparable result is PASS or FAIL")


__all__ = ["AlignmentResult", "AlignmentStatus", "CanonicalScoringBatch", "ExperimentCase", "ExperimentDefinition", "InterventionSpec",
           "IsolationScope", "KnobDescriptor", "MaterializationStatus", "MaterializedCase", "PlanningStrategy", "RuntimeProvenance",
           "ScoreArtifact", "ScoreSide", "ScorerSpec", "SemanticIdentitySpec", "SerializableModel", "TokenComparisonArtifact", "freeze",
           "serialize_value"]
