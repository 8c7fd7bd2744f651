"""Attention contracts at the framework boundary.

Two jobs:

1. attach a contract to a framework's attention layers (``contract_from_layer`` and ``bind_attention_contracts(layers,
   ...)``: explicit contract > contract derived from the layer's config > refusal in strict mode);
2. decide whether a rollout-side and a training-side contract describe the same computation
   (``bind_attention_contracts(rollout_contract=..., training_contract=..., ...)`` and, from what the runtimes actually
   executed, ``bind_attention_runtime_readbacks``).  The two engines never hold *equal* contracts -- training scores
   whole context-parallel sequences, rollout runs paged chunked prefill and decode -- so fields fall into three
   tiers: IDENTITY fields must agree exactly or the pair is not comparable at all; SEMANTIC fields (the reduction:
   merge, accumulation dtype, order, downcast point; the compute dtype; split-KV plans; the input boundary and the
   projections) must agree and satisfy the mandate or the pair fails closed; everything else that is expected to
   differ (mode, backend, paging, RoPE fusion boundary) is RECORDED in the provenance.
   (parity: rl_engine/integrations/common/attention_binding.py:93-1430.)
"""
from __future__ import annotations

import hashlib
import json
from collections.abc import Mapping, Sequence
from dataclasses import dataclass, field
from enum import Enum
from types import MappingProxyType
from typing import Any

from rl_kernel_b200.contracts.operators.attention import (AttentionContract, AttentionContractError, AttentionDType, AttentionMerge,
                                                          AttentionRole, CPLayout, DowncastPoint, ReductionOrder,
                                                          SplitKVRuntimePlanSet, validate_split_kv_plan_set_alignment)
from rl_kernel_b200.ops.attention.preprocess import (ALLOWED_ATTENTION_PREPROCESS_BACKENDS, MANDATED_ATTENTION_PREPROCESS_BACKENDS,
                                                     PREPROCESS_POLICY_ID)
from rl_kernel_b200.ops.attention.projection import (DETERMINISTIC_PROJECTION_BACKEND_ID, PROJECTION_POLICY_ID,
                                                     REFERENCE_PROJECTION_BACKEND_ID)
from rl_kernel_b200.runtime.policy import strict_contract_enabled


def contract_from_layer(layer, tp_size: int = 1, cp_size: int = 1, cp_layout: str = "zigzag", *, seq_len: int | None = None,
                        batch_size: int = 1, tp_rank: int = 0, cp_rank: int = 0) -> AttentionContract:
    def pick(*names):
        for n in names:
            if hasattr(layer, n):
                return getattr(layer, n)
        raise AttributeError(f"attention layer {type(layer).__name__} exposes none of {names}")

    hq = int(pick("num_heads", "num_attention_heads", "total_num_heads"))
    hkv = int(pick("num_kv_heads", "num_key_value_heads", "total_num_kv_heads", "num_query_groups"))
    d = int(pick("head_dim", "head_size", "hidden_size_per_attention_head"))
    layout = CPLayout(cp_layout) if cp_size > 1 else CPLayout.NONE
    if seq_len is None:                      # the binding happens before any batch exists: one canonical block per chunk
        seq_len = 128 * (2 * cp_size if layout is CPLayout.ZIGZAG else cp_size)
    return AttentionContract.for_layout(hq, hkv, head_dim=d, seq_len=seq_len, batch_size=batch_size, tp_rank=tp_rank,
                                        tp_world_size=tp_size, cp_rank=cp_rank, cp_world_size=cp_size, layout=layout)


def bind_attention_contracts(layers=None, *, explicit: AttentionContract | None = None, tp_size: int = 1, cp_size: int = 1,
                             cp_layout: str = "zigzag", **pair_kwargs):
    """Two call forms.  ``bind_attention_contracts(layers, ...)`` attaches a contract to every layer and returns the
    list.  ``bind_attention_contracts(rollout_contract=..., training_contract=..., rollout_identity=...,
    training_identity=..., rollout_backend_id=..., training_backend_id=..., ...)`` compares the two engines' contracts
    (``bind_contract_pair``) and returns an ``AttentionBindingResult``."""
    if pair_kwargs:
        if layers is not None or explicit is not None:
            raise TypeError("pass either layers or the rollout / training pair, not both")
        return bind_contract_pair(**pair_kwargs)
    if layers is None:
        raise TypeError("bind_attention_contracts needs layers or a rollout / training contract pair")
    out = []
    for layer in layers:
        if explicit is not None:
            c = explicit
        else:
            try:
                c = contract_from_layer(layer, tp_size, cp_size, cp_layout)
            except (AttributeError, ValueError) as exc:
                if strict_contract_enabled():
                    raise RuntimeError(f"strict mode: cannot bind an attention contract to {type(layer).__name__}: {exc}")
                c = None
        if c is not None:
            setattr(layer, "rl_kernel_attention_contract", c)
        out.append(c)
    return out


# ------------------------------------------------------------------------------------------------ binding findings
class BindingErrorCode(str, Enum):
    """Stable machine-readable reasons a rollout / training binding is rejected (parity: BindingErrorCode,
    rl_engine/integrations/common/attention_binding.py:105-135)."""
    IDENTITY_MISSING = "IDENTITY_MISSING"
    IDENTITY_MISMATCH = "IDENTITY_MISMATCH"
    REDUCTION_SEMANTIC_MISMATCH = "REDUCTION_SEMANTIC_MISMATCH"
    REDUCTION_MANDATE_VIOLATION = "REDUCTION_MANDATE_VIOLATION"
    LSE_NOT_EXPORTED = "LSE_NOT_EXPORTED"
    ROLE_COLLISION = "ROLE_COLLISION"
    DETERMINISM_INCOMPATIBLE = "DETERMINISM_INCOMPATIBLE"
    TOPOLOGY_MISMATCH = "TOPOLOGY_MISMATCH"
    SPLIT_KV_RUNTIME_MISSING = "SPLIT_KV_RUNTIME_MISSING"
    SPLIT_KV_MISMATCH = "SPLIT_KV_MISMATCH"
    SPLIT_KV_FALLBACK = "SPLIT_KV_FALLBACK"
    ATTENTION_PREPROCESS_MISSING = "ATTENTION_PREPROCESS_MISSING"
    ATTENTION_PREPROCESS_MISMATCH = "ATTENTION_PREPROCESS_MISMATCH"
    ATTENTION_PREPROCESS_FALLBACK = "ATTENTION_PREPROCESS_FALLBACK"
    ATTENTION_PROJECTION_MISSING = "ATTENTION_PROJECTION_MISSING"
    ATTENTION_PROJECTION_MISMATCH = "ATTENTION_PROJECTION_MISMATCH"
    ATTENTION_CORE_MISSING = "ATTENTION_CORE_MISSING"
    ATTENTION_CORE_MISMATCH = "ATTENTION_CORE_MISMATCH"
    ATTENTION_CORE_SCHEDULE = "ATTENTION_CORE_SCHEDULE"
    ATTENTION_NATIVE_ARITHMETIC = "ATTENTION_NATIVE_ARITHMETIC"
    ATTENTION_CORE_SPLIT_K = "ATTENTION_CORE_SPLIT_K"
    ATTENTION_BACKEND_MISSING = "ATTENTION_BACKEND_MISSING"
    ATTENTION_NOT_PRODUCTION_READY = "ATTENTION_NOT_PRODUCTION_READY"


class BindingTier(str, Enum):
    """IDENTITY: the two sides do not describe the same computation.  SEMANTIC: they do, but with arithmetic that
    cannot agree bit for bit.  ADVISORY: recorded, not blocking."""
    IDENTITY = "identity"
    SEMANTIC = "semantic"
    ADVISORY = "advisory"
    IDENTICAL = "identity"        # the reference's names for the first and the last tier
    RECORDED = "advisory"


@dataclass(frozen=True)
class BindingIssue:
    code: BindingErrorCode
    tier: BindingTier
    field: str
    message: str
    rollout: Any = None
    training: Any = None

    def to_dict(self) -> dict:
        return {"code": self.code.value, "tier": self.tier.value, "field": self.field, "message": self.message,
                "rollout": self.rollout, "training": self.training}

    @property
    def blocking(self) -> bool:
        return self.tier is not BindingTier.ADVISORY


# ------------------------------------------------------------------------------------------------ pair binding
class AttentionBindingError(ValueError):
    """The caller handed over inputs that cannot be bound at all (wrong roles, wrong types)."""


ATTENTION_LSE_DOMAIN = "attention"      # never the vocabulary log-sum-exp of the log-prob contract

# Both engines must state these and agree on them exactly; a difference makes any drift number meaningless.
IDENTITY_FIELDS: tuple[str, ...] = (
    "checkpoint_id", "model_version", "weight_version", "tokenizer_fingerprint", "token_ids_fingerprint",
    "active_mask_fingerprint", "position_ids_fingerprint", "padding_side", "pre_update_state",
    "q_heads", "kv_heads", "head_dim", "rope_theta", "rope_scaling", "rotary_dim", "qk_layernorm",     # what attention means
    "batch_size",                                                                                     # which rows share a launch
    "global_token_positions_fingerprint", "kv_seq_lens_fingerprint")                                   # decode replay
# ... except these, which a side may leave unset when it has nothing to declare (no scaling, no cache)
NULLABLE_IDENTITY_FIELDS: frozenset[str] = frozenset({"rope_scaling", "global_token_positions_fingerprint", "kv_seq_lens_fingerprint"})

SEMANTIC_REDUCTION_FIELDS: tuple[str, ...] = ("merge", "acc_dtype", "order", "downcast_at")
SEMANTIC_CONTRACT_FIELDS: tuple[str, ...] = ("dtype",)
TOPOLOGY_FIELDS: tuple[str, ...] = (
    "tp_rank", "tp_world_size", "cp_rank", "cp_world_size", "global_q_heads", "global_kv_heads", "local_q_head_start", "local_q_heads",
    "local_kv_head_start", "local_kv_heads", "global_sequence_length", "local_sequence_length", "global_block_indices",
    "global_block_token_starts", "local_block_offsets", "packed_sequence_offsets")
# The numerical claim: one online-softmax state per row, fp32, keys consumed in ascending global block order, one
# rounding at the final write.  Written out even where an enum has one member, so that widening it fails here.
WS2_ATTENTION_REDUCTION_MANDATE: Mapping[str, str] = MappingProxyType({
    "merge": AttentionMerge.ONLINE_SOFTMAX_LSE.value, "acc_dtype": AttentionDType.FP32.value,
    "order": ReductionOrder.GLOBAL_BLOCK_INDEX.value, "downcast_at": DowncastPoint.FINAL_WRITE.value})
RECORDED_FIELDS: tuple[str, ...] = (
    "mode", "backend_id", "reduction.engine", "reduction.kv_block", "rope.fusion_boundary", "rope.q_state", "rope.k_state",
    "rope.k_cache_state", "rope.cast_at", "rope.output_dtype", "preprocess.qk_rmsnorm", "preprocess.rope", "preprocess.fallback",
    "kv_cache.page_size", "kv_cache.prefix_cache_enabled", "kv_cache.block_table_shape")


@dataclass(frozen=True)
class AttentionBindingResult:
    """``comparable``: the identity tier holds, a drift number from this pair means something.  ``passed``: comparable
    and no semantic finding -- only then may the pair be reported as aligned."""
    comparable: bool
    passed: bool
    issues: tuple[BindingIssue, ...] = ()
    identity_fingerprint: str = ""
    reduction_fingerprint: str = ""
    binding_fingerprint: str = ""
    recorded_differences: Mapping[str, Mapping[str, Any]] = field(default_factory=dict)
    provenance: Mapping[str, Any] = field(default_factory=dict)
    schema_version: str = "cross_config.attention_binding.v3"

    def issues_by_code(self, code: BindingErrorCode) -> tuple[BindingIssue, ...]:
        return tuple(i for i in self.issues if i.code is code)

    def issues_by_tier(self, tier: BindingTier) -> tuple[BindingIssue, ...]:
        return tuple(i for i in self.issues if i.tier is tier)

    def to_dict(self) -> dict[str, Any]:
        return {"schema_version": self.schema_version, "comparable": self.comparable, "passed": self.passed,
                "issues": [i.to_dict() for i in self.issues], "identity_fingerprint": self.identity_fingerprint,
                "reduction_fingerprint": self.reduction_fingerprint, "binding_fingerprint": self.binding_fingerprint,
                "recorded_differences": {k: dict(v) for k, v in self.recorded_differences.items()},
                "provenance": dict(self.provenance)}


def _fingerprint(payload: Any) -> str:
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":"), default=str).encode()).hexdigest()


def identity_fingerprint(identity: Mapping[str, Any]) -> str:
    """Digest of the identity fields only (extra keys a caller carries along do not change it)."""
    return _fingerprint({k: identity.get(k) for k in IDENTITY_FIELDS})


def _missing_identity_fields(identity: Mapping[str, Any]) -> tuple[str, ...]:
    return tuple(k for k in IDENTITY_FIELDS if k not in NULLABLE_IDENTITY_FIELDS and identity.get(k) is None)


def _val(x: Any) -> Any:
    return getattr(x, "value", x)


def _reduction_view(c: AttentionContract) -> dict[str, Any]:
    r = c.reduction
    return {"merge": _val(r.merge), "acc_dtype": _val(r.acc_dtype), "order": _val(r.order), "downcast_at": _val(r.downcast_at),
            "engine": _val(r.engine), "kv_block": r.kv_block}


def _topology_view(c: AttentionContract) -> dict[str, Any]:
    sh = c.sharding
    return {k: (list(v) if isinstance(v := getattr(sh, k), tuple) else v) for k in TOPOLOGY_FIELDS}


def _recorded_view(c: AttentionContract, extra: Mapping[str, Any] | None) -> dict[str, Any]:
    red = _reduction_view(c)
    out: dict[str, Any] = {"mode": _val(c.mode), "reduction.engine": red["engine"], "reduction.kv_block": red["kv_block"]}
    if c.rope is not None:
        out.update({f"rope.{k}": _val(getattr(c.rope, k)) for k in ("fusion_boundary", "q_state", "k_state", "k_cache_state", "cast_at",
                                                                    "output_dtype")})
    if c.kv_cache is not None:
        bt = c.kv_cache.block_table
        out.update({"kv_cache.page_size": c.kv_cache.page_size, "kv_cache.prefix_cache_enabled": c.kv_cache.prefix_cache_enabled,
                    "kv_cache.block_table_shape": [len(bt), max((len(r) for r in bt), default=0)]})
    for k, v in (extra or {}).items():
        out[str(k)] = v
    return out


def _split_kv_fallbacks(plan_set: SplitKVRuntimePlanSet) -> list[dict[str, Any]]:
    return [e.to_dict() for e in plan_set.entries
            if e.execution.fallback or e.execution.actual_mode is None or e.execution.source in ("unknown", "fallback")]


def _split_kv_plan_contract_error(c: AttentionContract, plan_set: SplitKVRuntimePlanSet) -> str | None:
    """Why ``plan_set`` cannot be the runtime evidence of ``c`` (None when it can)."""
    sh = c.sharding
    if plan_set.batch_size != c.batch_size:
        return f"split-KV plan set covers batch_size={plan_set.batch_size}, the contract {c.batch_size}"
    if plan_set.tp_world_size != sh.tp_world_size or plan_set.cp_world_size != sh.cp_world_size:
        return (f"split-KV plan set covers tp x cp = {plan_set.tp_world_size} x {plan_set.cp_world_size}, the contract "
                f"{sh.tp_world_size} x {sh.cp_world_size}")
    for e in plan_set.entries:
        if e.execution.requested_mode is not c.split_kv.mode:
            return (f"plan at {e.coordinate.to_dict()} was requested as {e.execution.requested_mode.value!r}, the contract asks for "
                    f"{c.split_kv.mode.value!r}")
        if c.split_kv.fixed_split_size is not None and e.execution.requested_split_size != c.split_kv.fixed_split_size:
            return (f"plan at {e.coordinate.to_dict()} requested split size {e.execution.requested_split_size}, the contract "
                    f"{c.split_kv.fixed_split_size}")
    return None


def _issue(code, tier, fld, message, rollout=None, training=None) -> BindingIssue:
    return BindingIssue(code, tier, fld, message, rollout, training)


def bind_contract_pair(*, rollout_contract: AttentionContract, training_contract: AttentionContract,
                       rollout_identity: Mapping[str, Any], training_identity: Mapping[str, Any], rollout_backend_id: str,
                       training_backend_id: str, determinism_issues: Sequence[BindingIssue] = (), require_full_identity: bool = True,
                       allow_dtype_difference: bool = False, rollout_split_kv_plan_set: SplitKVRuntimePlanSet | None = None,
                       training_split_kv_plan_set: SplitKVRuntimePlanSet | None = None,
                       rollout_recorded_extra: Mapping[str, Any] | None = None,
                       training_recorded_extra: Mapping[str, Any] | None = None) -> AttentionBindingResult:
    """Bind the rollout engine's attention contract to the training engine's.

    ``determinism_issues`` come from the probes of the two frameworks (``validation.cross_config.determinism``); they
    are threaded through so that this module needs neither framework.  ``require_full_identity=False`` is for a
    single-process harness that has no cache or decode identity to declare.  ``allow_dtype_difference=True`` is for a
    deliberate precision sweep (bf16 against an fp32 reference) and nothing else.  A configured split-KV policy is not
    evidence: both sides must hand over the plans their ranks actually executed.  The ``*_recorded_extra`` mappings are
    diagnostic only and can never make a semantic finding admissible."""
    if rollout_contract.role is not AttentionRole.INFER:
        raise AttentionBindingError(f"rollout_contract.role must be {AttentionRole.INFER.value!r}, got {rollout_contract.role.value!r}")
    if training_contract.role is not AttentionRole.TRAIN:
        raise AttentionBindingError(f"training_contract.role must be {AttentionRole.TRAIN.value!r}, got {training_contract.role.value!r}")
    issues: list[BindingIssue] = []
    T, C = BindingTier, BindingErrorCode

    # ---- identity
    if require_full_identity:
        for side, ident in (("rollout", rollout_identity), ("training", training_identity)):
            issues += [_issue(C.IDENTITY_MISSING, T.IDENTITY, f"{side}.{k}", f"{side} identity does not declare {k!r}")
                       for k in _missing_identity_fields(ident)]
    for k in IDENTITY_FIELDS:
        a, b = rollout_identity.get(k), training_identity.get(k)
        if a != b:
            issues.append(_issue(C.IDENTITY_MISMATCH, T.IDENTITY, k, f"{k!r} differs between the sides: the pair is not comparable", a, b))
    rt, tt = _topology_view(rollout_contract), _topology_view(training_contract)
    for k in TOPOLOGY_FIELDS:
        if rt[k] != tt[k]:
            issues.append(_issue(C.TOPOLOGY_MISMATCH, T.IDENTITY, f"sharding.{k}",
                                 f"sharding.{k} changes which heads / tokens a rank owns: not the same local problem", rt[k], tt[k]))
    for k, a, b in (("head_dim", rollout_contract.head_dim, training_contract.head_dim), ("causal", rollout_contract.causal, training_contract.causal)):
        if a != b:
            issues.append(_issue(C.IDENTITY_MISMATCH, T.IDENTITY, f"contract.{k}", f"contract.{k} differs between the sides", a, b))
    comparable = not any(i.tier is T.IDENTITY for i in issues)

    # ---- semantics
    rr, tr = _reduction_view(rollout_contract), _reduction_view(training_contract)
    for k in SEMANTIC_REDUCTION_FIELDS:
        if rr[k] != tr[k]:
            issues.append(_issue(C.REDUCTION_SEMANTIC_MISMATCH, T.SEMANTIC, f"reduction.{k}",
                                 f"reduction.{k} is decided by the contract, not by a backend; the sides disagree", rr[k], tr[k]))
        for side, view in (("rollout", rr), ("training", tr)):
            if view[k] != WS2_ATTENTION_REDUCTION_MANDATE[k]:
                issues.append(_issue(C.REDUCTION_MANDATE_VIOLATION, T.SEMANTIC, f"{side}.reduction.{k}",
                                     f"reduction.{k} must be {WS2_ATTENTION_REDUCTION_MANDATE[k]!r}; {side} declares {view[k]!r}", rr[k], tr[k]))
    if not allow_dtype_difference and rollout_contract.dtype is not training_contract.dtype:
        issues.append(_issue(C.REDUCTION_SEMANTIC_MISMATCH, T.SEMANTIC, "dtype",
                             "the sides compute in different dtypes; the drift would not be attributable "
                             "(allow_dtype_difference=True only for a deliberate precision sweep)",
                             rollout_contract.dtype.value, training_contract.dtype.value))
    if rollout_contract.split_kv != training_contract.split_kv:
        issues.append(_issue(C.SPLIT_KV_MISMATCH, T.SEMANTIC, "split_kv", "the sides must request the same split-KV policy",
                             rollout_contract.split_kv.to_dict(), training_contract.split_kv.to_dict()))
    for side, contract, ps in (("rollout", rollout_contract, rollout_split_kv_plan_set), ("training", training_contract, training_split_kv_plan_set)):
        fld = f"{side}.split_kv_runtime_plan_set"
        if ps is None:
            issues.append(_issue(C.SPLIT_KV_RUNTIME_MISSING, T.SEMANTIC, fld,
                                 f"{side} did not report the split-KV plans its ranks executed; a configured policy is not evidence"))
            continue
        shown = {"rollout": ps.to_dict() if side == "rollout" else None, "training": ps.to_dict() if side == "training" else None}
        err = _split_kv_plan_contract_error(contract, ps)
        if err is not None:
            issues.append(_issue(C.SPLIT_KV_MISMATCH, T.SEMANTIC, fld, err, **shown))
        fb = _split_kv_fallbacks(ps)
        if fb:
            issues.append(_issue(C.SPLIT_KV_FALLBACK, T.SEMANTIC, fld, f"{side} split-KV runtime used an unknown or fallback plan",
                                 fb if side == "rollout" else None, fb if side == "training" else None))
    if rollout_split_kv_plan_set is not None and training_split_kv_plan_set is not None:
        try:
            validate_split_kv_plan_set_alignment(training_split_kv_plan_set, rollout_split_kv_plan_set)
        except AttentionContractError as exc:
            issues.append(_issue(C.SPLIT_KV_MISMATCH, T.SEMANTIC, "split_kv_runtime_plan_set", str(exc),
                                 rollout_split_kv_plan_set.to_dict(), training_split_kv_plan_set.to_dict()))
    for side, contract in (("rollout", rollout_contract), ("training", training_contract)):
        if not contract.export_lse:
            issues.append(_issue(C.LSE_NOT_EXPORTED, T.SEMANTIC, f"{side}.export_lse",
                                 "the attention log-sum-exp must be exported: the context-parallel merge cannot be validated without it"))
    issues.extend(determinism_issues)

    # ---- recorded
    rrec, trec = _recorded_view(rollout_contract, rollout_recorded_extra), _recorded_view(training_contract, training_recorded_extra)
    rrec["backend_id"], trec["backend_id"] = rollout_backend_id, training_backend_id
    recorded = {k: {"rollout": rrec.get(k), "training": trec.get(k)} for k in RECORDED_FIELDS if rrec.get(k) != trec.get(k)}
    if rollout_backend_id and rollout_backend_id == training_backend_id:
        recorded.setdefault("backend_id", {"rollout": rollout_backend_id, "training": training_backend_id,
                                           "note": "same backend on both sides: this is not a cross-implementation comparison"})
    ident_fp = identity_fingerprint(training_identity if comparable else rollout_identity)
    red_fp = _fingerprint({k: tr[k] for k in SEMANTIC_REDUCTION_FIELDS})
    split = {"rollout": None if rollout_split_kv_plan_set is None else rollout_split_kv_plan_set.to_dict(),
             "training": None if training_split_kv_plan_set is None else training_split_kv_plan_set.to_dict()}
    provenance = {"lse_domain": ATTENTION_LSE_DOMAIN, "dtype": training_contract.dtype.value, "split_kv_runtime": split,
                  "rollout": {"contract": rollout_contract.to_dict(), "backend_id": rollout_backend_id, "recorded": rrec},
                  "training": {"contract": training_contract.to_dict(), "backend_id": training_backend_id, "recorded": trec}}
    pre = {side: {k: rec.get(f"preprocess.{k}") for k in (*MANDATED_ATTENTION_PREPROCESS_BACKENDS, "fallback")}
           for side, rec in (("rollout", rrec), ("training", trec))}
    binding_fp = _fingerprint({"identity": ident_fp, "reduction": red_fp, "topology": tt, "split_kv": split, "lse_domain": ATTENTION_LSE_DOMAIN,
                               "rollout_backend": rollout_backend_id, "training_backend": training_backend_id, "attention_preprocess": pre})
    passed = comparable and not any(i.tier is T.SEMANTIC for i in issues)
    return AttentionBindingResult(comparable, passed, tuple(issues), ident_fp, red_fp, binding_fp, recorded, provenance)


# ------------------------------------------------------------------------------------------------ runtime readbacks
@dataclass(frozen=True)
class AttentionRuntimeReadback:
    """What one engine actually executed: its contract rebuilt from the live layer, the knobs it read back, the
    split-KV plans of all its ranks, and which kernels ran at the input boundary, in the projections and in the core."""
    contract: AttentionContract
    actual_knobs: Mapping[str, Any]
    split_kv_plan_set: SplitKVRuntimePlanSet
    source: str
    frozen_scope_verified: bool
    preprocess_backends: Mapping[str, str] = field(default_factory=dict)
    preprocess_fallback: bool = False
    preprocess_fallback_reason: str | None = None
    preprocess_probe_id: str = ""
    preprocess_policy_id: str = PREPROCESS_POLICY_ID
    projection_plans: Mapping[str, Mapping[str, Any]] = field(default_factory=dict)
    strict_mode: bool = False
    strict_core_id: str | None = None
    strict_schedule: str | None = None
    native_attention_arithmetic: bool = True
    strict_split_kv_policy: str | None = None
    actual_backend: str | None = None
    communication_backend: str | None = None
    production_ready: bool = False
    attention_fallback: bool = False
    reference_only: bool = False

    def __post_init__(self) -> None:
        def need(cond: bool, kind, msg: str) -> None:
            if not cond:
                raise kind(msg)

        need(isinstance(self.contract, AttentionContract), TypeError, "runtime readback contract must be an AttentionContract")
        need(isinstance(self.actual_knobs, Mapping), TypeError, "runtime readback actual_knobs must be a mapping")
        need(isinstance(self.split_kv_plan_set, SplitKVRuntimePlanSet), TypeError, "runtime readback requires a complete SplitKVRuntimePlanSet")
        need(isinstance(self.source, str) and bool(self.source.strip()), ValueError, "runtime readback source must be a non-empty string")
        for name in ("frozen_scope_verified", "preprocess_fallback", "strict_mode", "native_attention_arithmetic", "production_ready",
                     "attention_fallback", "reference_only"):
            need(isinstance(getattr(self, name), bool), TypeError, f"{name} must be a bool")
        need(isinstance(self.preprocess_backends, Mapping), TypeError, "runtime readback preprocess_backends must be a mapping")
        for k, v in self.preprocess_backends.items():
            need(isinstance(k, str) and bool(k.strip()) and isinstance(v, str) and bool(v.strip()), ValueError,
                 "preprocess backend names and ids must be non-empty strings")
        need(not self.preprocess_fallback or bool(self.preprocess_fallback_reason), ValueError,
             "preprocess_fallback_reason is required when preprocess_fallback is true")
        need(isinstance(self.preprocess_probe_id, str), TypeError, "preprocess_probe_id must be a string")
        need(isinstance(self.preprocess_policy_id, str) and bool(self.preprocess_policy_id.strip()), ValueError,
             "preprocess_policy_id must be a non-empty string")
        need(isinstance(self.projection_plans, Mapping), TypeError, "projection_plans must be a mapping")
        for name in ("strict_core_id", "strict_schedule", "actual_backend", "communication_backend"):
            v = getattr(self, name)
            need(v is None or (isinstance(v, str) and bool(v.strip())), ValueError, f"{name} must be a non-empty string when provided")
        need(self.strict_split_kv_policy in (None, "disabled", "fixed", "auto"), ValueError,
             "strict_split_kv_policy must be disabled, fixed, or auto")
        plans = {}
        for k, v in self.projection_plans.items():
            need(isinstance(k, str) and isinstance(v, Mapping), TypeError, "projection_plans must map projection names to mappings")
            plans[k] = MappingProxyType(dict(v))
        err = _split_kv_plan_contract_error(self.contract, self.split_kv_plan_set)
        need(err is None, ValueError, err or "")
        object.__setattr__(self, "actual_knobs", MappingProxyType(dict(self.actual_knobs)))
        object.__setattr__(self, "preprocess_backends", MappingProxyType(dict(self.preprocess_backends)))
        object.__setattr__(self, "projection_plans", MappingProxyType(plans))

    @property
    def split_kv_fallback(self) -> bool:
        return bool(_split_kv_fallbacks(self.split_kv_plan_set))

    def to_dict(self) -> dict[str, Any]:
        return {"source": self.source, "frozen_scope_verified": self.frozen_scope_verified, "actual_knobs": dict(self.actual_knobs),
                "contract": self.contract.to_dict(),
                "attention_preprocess": {"backends": dict(self.preprocess_backends), "fallback": self.preprocess_fallback,
                                         "fallback_reason": self.preprocess_fallback_reason, "probe_id": self.preprocess_probe_id,
                                         "policy_id": self.preprocess_policy_id},
                "attention_projections": {k: dict(v) for k, v in self.projection_plans.items()},
                "strict_attention": {"enabled": self.strict_mode, "core_id": self.strict_core_id, "schedule": self.strict_schedule,
                                     "native_attention_arithmetic": self.native_attention_arithmetic,
                                     "split_kv_policy": self.strict_split_kv_policy},
                "runtime_backend": {"actual_backend": self.actual_backend, "communication_backend": self.communication_backend,
                                    "production_ready": self.production_ready, "fallback": self.attention_fallback,
                                    "reference_only": self.reference_only},
                "split_kv_runtime_plan_set": self.split_kv_plan_set.to_dict()}


SUPPORTED_CP_COMMUNICATION = frozenset({"symmetric_memory_peer_loads", "torch_distributed_all_gather"})
ALLOWED_PROJECTION_BACKENDS = frozenset({DETERMINISTIC_PROJECTION_BACKEND_ID, REFERENCE_PROJECTION_BACKEND_ID})


def _side(side: str, value: Any) -> dict[str, Any]:
    return {"rollout": value if side == "rollout" else None, "training": value if side == "training" else None}


def _preprocess_issues(side: str, rb: AttentionRuntimeReadback) -> list[BindingIssue]:
    T, C, out = BindingTier, BindingErrorCode, []
    for name, mandated in MANDATED_ATTENTION_PREPROCESS_BACKENDS.items():
        actual = rb.preprocess_backends.get(name)
        if actual is None:
            out.append(_issue(C.ATTENTION_PREPROCESS_MISSING, T.SEMANTIC, f"{side}.preprocess.{name}",
                              f"{side} did not report which {name} kernel ran: the input boundary of attention is unverified"))
        elif actual not in ALLOWED_ATTENTION_PREPROCESS_BACKENDS[name]:
            out.append(_issue(C.ATTENTION_PREPROCESS_MISMATCH, T.SEMANTIC, f"{side}.preprocess.{name}",
                              f"{side} executed {actual!r}; the pair requires {mandated!r} or the reference of the same expression",
                              **_side(side, actual)))
    if rb.preprocess_fallback:
        out.append(_issue(C.ATTENTION_PREPROCESS_FALLBACK, T.SEMANTIC, f"{side}.preprocess.fallback",
                          f"{side} fell back at the input boundary: {rb.preprocess_fallback_reason}", **_side(side, True)))
    return out


def _projection_issues(side: str, rb: AttentionRuntimeReadback) -> list[BindingIssue]:
    T, C, out = BindingTier, BindingErrorCode, []
    for name in ("qkv", "o_proj"):
        plan = rb.projection_plans.get(name)
        fld = f"{side}.projection.{name}"
        if plan is None:
            out.append(_issue(C.ATTENTION_PROJECTION_MISSING, T.SEMANTIC, fld, f"{side} did not report the executed {name} projection plan"))
            continue
        if plan.get("backend") not in ALLOWED_PROJECTION_BACKENDS:
            out.append(_issue(C.ATTENTION_PROJECTION_MISMATCH, T.SEMANTIC, f"{fld}.backend",
                              f"{side} ran {plan.get('backend')!r}; the projections must be the deterministic GEMM of this package",
                              **_side(side, plan.get("backend"))))
        if plan.get("policy_id") != PROJECTION_POLICY_ID:
            out.append(_issue(C.ATTENTION_PROJECTION_MISMATCH, T.SEMANTIC, f"{fld}.policy_id", "projection policy differs from this package's",
                              **_side(side, plan.get("policy_id"))))
        if plan.get("split_k"):
            out.append(_issue(C.ATTENTION_CORE_SPLIT_K, T.SEMANTIC, f"{fld}.split_k", "split-K changes the order of the K sum", **_side(side, True)))
        if plan.get("fallback"):
            out.append(_issue(C.ATTENTION_PROJECTION_MISMATCH, T.SEMANTIC, f"{fld}.fallback", f"{side} {name} projection fell back",
                              **_side(side, True)))
    return out


def _core_issues(side: str, rb: AttentionRuntimeReadback) -> list[BindingIssue]:
    if not rb.strict_mode:
        return []
    T, C, out = BindingTier, BindingErrorCode, []
    if not rb.actual_backend:
        out.append(_issue(C.ATTENTION_BACKEND_MISSING, T.SEMANTIC, f"{side}.runtime.actual_backend",
                          f"{side} strict attention did not report the core it executed"))
    if rb.contract.sharding.cp_world_size > 1 and rb.communication_backend not in SUPPORTED_CP_COMMUNICATION:
        out.append(_issue(C.ATTENTION_BACKEND_MISSING, T.SEMANTIC, f"{side}.runtime.communication_backend",
                          f"{side} context-parallel attention did not run one of {sorted(SUPPORTED_CP_COMMUNICATION)}",
                          **_side(side, rb.communication_backend)))
    if not rb.production_ready or rb.reference_only or rb.attention_fallback:
        out.append(_issue(C.ATTENTION_NOT_PRODUCTION_READY, T.SEMANTIC, f"{side}.runtime.production_ready",
                          f"{side} strict attention ran a reference-only or fallback core",
                          **_side(side, {"production_ready": rb.production_ready, "reference_only": rb.reference_only,
                                         "fallback": rb.attention_fallback})))
    if not rb.strict_core_id:
        out.append(_issue(C.ATTENTION_CORE_MISSING, T.SEMANTIC, f"{side}.strict_attention.core_id", f"{side} did not name its strict core"))
    if not rb.strict_schedule:
        out.append(_issue(C.ATTENTION_CORE_SCHEDULE, T.SEMANTIC, f"{side}.strict_attention.schedule",
                          f"{side} did not report the key-block schedule of its strict core"))
    if rb.native_attention_arithmetic:
        out.append(_issue(C.ATTENTION_NATIVE_ARITHMETIC, T.SEMANTIC, f"{side}.strict_attention.native_attention_arithmetic",
                          f"{side} left the framework's own attention arithmetic in place under strict mode", **_side(side, True)))
    if rb.strict_split_kv_policy == "auto":
        out.append(_issue(C.ATTENTION_CORE_SPLIT_K, T.SEMANTIC, f"{side}.strict_attention.split_kv_policy",
                          "an automatically chosen split-KV schedule depends on the batch", **_side(side, "auto")))
    return out


def bind_attention_runtime_readbacks(*, rollout: AttentionRuntimeReadback, training: AttentionRuntimeReadback,
                                     rollout_identity: Mapping[str, Any], training_identity: Mapping[str, Any], rollout_backend_id: str,
                                     training_backend_id: str, determinism_issues: Sequence[BindingIssue] = ()) -> AttentionBindingResult:
    """The strict hand-over from two executed runtimes: nothing configured-only is accepted.  Findings about the frozen
    scope, the input boundary, the projections and the core of each side, and about the pair, are added to the contract
    binding as semantic issues."""
    T, C = BindingTier, BindingErrorCode
    found: list[BindingIssue] = []
    for side, rb in (("rollout", rollout), ("training", training)):
        if not rb.frozen_scope_verified:
            found.append(_issue(C.DETERMINISM_INCOMPATIBLE, T.SEMANTIC, f"{side}.frozen_scope_verified",
                                f"{side} runtime did not verify the frozen attention scope"))
        found += _preprocess_issues(side, rb) + _projection_issues(side, rb) + _core_issues(side, rb)
    if rollout.preprocess_fallback != training.preprocess_fallback:
        found.append(_issue(C.ATTENTION_PREPROCESS_MISMATCH, T.SEMANTIC, "preprocess.fallback",
                            "both runtimes must run the same input-boundary path", rollout.preprocess_fallback, training.preprocess_fallback))
    if rollout.preprocess_policy_id != training.preprocess_policy_id:
        found.append(_issue(C.ATTENTION_PREPROCESS_MISMATCH, T.SEMANTIC, "preprocess.policy_id", "QK-norm / RoPE policy ids differ",
                            rollout.preprocess_policy_id, training.preprocess_policy_id))
    if rollout.preprocess_probe_id and training.preprocess_probe_id and rollout.preprocess_probe_id != training.preprocess_probe_id:
        found.append(_issue(C.ATTENTION_PREPROCESS_MISMATCH, T.SEMANTIC, "preprocess.probe_id",
                            "the two runtimes built their RoPE tables / norm constants from different parameters",
                            rollout.preprocess_probe_id, training.preprocess_probe_id))
    for name in ("qkv", "o_proj"):
        a, b = rollout.projection_plans.get(name, {}), training.projection_plans.get(name, {})
        for key in ("fallback", "canonical_k_chunks", "k_order", "acc_dtype"):
            if a.get(key) != b.get(key) and a and b:
                found.append(_issue(C.ATTENTION_PROJECTION_MISMATCH, T.SEMANTIC, f"projection.{name}.{key}",
                                    f"the {name} projections of the two runtimes differ in {key}", a.get(key), b.get(key)))
    if rollout.strict_mode != training.strict_mode:
        found.append(_issue(C.ATTENTION_CORE_MISMATCH, T.SEMANTIC, "strict_attention.enabled", "strict attention is on for one side only",
                            rollout.strict_mode, training.strict_mode))
    elif rollout.strict_mode:
        for key, code in (("strict_core_id", C.ATTENTION_CORE_MISMATCH), ("strict_schedule", C.ATTENTION_CORE_SCHEDULE),
                          ("strict_split_kv_policy", C.ATTENTION_CORE_SPLIT_K)):
            a, b = getattr(rollout, key), getattr(training, key)
            if a != b:
                found.append(_issue(code, T.SEMANTIC, f"strict_attention.{key.removeprefix('strict_')}",
                                    f"the strict cores of the two runtimes differ in {key}", a, b))
    extra = {side: {"preprocess.qk_rmsnorm": rb.preprocess_backends.get("qk_rmsnorm"), "preprocess.rope": rb.preprocess_backends.get("rope"),
                    "preprocess.fallback": rb.preprocess_fallback} for side, rb in (("rollout", rollout), ("training", training))}
    res = bind_contract_pair(rollout_contract=rollout.contract, training_contract=training.contract, rollout_identity=rollout_identity,
                             training_identity=training_identity, rollout_backend_id=rollout_backend_id,
                             training_backend_id=training_backend_id, determinism_issues=(*found, *determinism_issues),
                             rollout_split_kv_plan_set=rollout.split_kv_plan_set, training_split_kv_plan_set=training.split_kv_plan_set,
                             rollout_recorded_extra=extra["rollout"], training_recorded_extra=extra["training"])
    prov = dict(res.provenance)
    prov["runtime_readbacks"] = {"rollout": rollout.to_dict(), "training": training.to_dict()}
    return AttentionBindingResult(res.comparable, res.passed, res.issues, res.identity_fingerprint, res.reduction_fingerprint,
                                  _fingerprint({"binding": res.binding_fingerprint, "readbacks": prov["runtime_readbacks"]}),
                                  res.recorded_differences, prov)


def summarize_binding(result: AttentionBindingResult) -> str:
    """One line for a CLI or an exception message."""
    if result.passed:
        return (f"attention binding OK (identity={result.identity_fingerprint[:12]}, "
                f"{len(result.recorded_differences)} recorded difference(s))")
    tier = BindingTier.SEMANTIC if result.comparable else BindingTier.IDENTITY
    fields = ", ".join(sorted({i.field for i in result.issues if i.tier is tier}))
    return (f"attention binding FAILED CLOSED; semantic problems: {fields}" if result.comparable
            else f"attention binding NOT COMPARABLE; identity problems: {fields}")


def first_blocking_issue(result: AttentionBindingResult) -> BindingIssue | None:
    """The issue to report: identity findings come before semantic ones."""
    for tier in (BindingTier.IDENTITY, BindingTier.SEMANTIC):
        for i in result.issues:
            if i.tier is tier:
                return i
    return None


__all__ = ["ATTENTION_LSE_DOMAIN", "AttentionBindingError", "AttentionBindingResult", "AttentionRuntimeReadback", "BindingErrorCode",
           "BindingIssue", "BindingTier", "IDENTITY_FIELDS", "NULLABLE_IDENTITY_FIELDS", "RECORDED_FIELDS", "SEMANTIC_CONTRACT_FIELDS",
           "SEMANTIC_REDUCTION_FIELDS", "TOPOLOGY_FIELDS", "WS2_ATTENTION_REDUCTION_MANDATE", "bind_attention_contracts",
           "bind_attention_runtime_readbacks", "bind_contract_pair", "contract_from_layer", "first_blocking_issue", "identity_fingerprint",
           "summarize_binding"]
