"""Cross-side determinism probing (parity: rl_engine/validation/cross_config/determinism.py:78-305).

A rollout engine and a trainer each have a "deterministic" switch that covers different things:
vLLM's ``VLLM_BATCH_INVARIANT`` replaces matmul / softmax / norm kernels and pins TF32, reduced-
precision reductions and ten NCCL variables; Megatron's ``deterministic_mode`` pins the NCCL
algorithm family and forbids FlashAttention and fused cross entropy, and manages neither TF32 nor
the reduction precision.  This framework's own engine is deterministic by construction (fixed
reduction orders in every kernel, its own collectives) and reports that as a probe as well.  The
comparison makes the differences explicit: a side with the switch off, or a difference in a variable
that changes arithmetic, is blocking; the rest is recorded.  Probes are built from plain mappings --
no framework is imported.
"""
from __future__ import annotations

import hashlib
import json
from collections.abc import Mapping
from dataclasses import dataclass, field
from typing import Any, Optional

from rl_kernel_b200.integrations.common.attention_binding import BindingErrorCode, BindingIssue, BindingTier

COMPARED_NCCL_KEYS: tuple[str, ...] = ("NCCL_ALGO", "NCCL_PROTO", "NCCL_MIN_NCHANNELS", "NCCL_MAX_NCHANNELS", "NCCL_NTHREADS",
                                       "NCCL_SOCKET_NTHREADS", "NCCL_COLLNET_ENABLE", "NCCL_NVLS_ENABLE", "NCCL_P2P_NET_DISABLE",
                                       "NCCL_LAUNCH_MODE", "CUBLAS_WORKSPACE_CONFIG")
_ARITHMETIC_KEYS = frozenset({"NCCL_ALGO", "NCCL_PROTO", "CUBLAS_WORKSPACE_CONFIG"})


@dataclass(frozen=True)
class DeterminismProbe:
    """What one side has switched on.  The tri-state fields use None for "the framework does not manage this"."""
    side: str
    framework: str
    mode_flag: str
    enabled: bool
    env: Mapping[str, Any] = field(default_factory=dict)
    tf32_disabled: Optional[bool] = None
    bf16_reduced_precision_reduction: Optional[bool] = None
    forbids_flash_attention: Optional[bool] = None
    own_collectives: bool = False          # reductions across ranks run in the framework's own fixed-order kernels, not NCCL
    evidence: Mapping[str, Any] = field(default_factory=dict)
    schema_version: str = "cross_config.determinism_probe.v1"

    def __post_init__(self) -> None:
        if self.side not in ("rollout", "training"):
            raise ValueError("side must be 'rollout' or 'training'")
        if not self.framework:
            raise ValueError("framework must not be empty")
        object.__setattr__(self, "env", dict(self.env))
        object.__setattr__(self, "evidence", dict(self.evidence))

    @property
    def env_fingerprint(self) -> str:
        payload = {k: self.env.get(k) for k in COMPARED_NCCL_KEYS}
        return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":"), default=str).encode()).hexdigest()

    def to_dict(self) -> dict[str, Any]:
        return {"schema_version": self.schema_version, "side": self.side, "framework": self.framework, "mode_flag": self.mode_flag,
                "enabled": self.enabled, "env": {k: self.env.get(k) for k in COMPARED_NCCL_KEYS},
                "env_fingerprint": self.env_fingerprint, "tf32_disabled": self.tf32_disabled,
                "bf16_reduced_precision_reduction": self.bf16_reduced_precision_reduction,
                "forbids_flash_attention": self.forbids_flash_attention, "own_collectives": self.own_collectives,
                "evidence": dict(self.evidence)}


@dataclass(frozen=True)
class DeterminismReport:
    rollout: DeterminismProbe
    training: DeterminismProbe
    issues: tuple[BindingIssue, ...] = ()
    differences: Mapping[str, Mapping[str, Any]] = field(default_factory=dict)
    schema_version: str = "cross_config.determinism_report.v1"

    @property
    def compatible(self) -> bool:
        return not self.issues

    def to_dict(self) -> dict[str, Any]:
        return {"schema_version": self.schema_version, "compatible": self.compatible, "rollout": self.rollout.to_dict(),
                "training": self.training.to_dict(), "issues": [i.to_dict() for i in self.issues],
                "differences": {k: dict(v) for k, v in self.differences.items()}}


def _value(v: Any) -> Any:
    return getattr(v, "value", v)


def _get(config: Any, name: str, default: Any = None) -> Any:
    """Attribute of a config object or key of a mapping."""
    if isinstance(config, Mapping):
        return config.get(name, default)
    return getattr(config, name, default)


def megatron_probe_from_config(config: Any, env: Optional[Mapping[str, str]] = None) -> DeterminismProbe:
    """Training-side probe from anything exposing ``deterministic_mode`` (a ModelParallelConfig, a namespace, a double)."""
    e = dict(env or {})
    on = bool(_get(config, "deterministic_mode", False))
    return DeterminismProbe("training", "megatron", "deterministic_mode", on, {k: e.get(k) for k in COMPARED_NCCL_KEYS}, None, None, on,
                            False, {"nvte_allow_nondeterministic_algo": e.get("NVTE_ALLOW_NONDETERMINISTIC_ALGO"),
                                    "cross_entropy_loss_fusion": _get(config, "cross_entropy_loss_fusion", None),
                                    "attention_backend": _value(_get(config, "attention_backend", None)),
                                    "tensor_model_parallel_size": _get(config, "tensor_model_parallel_size", None),
                                    "context_parallel_size": _get(config, "context_parallel_size", None),
                                    "sequence_parallel": _get(config, "sequence_parallel", None), "manages_tf32": False,
                                    "manages_bf16_reduced_precision_reduction": False})


def vllm_probe_from_env(env: Mapping[str, str], *, model_config: Any = None) -> DeterminismProbe:
    """Rollout-side probe from a (possibly remote) worker's reported environment."""
    on = str(env.get("VLLM_BATCH_INVARIANT", "0")).strip() in ("1", "true", "True")
    return DeterminismProbe("rollout", "vllm", "VLLM_BATCH_INVARIANT", on, {k: env.get(k) for k in COMPARED_NCCL_KEYS}, on or None,
                            False if on else None, False, False,
                            {"vllm_allreduce_use_symm_mem": env.get("VLLM_ALLREDUCE_USE_SYMM_MEM"),
                             "vllm_use_aot_compile": env.get("VLLM_USE_AOT_COMPILE"),
                             "enforce_eager": _get(model_config, "enforce_eager", None),
                             "disable_cascade_attn": _get(model_config, "disable_cascade_attn", None),
                             "quantization": _get(model_config, "quantization", None), "manages_tf32": True,
                             "manages_bf16_reduced_precision_reduction": True})


def engine_probe(side: str, *, env: Optional[Mapping[str, str]] = None, tp_size: int = 1, cp_size: int = 1,
                 strict: bool = True) -> DeterminismProbe:
    """Probe of this framework's own engine on either side.  Its kernels fix every reduction order and its tensor- and
    context-parallel reductions run in its own peer-memory kernels, so NCCL's algorithm choice does not enter the
    arithmetic; bf16 operands never take a TF32 path.  ``strict`` is the strict-contract policy: with it off the
    engine may dispatch to library kernels and is reported as not enabled."""
    e = dict(env or {})
    return DeterminismProbe(side, "rl_kernel_b200", "strict_contract", bool(strict), {k: e.get(k) for k in COMPARED_NCCL_KEYS}, True,
                            False, False, True, {"tensor_parallel_size": tp_size, "context_parallel_size": cp_size,
                                                 "reduction_order": "fixed in every kernel", "manages_tf32": True,
                                                 "manages_bf16_reduced_precision_reduction": True})


def compare_determinism(*, rollout: DeterminismProbe, training: DeterminismProbe) -> DeterminismReport:
    if rollout.side != "rollout" or training.side != "training":
        raise ValueError("compare_determinism expects one rollout probe and one training probe")
    issues: list[BindingIssue] = []
    diffs: dict[str, dict[str, Any]] = {}
    for p in (rollout, training):
        if not p.enabled:
            issues.append(BindingIssue(BindingErrorCode.DETERMINISM_INCOMPATIBLE, BindingTier.SEMANTIC, f"{p.side}.{p.mode_flag}",
                                       f"{p.framework} {p.mode_flag} is not enabled; the {p.side} side is not batch-invariant and "
                                       "cannot anchor a cross-configuration comparison", rollout.enabled, training.enabled))
    nccl_matters = not (rollout.own_collectives and training.own_collectives)
    for k in COMPARED_NCCL_KEYS:
        a, b = rollout.env.get(k), training.env.get(k)
        if a == b:
            continue
        diffs[k] = {"rollout": a, "training": b}
        arithmetic = k in _ARITHMETIC_KEYS and (nccl_matters or k == "CUBLAS_WORKSPACE_CONFIG")
        if arithmetic:
            issues.append(BindingIssue(BindingErrorCode.DETERMINISM_INCOMPATIBLE, BindingTier.SEMANTIC, f"env.{k}",
                                       f"{k} differs between the sides; they would reduce with different arithmetic and the "
                                       "drift could not be attributed", a, b))
    for name in ("tf32_disabled", "bf16_reduced_precision_reduction"):
        a, b = getattr(rollout, name), getattr(training, name)
        if a != b:
            diffs[name] = {"rollout": a, "training": b, "note": "None: the framework does not manage this setting"}
    if rollout.forbids_flash_attention != training.forbids_flash_attention:
        diffs["forbids_flash_attention"] = {"rollout": rollout.forbids_flash_attention, "training": training.forbids_flash_attention}
    return DeterminismReport(rollout, training, tuple(issues), diffs)


__all__ = ["COMPARED_NCCL_KEYS", "DeterminismProbe", "DeterminismReport", "compare_determinism", "engine_probe",
           "megatron_probe_from_config", "vllm_probe_from_env"]
