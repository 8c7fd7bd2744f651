"""Operator bridge: one call that resolves the selected-log-prob operator for an integration and
records the execution (parity: OperatorBridge / selected_logprobs_with_operator,
rl_engine/runtime/operators.py:105-307)."""
from __future__ import annotations

import torch

from rl_kernel_b200.runtime.registry import kernel_registry
from rl_kernel_b200.runtime.semantic_registry import OperatorSession, semantic_catalog


class OperatorBridge:
    def __init__(self, session: OperatorSession | None = None, temperature: float = 1.0):
        self.session = session or semantic_catalog.session("bridge")
        self.temperature = temperature

    def selected_logprobs(self, *, logits: torch.Tensor | None = None, hidden: torch.Tensor | None = None,
                          lm_head_weight: torch.Tensor | None = None, token_ids: torch.Tensor,
                          mask: torch.Tensor | None = None, module: str = "") -> torch.Tensor:
        if (logits is None) == (hidden is None):
            raise ValueError("give exactly one of logits / hidden")
        if hidden is not None:
            if lm_head_weight is None:
                raise ValueError("hidden input needs lm_head_weight")
            op = kernel_registry.get_op("linear_logp", temperature=self.temperature, operand_device=hidden.device)
            lp = op(hidden, lm_head_weight, token_ids)
        else:
            op = kernel_registry.get_op("batch_invariant_logp", temperature=self.temperature, operand_device=logits.device)
            lp = op(logits, token_ids)
        res = kernel_registry.last_resolution
        backend = "reference" if res.actual.name.startswith("REF") else "b200-tcgen05"
        self.session.observe("selected_logprob", backend, module, res.fallback)
        return lp if mask is None else lp.masked_fill(~mask.bool(), 0.0)


def selected_logprobs_with_operator(logits, token_ids, mask=None, temperature: float = 1.0):
    return OperatorBridge(temperature=temperature).selected_logprobs(logits=logits, token_ids=token_ids, mask=mask)


# ================================================================================================ per-target overrides
# (parity: OperatorOverride / ResolvedOperatorOverride / OperatorBridge.resolve_override, rl_engine/runtime/operators.py:29-196)
from dataclasses import dataclass as _dataclass
from typing import Any as _Any, Mapping as _Mapping, Optional as _Optional

from rl_kernel_b200.runtime.semantic_registry import (OperatorRequirements, OperatorResolution, OperatorResolutionPolicy,
                                                      SemanticOperatorCatalog)

_TARGETS = ("rollout", "training")


def _norm_backend(v):
    if v is None:
        return None
    s = str(v).strip()
    return None if s.lower() in ("", "auto", "default", "native") else s


@_dataclass(frozen=True)
class OperatorOverride:
    """Which backend serves one semantic operator on which side.  ``None`` leaves the side to automatic resolution."""
    semantic_op: str
    rollout_backend: _Optional[str] = None
    training_backend: _Optional[str] = None

    def __post_init__(self) -> None:
        if not self.semantic_op:
            raise ValueError("semantic_op must not be empty")
        object.__setattr__(self, "rollout_backend", _norm_backend(self.rollout_backend))
        object.__setattr__(self, "training_backend", _norm_backend(self.training_backend))

    @classmethod
    def for_target(cls, semantic_op: str, target: str, backend: str) -> "OperatorOverride":
        if target not in _TARGETS:
            raise ValueError("target must be rollout or training")
        return cls(semantic_op, **{f"{target}_backend": backend})

    def backend_for(self, target: str) -> _Optional[str]:
        if target not in _TARGETS:
            raise ValueError("target must be rollout or training")
        return getattr(self, f"{target}_backend")

    def to_dict(self) -> dict:
        return {"semantic_op": self.semantic_op, "rollout": self.rollout_backend, "training": self.training_backend}


@_dataclass(frozen=True)
class ResolvedOperatorOverride:
    override: OperatorOverride
    rollout: _Optional[OperatorResolution]
    training: _Optional[OperatorResolution]

    def for_target(self, target: str) -> _Optional[OperatorResolution]:
        return {"rollout": self.rollout, "training": self.training}[target]

    def to_dict(self) -> dict:
        return {"override": self.override.to_dict(), "rollout": None if self.rollout is None else self.rollout.to_dict(),
                "training": None if self.training is None else self.training.to_dict()}


def _resolve_override(self, override: OperatorOverride, *, requirements: _Mapping[str, OperatorRequirements] | None = None,
                      catalog: SemanticOperatorCatalog | None = None, policy: OperatorResolutionPolicy | None = None) -> ResolvedOperatorOverride:
    """Resolve both sides of an override against the catalog.  A side without a named backend resolves automatically;
    a named backend that cannot serve the side's requirements is an error under the strict policy."""
    cat = catalog or semantic_catalog
    out = {}
    for target in _TARGETS:
        req = (requirements or {}).get(target) or OperatorRequirements(override.semantic_op, target=target)
        out[target] = cat.resolve(req, backend=override.backend_for(target), policy=policy)
    return ResolvedOperatorOverride(override, out["rollout"], out["training"])


def _instantiate(self, resolution: OperatorResolution, **kwargs) -> _Any:
    op = semantic_catalog.instantiate(resolution, **kwargs)
    self.session.observe(resolution.semantic_op, resolution.actual_backend if (resolution.semantic_op, resolution.actual_backend)
                         in semantic_catalog._by_key else "reference", "bridge", resolution.fallback)
    return op


OperatorBridge.resolve_override = _resolve_override
OperatorBridge.instantiate = _instantiate
OperatorBridge.instance_provenance = lambda self, resolution, instance: semantic_catalog.instance_provenance(resolution, instance)
