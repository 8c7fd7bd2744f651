"""Shared implementation of the two framework-side attention materialisers."""
from __future__ import annotations

import hashlib
import json
from typing import Any, Mapping, Optional

from rl_kernel_b200.contracts.operators.attention import AttentionContract, AttentionMode, AttentionRole, CPLayout, ReductionEngine
from rl_kernel_b200.integrations.common.cross_config import (QWEN3_8B, Qwen3ModelSpec, application, build_sharding_spec,
                                                             unsupported_reduction_reason)
from rl_kernel_b200.validation.cross_config.runtime import AdapterMaterialization
from rl_kernel_b200.validation.cross_config.schema import MaterializationStatus


def value(config: Any, name: str) -> Any:
    if config is None:
        return None
    if isinstance(config, Mapping):
        return config.get(name)
    v = getattr(config, name, None)
    return getattr(v, "value", v)


def fingerprint(payload: Mapping[str, Any]) -> str:
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":"), default=str).encode()).hexdigest()


class AttentionMaterializerBase:
    """Translates a case's knobs into an ``AttentionContract`` for one side and reports, per knob, whether the runtime
    honours it.  Subclasses name the side's knob prefix, role and the values their runtime accepts."""
    target = ""
    side_prefix = ""
    role = AttentionRole.TRAIN
    runtime_kind = ""

    def __init__(self, *, model: Qwen3ModelSpec = QWEN3_8B, global_sequence_length: int = 4096, tp_rank: int = 0, cp_rank: int = 0,
                 mode: AttentionMode = AttentionMode.PREFILL, backend_id: str = "", provenance=None, runtime_readback: Optional[Mapping] = None):
        self.model, self.global_sequence_length, self.tp_rank, self.cp_rank = model, global_sequence_length, tp_rank, cp_rank
        self.mode, self.backend_id, self.provenance, self.runtime_readback = mode, backend_id, provenance, dict(runtime_readback or {})

    def implementation_fingerprint(self) -> str:
        return fingerprint({"class": f"{type(self).__module__}.{type(self).__qualname__}", "model": self.model.fingerprint_payload(),
                            "seq": self.global_sequence_length, "mode": self.mode.value, "backend": self.backend_id})

    def effective_cp_world_size(self, flat: Mapping[str, Any]) -> int:
        return 1 if self.mode is AttentionMode.DECODE else int(flat.get(f"{self.side_prefix}.context_parallel_size", 1))

    def build_contract(self, flat: Mapping[str, Any]) -> AttentionContract:
        reason = unsupported_reduction_reason(flat)
        if reason:
            raise ValueError(reason)
        tp = int(flat.get(f"{self.side_prefix}.tensor_parallel_size", 1))
        cp = self.effective_cp_world_size(flat)
        sh = build_sharding_spec(model=self.model, tp_rank=self.tp_rank, tp_world_size=tp, cp_rank=self.cp_rank if cp > 1 else 0,
                                 cp_world_size=cp, global_sequence_length=self.global_sequence_length)
        return AttentionContract.for_layout(self.model.q_heads, self.model.kv_heads, head_dim=self.model.head_dim,
                                            seq_len=self.global_sequence_length, batch_size=int(flat.get("batch.size", 1)),
                                            tp_rank=self.tp_rank, tp_world_size=tp, cp_rank=self.cp_rank if cp > 1 else 0, cp_world_size=cp,
                                            layout=sh.cp_layout if hasattr(sh, "cp_layout") else (CPLayout.NONE if cp == 1 else CPLayout.ZIGZAG),
                                            role=self.role, mode=self.mode,
                                            engine=ReductionEngine(flat.get("attention.reduction_engine", "in_kernel")))

    # per-knob acceptance: {path: callable(value) -> reason or None}
    def _checks(self) -> dict:
        return {}

    def materialize(self, case, normalized: Mapping[str, Any]) -> AdapterMaterialization:
        checks = self._checks()
        apps, options = [], {}
        reduction_reason = unsupported_reduction_reason(normalized)
        for path, v in sorted(normalized.items()):
            if path.startswith("attention.reduction_") and reduction_reason:
                default = {"attention.reduction_acc_dtype": "fp32", "attention.reduction_order": "global_block_index",
                           "attention.reduction_downcast_at": "final_write"}.get(path)
                bad = (default is not None and v != default) or (path == "attention.reduction_engine" and v == "te_oracle")
                apps.append(application(path, self.target, v, None if bad else v,
                                        status=MaterializationStatus.UNSUPPORTED if bad else MaterializationStatus.APPLIED,
                                        reason=reduction_reason if bad else None))
                continue
            check = checks.get(path)
            if check is None:
                apps.append(application(path, self.target, v, status=MaterializationStatus.UNSUPPORTED,
                                        reason=f"{self.runtime_kind} has no such knob"))
                continue
            reason = check(v)
            if reason:
                apps.append(application(path, self.target, v, status=MaterializationStatus.UNSUPPORTED, reason=reason))
                continue
            actual = self.runtime_readback.get(path)
            status = MaterializationStatus.APPLIED
            if actual is not None and actual != v:
                status = MaterializationStatus.FALLBACK
            apps.append(application(path, self.target, v, v, actual=actual if status is MaterializationStatus.FALLBACK else None,
                                    status=status, reason=f"runtime reports {actual!r}" if status is MaterializationStatus.FALLBACK else None))
            options[path] = v
        if all(a.status is MaterializationStatus.APPLIED for a in apps):
            try:
                options["attention_contract_fingerprint"] = self.build_contract({**normalized}).cross_rank_fingerprint()
            except (ValueError, Exception) as exc:  # noqa: BLE001 - a contract that cannot be built makes the case unsupported
                apps.append(application("attention.contract", self.target, None, status=MaterializationStatus.UNSUPPORTED, reason=str(exc)))
        return AdapterMaterialization(self.target, tuple(apps), options)
