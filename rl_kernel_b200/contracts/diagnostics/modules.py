"""First-line debug axes of the three semantic operators -- attention, FFN, selected log-prob -- in one manifest (parity:
rl_engine/contracts/diagnostics/modules.py:23-183).  ``gate`` axes decide whether two runs are comparable at all;
``diagnostic`` axes are measured."""
from __future__ import annotations

from dataclasses import dataclass
from types import MappingProxyType
from typing import Any

from rl_kernel_b200.contracts.diagnostics.attention_axes import ATTENTION_DEBUG_AXES
from rl_kernel_b200.contracts.diagnostics.attention_matrix import (ATTENTION_DEBUG_MATRIX, ATTENTION_DEBUG_MATRIX_SCHEMA_VERSION,
                                                                   GATE_AXIS)

DEBUG_MATRIX_SCHEMA_VERSION = "rlkernel.debug_matrix.v1"


@dataclass(frozen=True)
class ModuleDebugAxis:
    module: str
    axis_id: str
    label: str
    representative_probe: str
    kind: str = "diagnostic"

    def __post_init__(self) -> None:
        for f in ("module", "axis_id", "label", "representative_probe"):
            v = getattr(self, f)
            if not isinstance(v, str) or not v.strip():
                raise ValueError(f"module debug {f} must be a non-empty string")
        if self.kind not in ("diagnostic", "gate"):
            raise ValueError(f"unknown module debug axis kind {self.kind!r}")

    def to_dict(self, *, row_id: str) -> dict[str, str]:
        return {"row": row_id, "id": self.axis_id, "label": self.label, "representative_probe": self.representative_probe,
                "kind": self.kind}


_M = ModuleDebugAxis
MODULE_DEBUG_AXES: MappingProxyType = MappingProxyType({
    "attention": tuple(_M("attention", a.axis_id, a.label, a.representative_subprobe, "gate" if a.axis_id == GATE_AXIS else "diagnostic")
                       for a in ATTENTION_DEBUG_AXES),
    "ffn": (_M("ffn", "weight_shard_ownership", "Weight shard / TP ownership", "tp_weight_ownership", "gate"),
            _M("ffn", "swiglu_rounding", "SwiGLU intermediate rounding", "swiglu_one_round"),
            _M("ffn", "gemm_reduction", "GEMM K-reduction / Split-K policy", "k_reduction_split_k"),
            _M("ffn", "token_collective", "Token gather / reduce-scatter", "sequence_parallel")),
    "logp": (_M("logp", "vocab_shard_ownership", "Vocabulary shard / TP ownership", "vocab_shard_bounds", "gate"),
             _M("logp", "selected_token_identity", "Selected-token and active-mask identity", "selected_token_active_mask", "gate"),
             _M("logp", "vocab_lse_reduction", "Vocabulary LSE tile / merge policy", "vocab_tile_merge")),
})
_BY_ID = MappingProxyType({(a.module, a.axis_id): a for axes in MODULE_DEBUG_AXES.values() for a in axes})
_BASELINE = {"attention": "A0", "ffn": "F0", "logp": "L0"}
_CONTROLS = {"attention": ["C0", "C1", "C2"], "ffn": ["FC0"], "logp": ["LC0"]}


def _module_rows(module: str) -> dict[str, Any]:
    axes = MODULE_DEBUG_AXES[module]
    rows = [_BASELINE[module]] + [f"{module[0].upper()}{i}" for i in range(1, len(axes) + 1)]
    return {"baseline_row": _BASELINE[module], "rows": rows, "invariant_controls": _CONTROLS[module],
            "axes": [a.to_dict(row_id=rows[i]) for i, a in enumerate(axes, start=1)]}


def module_debug_matrix() -> dict[str, Any]:
    return {"schema_version": DEBUG_MATRIX_SCHEMA_VERSION, "method": "fixed_replay_one_at_a_time", "cartesian_product": False,
            "comparison_edges": ["train_vs_rollout_prefill", "rollout_prefill_vs_decode"],
            "replay_identity": "same checkpoint, token IDs, selected-token IDs, masks, positions, cache metadata, and pre-update model state",
            "modules": {m: _module_rows(m) for m in MODULE_DEBUG_AXES},
            "attention_compatibility": {"schema_version": ATTENTION_DEBUG_MATRIX_SCHEMA_VERSION,
                                        "rows": [r.to_dict() for r in ATTENTION_DEBUG_MATRIX]}}


def module_debug_axis(module: str, axis_id: str) -> ModuleDebugAxis:
    try:
        return _BY_ID[(module, axis_id)]
    except KeyError:
        raise KeyError(f"unknown debug axis {axis_id!r} of module {module!r}") from None


__all__ = ["DEBUG_MATRIX_SCHEMA_VERSION", "MODULE_DEBUG_AXES", "ModuleDebugAxis", "module_debug_axis", "module_debug_matrix"]
