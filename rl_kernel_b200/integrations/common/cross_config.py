"""Pieces shared by the rollout- and training-side attention materialisers (parity: rl_engine/integrations/common/
cross_config.py:46-281): the frozen model geometry, knob -> contract translation, and the reasons a requested reduction
cannot be honoured."""
from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any

from rl_kernel_b200.contracts.operators.attention import (AttentionDType, CPLayout, ReductionEngine, ReductionSpec, ShardingSpec,
                                                          SplitKVSpec)
from rl_kernel_b200.validation.cross_config.runtime import KnobApplication
from rl_kernel_b200.validation.cross_config.schema import MaterializationStatus


@dataclass(frozen=True)
class Qwen3ModelSpec:
    """Architecture constants of the dense target: not knobs; both sides must agree on them or the comparison is void."""
    name: str = "qwen3-8b"
    hidden_size: int = 4096
    ffn_hidden_size: int = 12288
    num_layers: int = 36
    q_heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 151936
    rope_theta: float = 1_000_000.0
    rotary_dim: int = 128
    rms_norm_eps: float = 1e-6

    def fingerprint_payload(self) -> dict[str, Any]:
        return dict(self.__dict__)


QWEN3_8B = Qwen3ModelSpec()


def flatten(value: Mapping[str, Any], prefix: str = "") -> dict[str, Any]:
    out: dict[str, Any] = {}
    for k, v in value.items():
        path = f"{prefix}.{k}" if prefix else str(k)
        if isinstance(v, Mapping):
            out.update(flatten(v, path))
        else:
            out[path] = v
    return out


def application(path: str, target: str, requested: Any, materialized: Any = None, *, actual: Any = None,
                status: MaterializationStatus = MaterializationStatus.APPLIED, reason: str | None = None) -> KnobApplication:
    return KnobApplication(path, target, requested, materialized, actual, status, {"reason": reason} if reason else {})


def attention_dtype(value: Any, *, field: str) -> AttentionDType:
    name = {"bfloat16": "bf16", "float16": "fp16", "float32": "fp32"}.get(str(value).removeprefix("torch."), str(value))
    try:
        return AttentionDType(name)
    except ValueError:
        raise ValueError(f"{field}: {value!r} is not an attention dtype") from None


def split_kv_spec(flat: Mapping[str, Any]) -> SplitKVSpec:
    size = flat.get("attention.split_kv_policy")
    return SplitKVSpec.disabled() if size is None else SplitKVSpec.fixed(int(size))


def unsupported_reduction_reason(flat: Mapping[str, Any]) -> str | None:
    """Why the requested reduction knobs cannot be materialised, or None.  The control-group values describe arithmetic
    this framework's kernels never perform; they are refused, not approximated."""
    if flat.get("attention.reduction_acc_dtype", "fp32") != "fp32":
        return "partial attention states accumulate in fp32; a bf16 accumulator is a control group no kernel here implements"
    if flat.get("attention.reduction_order", "global_block_index") != "global_block_index":
        return "blocks are reduced in ascending global block index; arrival order is a control group"
    if flat.get("attention.reduction_downcast_at", "final_write") != "final_write":
        return "results are rounded once at the final write; per-block downcast is a control group"
    if flat.get("attention.reduction_engine", "in_kernel") == "te_oracle":
        return "Transformer Engine is not part of this runtime"
    return None


def build_reduction_spec(flat: Mapping[str, Any]) -> ReductionSpec:
    reason = unsupported_reduction_reason(flat)
    if reason:
        raise ValueError(reason)
    return ReductionSpec(engine=ReductionEngine(flat.get("attention.reduction_engine", "in_kernel")))


def build_sharding_spec(*, model: Qwen3ModelSpec, tp_rank: int, tp_world_size: int, cp_rank: int, cp_world_size: int,
                        global_sequence_length: int, layout: str | None = None) -> ShardingSpec:
    if model.q_heads % tp_world_size or model.kv_heads % tp_world_size:
        raise ValueError(f"tensor parallel size {tp_world_size} must divide {model.q_heads} query and {model.kv_heads} KV heads")
    lay = CPLayout.NONE if cp_world_size == 1 else CPLayout(layout or "zigzag")
    return ShardingSpec.for_layout(num_q_heads=model.q_heads, num_kv_heads=model.kv_heads, seq_len=global_sequence_length, tp_rank=tp_rank,
                                   tp_world_size=tp_world_size, cp_rank=cp_rank, cp_world_size=cp_world_size, layout=lay)


def causal_offsets_for(sharding: ShardingSpec, batch_size: int) -> tuple[int, ...]:
    """Causal offsets are expressed in global positions: every sequence starts at 0 whatever the rank owns."""
    return (0,) * batch_size


__all__ = ["QWEN3_8B", "Qwen3ModelSpec", "application", "attention_dtype", "build_reduction_spec", "build_sharding_spec",
           "causal_offsets_for", "flatten", "split_kv_spec", "unsupported_reduction_reason"]
