"""Binds an AttentionContract to a framework's attention layer in three tiers: explicit contract >
contract derived from the layer's config > refusal in strict mode (parity: bind_attention_contracts,
rl_engine/integrations/common/attention_binding.py:597)."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Any

from rl_kernel_b200.contracts.operators.attention import AttentionContract, CPLayout
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


def bind_attention_contracts(layers, *, explicit: AttentionContract | None = None, tp_size: int = 1, cp_size: int = 1,
                             cp_layout: str = "zigzag") -> list[AttentionContract]:
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
    ATTENTION_PREPROCESS_MISMATCH = "ATTENTION_PREPROCESS_MISMATCH"
    ATTENTION_PROJECTION_MISMATCH = "ATTENTION_PROJECTION_MISMATCH"
    ATTENTION_CORE_MISMATCH = "ATTENTION_CORE_MISMATCH"
    ATTENTION_BACKEND_MISSING = "ATTENTION_BACKEND_MISSING"
    ATTENTION_NOT_PRODUCTION_READY = "ATTENTION_NOT_PRODUCTION_READY"


class BindingTier(str, Enum):
    """IDENTITY: the two sides do not describe the same computation.  SEMANTIC: they do, but with arithmetic that
    cannot agree bit for bit.  ADVISORY: recorded, not blocking."""
    IDENTITY = "identity"
    SEMANTIC = "semantic"
    ADVISORY = "advisory"


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
