"""Attention knobs of the cross-configuration experiments (parity: rl_engine/integrations/common/knobs.py:20-161):
training-side parallelism, the two determinism switches, reduction knobs (what makes a drift attributable) and
materialisation knobs (differences an experiment measures).  Added to the planner's base knobs."""
from __future__ import annotations

from collections.abc import Mapping

from rl_kernel_b200.validation.cross_config.planner import (_NORMALIZERS, V1_KNOBS, Normalizer, _normalize_choice, _positive_int,
                                                            _strict_bool)
from rl_kernel_b200.validation.cross_config.schema import IsolationScope, KnobDescriptor

MEGATRON_ATTENTION_BACKENDS: tuple[str, ...] = ("flash", "fused", "unfused", "local", "auto")
_K, _E, _P, _D = KnobDescriptor, IsolationScope.ENGINE_CONSTRUCTION, IsolationScope.PROCESS, IsolationScope.DISTRIBUTED_CONTEXT
_BOTH = ("rollout", "training")

WS2_ATTENTION_KNOB_DESCRIPTORS: tuple[KnobDescriptor, ...] = (
    _K("training.tensor_parallel_size", _P, ("training",)),
    _K("training.context_parallel_size", _P, ("training",)),
    _K("training.deterministic_mode", _P, ("training",)),
    _K("rollout.batch_invariant", _P, ("rollout",)),
    # reduction knobs; 'arrival', 'per_block' and 'te_oracle' are control groups, not production values
    _K("attention.reduction_acc_dtype", _E, _BOTH, allowed_values=("fp32", "bf16")),
    _K("attention.reduction_order", _E, _BOTH, allowed_values=("global_block_index", "arrival")),
    _K("attention.reduction_downcast_at", _E, _BOTH, allowed_values=("final_write", "per_block")),
    _K("attention.reduction_engine", _E, _BOTH, allowed_values=("in_op_reference", "in_kernel", "te_oracle")),
    _K("attention.fusion_boundary", _E, _BOTH, allowed_values=("unfused_rope_attention", "fused_rope_attention")),
    _K("attention.split_kv_policy", _E, _BOTH),          # logical KV chunk size; the runtime must report its real boundaries
    _K("rollout.kv_block_size", _E, ("rollout",)),       # the serving engine's page size = the contract's page_size
    _K("training.cp_comm_type", _D, ("training",), allowed_values=("p2p", "all_gather", "a2a", "a2a+p2p", "peer_memory")),
)
WS2_ATTENTION_KNOBS: Mapping[str, KnobDescriptor] = {**V1_KNOBS, **{d.path: d for d in WS2_ATTENTION_KNOB_DESCRIPTORS}}
WS2_ATTENTION_NORMALIZERS: Mapping[str, Normalizer] = {
    **_NORMALIZERS,
    "training.attention_backend": _normalize_choice(*MEGATRON_ATTENTION_BACKENDS),
    "training.tensor_parallel_size": _positive_int, "training.context_parallel_size": _positive_int,
    "training.deterministic_mode": _strict_bool, "rollout.batch_invariant": _strict_bool,
    "attention.reduction_acc_dtype": _normalize_choice("fp32", "bf16"),
    "attention.reduction_order": _normalize_choice("global_block_index", "arrival"),
    "attention.reduction_downcast_at": _normalize_choice("final_write", "per_block"),
    "attention.reduction_engine": _normalize_choice("in_op_reference", "in_kernel", "te_oracle"),
    "attention.fusion_boundary": _normalize_choice("unfused_rope_attention", "fused_rope_attention"),
    "attention.split_kv_policy": _positive_int, "rollout.kv_block_size": _positive_int,
    "training.cp_comm_type": _normalize_choice("p2p", "all_gather", "a2a", "a2a+p2p", "peer_memory"),
}
# the attention experiments replace the base table's Hugging Face backend names by Megatron's
WS2_ATTENTION_KNOBS = {**WS2_ATTENTION_KNOBS, "training.attention_backend": _K("training.attention_backend", _E, ("training",),
                                                                            allowed_values=MEGATRON_ATTENTION_BACKENDS)}

__all__ = ["MEGATRON_ATTENTION_BACKENDS", "WS2_ATTENTION_KNOBS", "WS2_ATTENTION_KNOB_DESCRIPTORS", "WS2_ATTENTION_NORMALIZERS"]
