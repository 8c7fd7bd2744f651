"""Training-side (Megatron) attention materialiser and provenance adapter (parity: rl_engine/integrations/engines/train/
megatron/cross_config.py:137-481).  Works on a ``TransformerConfig``-like object, a namespace or a mapping."""
from __future__ import annotations

from typing import Any, Mapping, Optional

from rl_kernel_b200.contracts.operators.attention import AttentionMode, AttentionRole
from rl_kernel_b200.integrations._xc_common import AttentionMaterializerBase, fingerprint, value
from rl_kernel_b200.validation.cross_config.determinism import DeterminismProbe, megatron_probe_from_config

MEGATRON_CONSTRUCTION_KEYS = ("num_layers", "hidden_size", "ffn_hidden_size", "num_attention_heads", "num_query_groups", "kv_channels",
                              "attention_backend", "qk_layernorm", "normalization", "bf16", "params_dtype", "deterministic_mode",
                              "cross_entropy_loss_fusion", "apply_rope_fusion")
MEGATRON_DISTRIBUTED_KEYS = ("tensor_model_parallel_size", "context_parallel_size", "pipeline_model_parallel_size", "sequence_parallel",
                             "cp_comm_type", "expert_model_parallel_size")
MEGATRON_FROZEN_ASSERTIONS = {"pipeline_model_parallel_size": 1, "expert_model_parallel_size": 1, "qk_layernorm": True, "bf16": True}


class MegatronProvenanceAdapter:
    framework = "megatron"

    def __init__(self, config: Any = None, *, env: Optional[Mapping[str, str]] = None):
        self.config, self.env = config, dict(env or {})

    def construction_view(self) -> dict[str, Any]:
        return {k: value(self.config, k) for k in MEGATRON_CONSTRUCTION_KEYS}

    def distributed_view(self) -> dict[str, Any]:
        return {k: value(self.config, k) for k in MEGATRON_DISTRIBUTED_KEYS}

    @property
    def construction_fingerprint(self) -> str:
        return fingerprint(self.construction_view())

    @property
    def distributed_context_fingerprint(self) -> str:
        return fingerprint(self.distributed_view())

    def determinism_probe(self) -> DeterminismProbe:
        return megatron_probe_from_config(self.config, self.env)

    def frozen_scope_violations(self) -> tuple[str, ...]:
        out = []
        for name, want in MEGATRON_FROZEN_ASSERTIONS.items():
            got = value(self.config, name)
            if got is not None and got != want:
                out.append(f"{name}={got!r} (expected {want!r})")
        return tuple(out)

    def to_dict(self) -> dict[str, Any]:
        return {"framework": self.framework, "construction": self.construction_view(), "distributed_context": self.distributed_view(),
                "construction_fingerprint": self.construction_fingerprint,
                "distributed_context_fingerprint": self.distributed_context_fingerprint,
                "frozen_scope_violations": list(self.frozen_scope_violations()), "determinism": self.determinism_probe().to_dict()}


class MegatronAttentionMaterializer(AttentionMaterializerBase):
    target, side_prefix, role, runtime_kind = "training", "training", AttentionRole.TRAIN, "megatron_attention"

    def __init__(self, *, mode: AttentionMode = AttentionMode.PREFILL, backend_id: str = "rlkernel.b200.cp_attention.v1", **kw):
        super().__init__(mode=mode, backend_id=backend_id, **kw)

    def _checks(self) -> dict:
        div = lambda n, what: (lambda v: None if n % int(v) == 0 else f"{v} does not divide the {n} {what}")  # noqa: E731
        return {"batch.size": lambda v: None, "training.tensor_parallel_size": div(self.model.kv_heads, "KV heads"),
                "training.context_parallel_size": lambda v: None if self.global_sequence_length % (2 * int(v)) == 0
                else "zigzag context parallelism cuts the sequence into 2 x cp chunks",
                "training.compute_dtype": lambda v: None if v == "bfloat16" else "the training kernels compute in bfloat16",
                "training.attention_backend": lambda v: None if v in ("auto", "local", "model_default") else
                f"attention backend {v!r} is replaced by this framework's operator; name it 'local' or 'auto'",
                "training.deterministic_mode": lambda v: None if v else "a training side that is not deterministic cannot anchor a comparison",
                "training.sharding": lambda v: None if v == "unsharded" else "parameter sharding is ZeRO over the DP group, not FSDP",
                "training.cp_comm_type": lambda v: None if v in ("peer_memory", "all_gather") else
                f"cp_comm_type {v!r}: this runtime reads remote K/V over peer memory or gathers it; ring exchanges are not built",
                "attention.fusion_boundary": lambda v: None, "attention.split_kv_policy": lambda v: None if int(v) % 128 == 0
                else "a fixed KV split must be a multiple of the 128-key block",
                "attention.reduction_engine": lambda v: None, "attention.reduction_acc_dtype": lambda v: None,
                "attention.reduction_order": lambda v: None, "attention.reduction_downcast_at": lambda v: None,
                "logp.backend": lambda v: None if v in ("native", "rlkernel.b200_linear_logp", "rlkernel.reference_logp") else "unknown log-prob backend"}


__all__ = ["MEGATRON_FROZEN_ASSERTIONS", "MegatronAttentionMaterializer", "MegatronProvenanceAdapter"]
