"""Rollout-side (vLLM) attention materialiser and provenance adapter for cross-configuration experiments (parity:
rl_engine/integrations/engines/rollout/vllm/cross_config.py:124-540).  Reads plain config objects or mappings; vLLM is
never imported."""
from __future__ import annotations

from typing import Any, Mapping, Optional

from rl_kernel_b200.contracts.operators.attention import AttentionMode, AttentionRole
from rl_kernel_b200.integrations._xc_common import AttentionMaterializerBase, fingerprint, value
from rl_kernel_b200.validation.cross_config.determinism import DeterminismProbe, vllm_probe_from_env

VLLM_MODEL_KEYS = ("model", "dtype", "max_model_len", "enforce_eager", "quantization", "disable_cascade_attn", "seed")
VLLM_CACHE_KEYS = ("block_size", "cache_dtype", "enable_prefix_caching", "calculate_kv_scales", "sliding_window")
VLLM_ATTENTION_KEYS = ("backend", "flash_attn_max_num_splits_for_cuda_graph")
VLLM_PARALLEL_KEYS = ("tensor_parallel_size", "pipeline_parallel_size", "data_parallel_size", "prefill_context_parallel_size",
                      "decode_context_parallel_size")
VLLM_FROZEN_ASSERTIONS = {"quantization": None, "disable_cascade_attn": True, "cache_dtype": "auto", "calculate_kv_scales": False,
                          "sliding_window": None, "pipeline_parallel_size": 1, "data_parallel_size": 1}


class VllmProvenanceAdapter:
    framework = "vllm"

    def __init__(self, *, model_config: Any = None, cache_config: Any = None, attention_config: Any = None, parallel_config: Any = None,
                 env: Optional[Mapping[str, str]] = None):
        self.model_config, self.cache_config, self.attention_config, self.parallel_config = model_config, cache_config, attention_config, parallel_config
        self.env = dict(env or {})

    def construction_view(self) -> dict[str, Any]:
        view = {}
        for prefix, cfg, keys in (("model", self.model_config, VLLM_MODEL_KEYS), ("cache", self.cache_config, VLLM_CACHE_KEYS),
                                  ("attention", self.attention_config, VLLM_ATTENTION_KEYS)):
            view.update({f"{prefix}.{k}": value(cfg, k) for k in keys})
        return view

    def distributed_view(self) -> dict[str, Any]:
        return {f"parallel.{k}": value(self.parallel_config, k) for k in VLLM_PARALLEL_KEYS}

    @property
    def construction_fingerprint(self) -> str:
        return fingerprint(self.construction_view())

    @property
    def distributed_context_fingerprint(self) -> str:
        return fingerprint(self.distributed_view())

    def determinism_probe(self) -> DeterminismProbe:
        return vllm_probe_from_env(self.env, model_config=self.model_config)

    def frozen_scope_violations(self) -> tuple[str, ...]:
        """Settings outside the experiments' frozen scope (quantisation, cascade attention, fp8 cache, PP / DP > 1)."""
        src = {"quantization": self.model_config, "disable_cascade_attn": self.model_config, "cache_dtype": self.cache_config,
               "calculate_kv_scales": self.cache_config, "sliding_window": self.cache_config, "pipeline_parallel_size": self.parallel_config,
               "data_parallel_size": self.parallel_config}
        out = []
        for name, want in VLLM_FROZEN_ASSERTIONS.items():
            if src[name] is None:
                continue
            got = value(src[name], name)
            if got is None and want is not None:
                continue                      # not set on this config object
            if got != want:
                out.append(f"{name}={got!r} (expected {want!r})")
        return tuple(out)

    @property
    def kv_page_size(self) -> Optional[int]:
        b = value(self.cache_config, "block_size")
        return None if b is None else int(b)

    def to_dict(self) -> dict[str, Any]:
        return {"framework": self.framework, "construction": self.construction_view(), "distributed_context": self.distributed_view(),
                "construction_fingerprint": self.construction_fingerprint,
                "distributed_context_fingerprint": self.distributed_context_fingerprint,
                "frozen_scope_violations": list(self.frozen_scope_violations()), "kv_page_size": self.kv_page_size,
                "determinism": self.determinism_probe().to_dict()}


class VllmRolloutMaterializer(AttentionMaterializerBase):
    target, side_prefix, role, runtime_kind = "rollout", "rollout", AttentionRole.INFER, "vllm_attention"

    def __init__(self, *, mode: AttentionMode = AttentionMode.CHUNKED_PREFILL, backend_id: str = "rlkernel.b200.paged_attention.v1", **kw):
        super().__init__(mode=mode, backend_id=backend_id, **kw)

    def _checks(self) -> dict:
        div = lambda n, what: (lambda v: None if n % int(v) == 0 else f"{v} does not divide the {n} {what}")  # noqa: E731
        return {"batch.size": lambda v: None, "rollout.tensor_parallel_size": div(self.model.kv_heads, "KV heads"),
                "rollout.context_parallel_size": lambda v: None if self.global_sequence_length % (2 * int(v) * 128) == 0 or int(v) == 1
                else "prefill context parallelism shards whole 128-token pages in 2 x cp chunks",
                "rollout.dtype": lambda v: None if v == "bfloat16" else "the serving kernels compute in bfloat16",
                "rollout.enable_prefix_caching": lambda v: None, "rollout.enforce_eager": lambda v: None,
                "rollout.batch_invariant": lambda v: None if v else "a rollout side that is not batch-invariant cannot anchor a comparison",
                "rollout.kv_block_size": lambda v: None if int(v) == 128 else "the paged attention kernel uses 128-token pages",
                "attention.fusion_boundary": lambda v: None,
                "attention.split_kv_policy": lambda v: "the paged kernel walks a request's pages in one pass (no split-KV)",
                "attention.reduction_engine": lambda v: None if v == "in_kernel" else "remote pages are read inside the attention kernel",
                "attention.reduction_acc_dtype": lambda v: None, "attention.reduction_order": lambda v: None,
                "attention.reduction_downcast_at": lambda v: None,
                "logp.backend": lambda v: None if v in ("native", "rlkernel.b200_linear_logp") else "the rollout log-prob comes from the fused LM head"}


__all__ = ["VLLM_FROZEN_ASSERTIONS", "VllmProvenanceAdapter", "VllmRolloutMaterializer"]
