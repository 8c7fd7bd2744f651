"""Qwen3-style decoder with a routed mixture-of-experts feed-forward block: every layer keeps the
dense family's attention (QK-norm, RoPE, GQA) and replaces the MLP by a softmax top-k router over
``num_experts`` SwiGLU experts plus one always-on shared expert.  The reference lists this family
as roadmap (docs/blog/2026-08-09-dsv4-flash-moe-consistency-roadmap.md:120-134) and pins expert
parallelism to 1 (rl_engine/validation/cross_config/run_arm.py:652); here it is a runnable stack.
"""
from __future__ import annotations

from dataclasses import dataclass

from rl_kernel_b200.models.qwen3.spec import Qwen3DenseSpec


@dataclass(frozen=True)
class Qwen3MoeSpec(Qwen3DenseSpec):
    """``intermediate_size`` is the shared expert's width; attention runs data parallel, so the
    canonical tensor-parallel degree is 1."""
    num_experts: int = 128
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 1536

    def __post_init__(self) -> None:
        super().__post_init__()
        if self.canonical_tp != 1:
            raise ValueError("the MoE stack shards experts, not attention: canonical_tp must be 1")
        if self.num_experts not in (32, 64, 128, 256):
            raise ValueError("num_experts must be 32, 64, 128 or 256")
        if not 1 <= self.num_experts_per_tok <= min(32, self.num_experts):
            raise ValueError("num_experts_per_tok out of range")
        if self.hidden_size % 256 or self.moe_intermediate_size % 256:
            raise ValueError("hidden and expert widths must be multiples of 256")

    @classmethod
    def roadmap(cls, layers: int = 8) -> "Qwen3MoeSpec":
        """8 layers, hidden 4096, 128 routed experts of width 1536 (top-8) + one shared expert."""
        return cls(num_hidden_layers=layers, hidden_size=4096, intermediate_size=1536, num_attention_heads=32,
                   num_key_value_heads=8, head_dim=128, vocab_size=151936, canonical_tp=1,
                   model_id=f"qwen3-moe-roadmap-{layers}L", num_experts=128, num_experts_per_tok=8,
                   moe_intermediate_size=1536)

    @classmethod
    def tiny(cls, *, layers: int = 2, hidden: int = 512, experts: int = 32, top_k: int = 4, expert_ffn: int = 256,
             shared_ffn: int = 256, q_heads: int = 4, kv_heads: int = 2, vocab: int = 2048) -> "Qwen3MoeSpec":
        return cls(num_hidden_layers=layers, hidden_size=hidden, intermediate_size=shared_ffn,
                   num_attention_heads=q_heads, num_key_value_heads=kv_heads, head_dim=128, vocab_size=vocab,
                   canonical_tp=1, model_id=f"qwen3-moe-tiny-{layers}x{hidden}", num_experts=experts,
                   num_experts_per_tok=top_k, moe_intermediate_size=expert_ffn)

    def param_count(self) -> int:
        h = self.hidden_size
        routed = self.num_experts * 3 * h * self.moe_intermediate_size + self.num_experts * h
        return super().param_count() + self.num_hidden_layers * routed

    def active_param_count(self) -> int:
        h = self.hidden_size
        routed = self.num_experts_per_tok * 3 * h * self.moe_intermediate_size + self.num_experts * h
        return super().param_count() + self.num_hidden_layers * routed
