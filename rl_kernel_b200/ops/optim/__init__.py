"""Optimizer operators: fused AdamW over flat bf16/fp32 shards (see models.qwen3.grpo.AdamW)."""
from rl_kernel_b200.models.qwen3.grpo import AdamW  # noqa: F401
