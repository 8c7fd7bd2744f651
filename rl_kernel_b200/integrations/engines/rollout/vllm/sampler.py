"""Shared-prefix sampler: the G samples of a GRPO group share the prompt, so the prompt is prefilled
once and its KV is shared by the group (parity: VLLMSharedPrefixSampler,
rl_engine/integrations/engines/rollout/vllm/sampler.py:77)."""
from __future__ import annotations

import torch


class SharedPrefixSampler:
    def __init__(self, trainer):
        """``trainer`` is a models.qwen3.grpo.GRPOTrainer (its rollout already shares prompt KV)."""
        self.trainer = trainer

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, seed: int = 0):
        return self.trainer.rollout(prompts, step_seed=seed)
