"""Contract between the orchestrator and training / scoring workers (parity:
rl_engine/integrations/engines/train/contract.py:22-1026)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Protocol

import torch

from rl_kernel_b200.ops.loss import group_advantages


@dataclass
class RolloutStageResult:
    tokens: torch.Tensor            # [B, S] prompt + response
    response_mask: torch.Tensor     # [B, R]
    rollout_logp: torch.Tensor      # [B, R] fp32, recorded by the sampler with the strict operator
    rewards: torch.Tensor           # [B]
    prompt_len: int
    samples_per_prompt: int
    weight_version: int = 0
    metadata: dict = field(default_factory=dict)

    def validate(self) -> None:
        B, R = self.rollout_logp.shape
        if self.tokens.shape[0] != B or self.response_mask.shape != (B, R) or self.rewards.shape[0] != B:
            raise ValueError("rollout result tensors disagree on the batch / response size")
        if self.tokens.shape[1] != self.prompt_len + R:
            raise ValueError("tokens must be prompt_len + response_len wide")
        if B % self.samples_per_prompt:
            raise ValueError("batch must be a multiple of samples_per_prompt")


@dataclass
class TrainingStageResult:
    loss: float
    policy_loss: float
    kl: float
    grad_norm: float
    train_logp: torch.Tensor
    mismatch_count: int
    tokens_compared: int
    weight_version: int
    metrics: dict = field(default_factory=dict)


class TrainingWorker(Protocol):
    def train(self, rollout: RolloutStageResult) -> TrainingStageResult: ...
    def publish_weights(self, weight_version: int): ...


class RolloutBatchMixin:
    @staticmethod
    def advantages(rollout: RolloutStageResult, eps: float = 1e-6) -> torch.Tensor:
        return group_advantages(rollout.rewards, rollout.samples_per_prompt, eps)

    @staticmethod
    def mismatches(train_logp: torch.Tensor, rollout: RolloutStageResult) -> int:
        m = rollout.response_mask.bool()
        return int(((train_logp.view(torch.int32) != rollout.rollout_logp.view(torch.int32)) & m).sum())


class StatelessScoringWorker:
    """Reference / reward scoring worker: no KV cache, no state between calls."""

    def __init__(self, executor):
        self.executor = executor

    def score(self, rollout: RolloutStageResult) -> torch.Tensor:
        lp = self.executor.score(rollout.tokens)
        return lp[:, -rollout.rollout_logp.shape[1]:]
