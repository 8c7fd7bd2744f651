"""Shared validation helpers (parity: rl_engine/validation/common.py as used by
examples/post_training/grpo_single_gpu.py)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from rl_kernel_b200.reference.definitions import (masked_mean, selected_logprobs_reference,  # noqa: F401
                                                  summarize_kernel_drift)


@dataclass
class SyntheticRLBatch:
    token_ids: torch.Tensor          # [B, L] completion ids
    prompt_ids: torch.Tensor         # [B, P]
    completion_mask: torch.Tensor    # [B, L] bool
    num_prompts: int
    samples_per_prompt: int

    @property
    def batch_size(self) -> int:
        return self.token_ids.shape[0]

    @property
    def completion_len(self) -> int:
        return self.token_ids.shape[1]


def make_synthetic_rl_kernel_batch(*, num_prompts: int, samples_per_prompt: int, prompt_len: int, completion_len: int,
                                   vocab_size: int, valid_density: float = 1.0, dtype=torch.float32, device="cpu",
                                   seed: int = 0) -> SyntheticRLBatch:
    g = torch.Generator().manual_seed(seed)
    B = num_prompts * samples_per_prompt
    prompts = torch.randint(0, vocab_size, (num_prompts, prompt_len), generator=g).repeat_interleave(samples_per_prompt, 0)
    toks = torch.randint(0, vocab_size, (B, completion_len), generator=g)
    lens = (torch.rand(B, generator=g) * (1 - valid_density) * completion_len).long()
    mask = torch.arange(completion_len)[None, :] < (completion_len - lens)[:, None]
    return SyntheticRLBatch(toks.to(device), prompts.to(device), mask.to(device), num_prompts, samples_per_prompt)


def active_token_count(mask: torch.Tensor) -> torch.Tensor:
    return mask.bool().sum()


def compute_policy_ratio(logp: torch.Tensor, old_logp: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return torch.exp((logp - old_logp.float()).masked_fill(~mask.bool(), 0.0))


def compute_reference_kl(logp: torch.Tensor, ref_logp: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    d = (ref_logp.float() - logp).masked_fill(~mask.bool(), 0.0)
    return torch.exp(d) - d - 1.0
