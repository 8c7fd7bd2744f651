"""RL-shaped synthetic batches for kernel tests and benchmarks (parity: rl_engine/validation/common/
rl_batch.py:13-199): a group of ``samples_per_prompt`` completions per prompt sharing the prompt
tokens, a completion mask of a chosen density, and the per-token tensors a GRPO loss consumes."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch


@dataclass
class SyntheticRLKernelBatch:
    input_ids: torch.Tensor            # [B, P + L]
    attention_mask: torch.Tensor       # [B, P + L] bool
    prompt_mask: torch.Tensor          # [B, P + L] bool
    completion_mask: torch.Tensor      # [B, L] bool
    token_ids: torch.Tensor            # [B, L] completion ids
    rewards: torch.Tensor              # [B]
    advantages: torch.Tensor           # [B, L]
    old_logps: torch.Tensor            # [B, L]
    ref_logps: torch.Tensor            # [B, L]
    valid_indices: torch.Tensor        # flat indices of the active completion tokens
    metadata: dict[str, Any] = field(default_factory=dict)

    @property
    def batch_size(self) -> int:
        return int(self.input_ids.shape[0])

    @property
    def total_seq_len(self) -> int:
        return int(self.input_ids.shape[1])

    @property
    def prompt_len(self) -> int:
        return self.total_seq_len - self.completion_len

    @property
    def completion_len(self) -> int:
        return int(self.token_ids.shape[1])

    # names the single-GPU example uses
    @property
    def num_prompts(self) -> int:
        return int(self.metadata["num_prompts"])

    @property
    def samples_per_prompt(self) -> int:
        return int(self.metadata["samples_per_prompt"])

    @property
    def prompt_ids(self) -> torch.Tensor:
        return self.input_ids[:, : self.prompt_len]

    def flat_completion_mask(self) -> torch.Tensor:
        return self.completion_mask.reshape(-1)

    def flat_token_ids(self) -> torch.Tensor:
        return self.token_ids.reshape(-1)

    def dense_completion_token_ids(self) -> torch.Tensor:
        return self.token_ids

    def dense_completion_values(self, values: torch.Tensor) -> torch.Tensor:
        """Compact [valid] values scattered back to [B, L]; inactive slots are zero."""
        if values.shape[0] != self.valid_indices.numel():
            raise ValueError(f"expected {self.valid_indices.numel()} compact values, got {values.shape[0]}")
        out = torch.zeros(self.batch_size * self.completion_len, *values.shape[1:], device=values.device, dtype=values.dtype)
        out[self.valid_indices.to(values.device)] = values
        return out.view(self.batch_size, self.completion_len, *values.shape[1:])

    def compact_completion_values(self, values: torch.Tensor) -> torch.Tensor:
        return values.reshape(self.batch_size * self.completion_len, *values.shape[2:])[self.valid_indices.to(values.device)]

    def compact_token_ids(self) -> torch.Tensor:
        return self.flat_token_ids()[self.valid_indices]

    def benchmark_metadata(self) -> dict[str, Any]:
        md = dict(self.metadata)
        md["dtype"] = str(md.get("dtype")).removeprefix("torch.")
        md["valid_fraction"] = md["valid_tokens"] / max(1, self.batch_size * self.completion_len)
        return md


def make_synthetic_rl_kernel_batch(*, num_prompts: int, samples_per_prompt: int, prompt_len: int, completion_len: int,
                                   vocab_size: int, valid_density: float = 1.0, dtype: torch.dtype = torch.float32,
                                   device: torch.device | str = "cpu", seed: int = 0) -> SyntheticRLKernelBatch:
    """Deterministic for (arguments, seed) on every device: values are drawn on the CPU and moved."""
    for name, v, lo in (("num_prompts", num_prompts, 1), ("samples_per_prompt", samples_per_prompt, 1),
                        ("prompt_len", prompt_len, 0), ("completion_len", completion_len, 1), ("vocab_size", vocab_size, 2)):
        if v < lo:
            raise ValueError(f"{name} must be at least {lo}")
    if not 0.0 <= valid_density <= 1.0:
        raise ValueError("valid_density must be in [0.0, 1.0]")
    g = torch.Generator().manual_seed(seed)
    B, L, P = num_prompts * samples_per_prompt, completion_len, prompt_len
    prompts = torch.randint(0, vocab_size, (num_prompts, P), generator=g).repeat_interleave(samples_per_prompt, 0)
    completions = torch.randint(0, vocab_size, (B, L), generator=g)
    n_valid = int(round(B * L * valid_density))
    cmask = torch.zeros(B * L, dtype=torch.bool)
    cmask[torch.randperm(B * L, generator=g)[:n_valid]] = True
    cmask = cmask.view(B, L)
    attn = torch.cat([torch.ones(B, P, dtype=torch.bool), cmask], 1)
    pmask = torch.cat([torch.ones(B, P, dtype=torch.bool), torch.zeros(B, L, dtype=torch.bool)], 1)
    rewards = torch.randn(B, generator=g)
    adv, old, ref = (torch.randn(B, L, generator=g) for _ in range(3))
    dev = torch.device(device)
    md = {"num_prompts": num_prompts, "samples_per_prompt": samples_per_prompt, "batch_size": B, "prompt_len": P,
          "completion_len": L, "total_seq_len": P + L, "vocab_size": vocab_size, "valid_density": valid_density,
          "valid_tokens": n_valid, "dtype": dtype, "device": str(dev), "seed": seed}
    return SyntheticRLKernelBatch(torch.cat([prompts, completions], 1).to(dev), attn.to(dev), pmask.to(dev), cmask.to(dev),
                                  completions.to(dev), rewards.to(dtype).to(dev), adv.to(dtype).to(dev), old.to(dtype).to(dev),
                                  ref.to(dtype).to(dev), cmask.reshape(-1).nonzero().squeeze(-1).to(dev), md)


SyntheticRLBatch = SyntheticRLKernelBatch

__all__ = ["SyntheticRLBatch", "SyntheticRLKernelBatch", "make_synthetic_rl_kernel_batch"]
