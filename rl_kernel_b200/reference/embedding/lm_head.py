"""LM-head reference operator (parity: NativeLMHeadOp, rl_engine/reference/embedding/lm_head.py:12-135):
``logits = hidden @ weight^T (+ bias)`` with one fp32 matmul as the gold path."""
from __future__ import annotations

import torch


class NativeLMHeadOp:
    op_class = "reduction"

    def __call__(self, hidden: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        return self.forward(hidden, weight, bias)

    def forward(self, hidden: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        """hidden [..., H], weight [V, H] -> logits [..., V] in hidden's dtype (rounded once)."""
        return self.forward_fp32(hidden, weight, bias).to(hidden.dtype)

    def forward_fp32(self, hidden: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        if hidden.shape[-1] != weight.shape[-1]:
            raise ValueError(f"hidden size {hidden.shape[-1]} does not match the weight's {weight.shape[-1]}")
        y = torch.matmul(hidden.float(), weight.float().t())
        return y if bias is None else y + bias.float()

    def vocab_parallel(self, hidden: torch.Tensor, weight_shard: torch.Tensor, *, gather=None) -> torch.Tensor:
        """Logits of one vocabulary shard; ``gather`` (a callable concatenating shards along the last axis) assembles the
        full row when the caller needs it."""
        y = self.forward(hidden, weight_shard)
        return gather(y) if gather is not None else y


__all__ = ["NativeLMHeadOp"]
