"""Selected-token log-prob from logits, the plain definition
(parity: NativeLogpOp, rl_engine/reference/logprob/logp.py:9)."""
from __future__ import annotations

import torch


class NativeLogpOp:
    is_fused_logp = False

    def __call__(self, logits: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        return self.apply_fp32(logits, token_ids).to(logits.dtype)

    forward = __call__

    def apply_fp32(self, logits: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        lf = logits.float()
        return torch.log_softmax(lf, dim=-1).gather(-1, token_ids.unsqueeze(-1).long()).squeeze(-1)
