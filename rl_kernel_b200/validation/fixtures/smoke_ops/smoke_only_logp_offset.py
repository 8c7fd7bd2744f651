"""Smoke-only operator that is wrong on purpose: the reference log-prob plus a fixed offset (parity: SmokeOnlyLogpOffset,
rl_engine/validation/fixtures/smoke_ops/smoke_only_logp_offset.py:22-97).  A harness that does not turn red with this
operator installed on one side is not measuring anything.  Host-side only."""
from __future__ import annotations

import torch

from rl_kernel_b200.validation.fixtures.smoke_ops.smoke_only_logp_reference import SmokeOnlyLogpReference

BACKEND_ID = "smoke_only.logp_offset"


class SmokeOnlyLogpOffset(SmokeOnlyLogpReference):
    backend_id = BACKEND_ID

    def __init__(self, offset: float = 0.25, temperature: float = 1.0):
        super().__init__(temperature)
        if offset == 0:
            raise ValueError("an offset of zero makes this the reference operator")
        self.offset = float(offset)

    def forward(self, logits: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        return super().forward(logits, token_ids) + self.offset

    def forward_with_lse(self, logits: torch.Tensor, token_ids: torch.Tensor):
        lp, lse = super().forward_with_lse(logits, token_ids)
        return lp + self.offset, lse


__all__ = ["BACKEND_ID", "SmokeOnlyLogpOffset"]
