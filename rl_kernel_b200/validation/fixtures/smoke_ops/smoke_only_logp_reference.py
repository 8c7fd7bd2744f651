"""Smoke-only selected-log-prob operator: plain fp32 log-softmax + gather (parity: SmokeOnlyLogpReference,
rl_engine/validation/fixtures/smoke_ops/smoke_only_logp_reference.py:20-112).  It exists so that the cross-configuration
runner can be exercised with an operator that is obviously not a production kernel; it registers under a ``smoke_only.``
id and is refused outside smoke runs."""
from __future__ import annotations

import torch

BACKEND_ID = "smoke_only.logp_reference"


def _validate(logits: torch.Tensor, token_ids: torch.Tensor) -> None:
    if logits.dim() < 2 or logits.shape[:-1] != token_ids.shape:
        raise ValueError(f"logits {tuple(logits.shape)} and token_ids {tuple(token_ids.shape)} do not line up")
    if token_ids.dtype != torch.long:
        raise ValueError("token_ids must be int64")
    if bool(((token_ids < 0) | (token_ids >= logits.shape[-1])).any()):
        raise ValueError("token ids outside the vocabulary")


class SmokeOnlyLogpReference:
    backend_id = BACKEND_ID
    smoke_only = True
    is_fused_logp = False

    def __init__(self, temperature: float = 1.0):
        if temperature <= 0:
            raise ValueError("temperature must be positive")
        self.temperature = temperature

    def __call__(self, logits: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        return self.forward(logits, token_ids)

    def forward(self, logits: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        _validate(logits, token_ids)
        lp = torch.log_softmax(logits.float() / self.temperature, -1)
        return lp.gather(-1, token_ids.unsqueeze(-1)).squeeze(-1)

    def forward_with_lse(self, logits: torch.Tensor, token_ids: torch.Tensor):
        _validate(logits, token_ids)
        z = logits.float() / self.temperature
        lse = torch.logsumexp(z, -1)
        return z.gather(-1, token_ids.unsqueeze(-1)).squeeze(-1) - lse, lse


__all__ = ["BACKEND_ID", "SmokeOnlyLogpReference"]
