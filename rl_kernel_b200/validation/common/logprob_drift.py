"""Absolute-drift summaries of selected log-probs (parity: rl_engine/validation/common/logprob_drift.py:14-57)."""
from __future__ import annotations

from dataclasses import asdict, dataclass

import torch


@dataclass(frozen=True)
class LogprobDriftStats:
    max_abs: float
    mean_abs: float
    p95_abs: float
    p99_abs: float
    active_count: int

    def to_dict(self) -> dict:
        return asdict(self)

    @property
    def bitwise_zero(self) -> bool:
        return self.active_count > 0 and self.max_abs == 0.0


def _quantile(sorted_values: torch.Tensor, q: float) -> float:
    """Linear-interpolated quantile of an ascending 1-D tensor of any length (torch.quantile caps the input size)."""
    n = sorted_values.numel()
    pos = q * (n - 1)
    lo = int(pos)
    hi = min(lo + 1, n - 1)
    return float(sorted_values[lo] + (sorted_values[hi] - sorted_values[lo]) * (pos - lo))


def summarize_logprob_drift(candidate: torch.Tensor, reference: torch.Tensor, *, mask: torch.Tensor | None = None) -> LogprobDriftStats:
    """|candidate - reference| over all entries, or over the entries where the bool ``mask`` is set."""
    if candidate.shape != reference.shape:
        raise ValueError(f"candidate shape {tuple(candidate.shape)} must match reference shape {tuple(reference.shape)}")
    diff = (candidate.double() - reference.double().to(candidate.device)).abs()
    if mask is not None:
        if mask.shape != diff.shape:
            raise ValueError("mask shape must match candidate and reference")
        if mask.dtype != torch.bool:
            raise ValueError("mask must be bool")
        diff = diff[mask.to(diff.device)]
    vals = diff.reshape(-1)
    if vals.numel() == 0:
        return LogprobDriftStats(0.0, 0.0, 0.0, 0.0, 0)
    s = vals.sort().values
    return LogprobDriftStats(float(s[-1]), float(vals.mean()), _quantile(s, 0.95), _quantile(s, 0.99), int(vals.numel()))


__all__ = ["LogprobDriftStats", "summarize_logprob_drift"]
