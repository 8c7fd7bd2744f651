"""Smoke-only operators used to prove that the harness detects a mismatch: ``logp_offset`` adds a
deliberate offset to the scores (parity: rl_engine/validation/fixtures/smoke_ops/
smoke_only_logp_offset.py).  Host-side fault injection only."""
from __future__ import annotations

import torch


def apply_operator_override(name: str | None, score: torch.Tensor) -> torch.Tensor:
    if name in (None, "", "none"):
        return score
    if name == "smoke_only.logp_offset":
        return score + torch.finfo(score.dtype).eps * 4
    if name == "smoke_only.flip_last_bit":
        v = score.clone().view(torch.int32 if score.dtype == torch.float32 else torch.int16)
        v[..., 0] ^= 1
        return v.view(score.dtype)
    raise ValueError(f"unknown operator override {name!r}")
