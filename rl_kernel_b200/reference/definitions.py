"""Shared definitions: masked reductions, the plain selected-log-prob gold and drift summaries
(parity: rl_engine/reference/definitions.py:15-142)."""
from __future__ import annotations

import torch


def masked_mean(x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    m = mask.to(x.dtype)
    return (x * m).sum() / m.sum().clamp_min(1.0)


def selected_logprobs_reference(logits: torch.Tensor, token_ids: torch.Tensor, mask: torch.Tensor | None = None,
                                output_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    lp = torch.log_softmax(logits.float(), dim=-1).gather(-1, token_ids.unsqueeze(-1).long()).squeeze(-1)
    if mask is not None:
        lp = lp.masked_fill(~mask.bool(), 0.0)
    return lp.to(output_dtype)


def summarize_kernel_drift(candidate: torch.Tensor, gold: torch.Tensor, mask: torch.Tensor | None = None) -> dict:
    c, g = candidate.float(), gold.float()
    diff = (c - g).abs()
    if mask is not None:
        m = mask.bool()
        diff = diff[m]
        c, g = c[m], g[m]
    n = diff.numel()
    if n == 0:
        return {"count": 0, "max_abs_error": 0.0, "mean_abs_error": 0.0, "mismatch_count": 0,
                "approx_kl": 0.0}
    mism = int((c.view(torch.int32) != g.view(torch.int32)).sum().item())
    d = g - c
    return {"count": n, "max_abs_error": float(diff.max()), "mean_abs_error": float(diff.mean()),
            "mismatch_count": mism, "approx_kl": float((torch.exp(d) - d - 1).mean())}


def masked_sum(x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    return (x * mask.to(x.dtype)).sum()


def active_token_count(mask: torch.Tensor) -> torch.Tensor:
    return mask.bool().sum()


def compute_policy_ratio(logp: torch.Tensor, old_logp: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """exp(logp - old_logp); inactive tokens read as ratio 1."""
    return torch.exp((logp - old_logp.float()).masked_fill(~mask.bool(), 0.0))


def compute_reference_kl(logp: torch.Tensor, ref_logp: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """k3 estimator exp(d) - d - 1 with d = ref_logp - logp; zero on inactive tokens."""
    d = (ref_logp.float() - logp).masked_fill(~mask.bool(), 0.0)
    return torch.exp(d) - d - 1.0
