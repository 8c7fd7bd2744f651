"""Rank-ordered merge of vocabulary-shard (lse, target-logit) pairs
(parity: rl_engine/backends/cuda/logprob/ordered_merge.py:6)."""
from __future__ import annotations

import torch


def ordered_logp_merge(local_lse: torch.Tensor, local_target: torch.Tensor):
    """local_lse / local_target [tp, rows] fp32 in rank order -> (logp [rows], lse [rows]).

    M = max_r lse_r; S = sum_r exp(lse_r - M) in ascending r; lse = M + log S;
    logp = (sum_r target_r) - lse, where exactly one rank holds a non-zero target logit per row."""
    if local_lse.dim() != 2 or local_lse.shape != local_target.shape:
        raise ValueError("local_lse and local_target must be [tp, rows]")
    lse32, tgt32 = local_lse.float(), local_target.float()
    M = lse32.max(dim=0).values
    safe = torch.where(torch.isinf(M), torch.zeros_like(M), M)
    S = torch.zeros_like(M)
    for r in range(lse32.shape[0]):
        S = S + torch.where(torch.isinf(lse32[r]), torch.zeros_like(S), torch.exp(lse32[r] - safe))
    lse = safe + torch.log(S)
    tgt = torch.zeros_like(M)
    for r in range(tgt32.shape[0]):
        tgt = tgt + tgt32[r]
    return tgt - lse, lse
