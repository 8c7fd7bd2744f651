"""Sampling support policy: which ids may be drawn under temperature / top-k / top-p
(parity: rl_engine/ops/sampling/policy.py:17-110)."""
from __future__ import annotations

import torch

from rl_kernel_b200.reference.sampling.policy import sampling_keep_mask  # noqa: F401


def keep_threshold(logits: torch.Tensor, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
                   real_vocab: int | None = None) -> torch.Tensor | None:
    """Per-row minimum scaled logit that stays in the support, or None when nothing is cut.
    The sm_100a sampler takes this threshold instead of a [rows, V] mask."""
    if (not top_k or top_k >= logits.shape[1]) and top_p >= 1.0:
        return None
    if logits.is_cuda and logits.dtype == torch.bfloat16 and logits.stride(-1) == 1:
        # native: two histogram passes over the 65536 possible bf16 values, no sort
        from rl_kernel_b200.backends import native as nv

        lg = logits if real_vocab is None else logits[:, :real_vocab]
        thr = torch.empty(lg.shape[0], dtype=torch.float32, device=lg.device)
        nv.sample_keep_threshold(lg, thr, inv_temp=1.0 / max(temperature, 1e-6), top_k=top_k, top_p=top_p)
        return thr
    keep = sampling_keep_mask(logits, temperature=temperature, top_k=top_k, top_p=top_p, real_vocab=real_vocab)
    z = logits.float() / max(temperature, 1e-6)
    return z.masked_fill(~keep, float("inf")).min(dim=-1).values


def vocab_parallel_sampling_keep_mask(local_logits: torch.Tensor, collective, *, temperature: float = 1.0,
                                      top_k: int = 0, top_p: float = 1.0, real_vocab: int | None = None):
    """Keep mask for a vocab shard: shards are gathered in rank order, the policy runs on the full
    row, and the local slice of the mask is returned (parity: policy.py:60-110)."""
    full = collective.all_gather(local_logits.contiguous())          # [tp, rows, V_local]
    tp, rows, vl = full.shape
    keep = sampling_keep_mask(full.permute(1, 0, 2).reshape(rows, tp * vl), temperature=temperature, top_k=top_k,
                              top_p=top_p, real_vocab=real_vocab)
    r = collective.rank
    return keep[:, r * vl:(r + 1) * vl]
