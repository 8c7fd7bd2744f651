"""Sampling support (temperature, top-k, top-p) over the real vocabulary: the keep mask is built
from an ascending-stable sort so ties resolve the same way everywhere
(parity: sampling_keep_mask, rl_engine/ops/sampling/policy.py:17-52)."""
from __future__ import annotations

import torch


def sampling_keep_mask(logits: torch.Tensor, *, temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0,
                       real_vocab: int | None = None) -> torch.Tensor:
    """Boolean [rows, V]: ids that may be sampled. Always keeps the arg-max."""
    rows, V = logits.shape
    z = logits.float() / max(temperature, 1e-6)
    if real_vocab is not None and real_vocab < V:
        z[:, real_vocab:] = float("-inf")
    keep = torch.isfinite(z)
    if top_k and top_k < V:
        kth = torch.topk(z, top_k, dim=-1).values[:, -1:]
        keep &= z >= kth
    if top_p < 1.0:
        zs, idx = torch.sort(z, dim=-1, descending=True, stable=True)
        p = torch.softmax(zs, dim=-1)
        cum = p.cumsum(-1)
        drop = (cum - p) >= top_p          # ids whose preceding mass already reaches top_p
        drop[:, 0] = False
        keep &= torch.zeros_like(keep).scatter(1, idx, ~drop)
    return keep


def sample_from_logits(logits, *, temperature=1.0, top_k=0, top_p=1.0, generator=None, real_vocab=None):
    keep = sampling_keep_mask(logits, temperature=temperature, top_k=top_k, top_p=top_p, real_vocab=real_vocab)
    z = (logits.float() / max(temperature, 1e-6)).masked_fill(~keep, float("-inf"))
    return torch.multinomial(torch.softmax(z, -1), 1, generator=generator).squeeze(-1)
