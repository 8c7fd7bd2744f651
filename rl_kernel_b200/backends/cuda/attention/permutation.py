"""Sequence permutation with an exact inverse in backward (parity:
rl_engine/backends/cuda/attention/permutation.py:9-45): zigzag / contiguous context-parallel
layouts reorder tokens before attention and restore them after it."""
from __future__ import annotations

import torch


class _SequencePermutation(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, order, sequence_dim):
        ctx.save_for_backward(order)
        ctx.sequence_dim = sequence_dim
        return tensor.index_select(sequence_dim, order)

    @staticmethod
    def backward(ctx, grad):
        (order,) = ctx.saved_tensors
        inv = torch.empty_like(order)
        inv[order] = torch.arange(order.numel(), device=order.device, dtype=order.dtype)
        return grad.index_select(ctx.sequence_dim, inv), None, None


def permute_sequence(tensor, order, *, sequence_dim, batch_dim=None):
    """``tensor`` with its ``sequence_dim`` reordered by ``order`` (a permutation; checked)."""
    del batch_dim
    order = order.to(device=tensor.device, dtype=torch.long)
    n = tensor.shape[sequence_dim]
    if order.numel() != n or not torch.equal(torch.sort(order).values, torch.arange(n, device=order.device)):
        raise ValueError("order must be a permutation of the sequence axis")
    return _SequencePermutation.apply(tensor, order, sequence_dim)
