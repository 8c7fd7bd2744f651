"""Embedding gather with a deterministic weight gradient (parity: rl_engine/ops/embedding/
canonical_embedding.py, SM90EmbeddingOp and _deterministic_embedding_grad_weight)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops._dispatch import use_native
from rl_kernel_b200.reference.embedding.embedding import NativeEmbeddingOp


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, w, vocab_start):
        from rl_kernel_b200.backends import native as nv

        out = torch.empty(ids.numel(), w.shape[1], device=w.device, dtype=w.dtype)
        nv.embedding_fwd(ids.reshape(-1).contiguous(), w, out, vocab_start)
        ctx.save_for_backward(ids)
        ctx.meta = (w.shape, vocab_start)
        return out.view(*ids.shape, w.shape[1])

    @staticmethod
    def backward(ctx, dy):
        from rl_kernel_b200.backends import native as nv

        (ids,) = ctx.saved_tensors
        shape, vocab_start = ctx.meta
        dw = torch.zeros(shape, device=dy.device, dtype=dy.dtype)
        sid, order = torch.sort(ids.reshape(-1), stable=True)
        nv.embedding_bwd(sid.contiguous(), order.contiguous(), dy.reshape(-1, shape[1]).contiguous(), dw, vocab_start)
        return None, dw, None


def embedding(ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    if not use_native(weight):
        return NativeEmbeddingOp()(ids, weight, vocab_start)
    return _EmbeddingFn.apply(ids, weight.contiguous(), vocab_start)


class EmbeddingOp:
    backend_id = "b200"
    backward_impl = "native"

    def __call__(self, ids, weight, vocab_start: int = 0):
        return embedding(ids, weight, vocab_start)

    forward = __call__
