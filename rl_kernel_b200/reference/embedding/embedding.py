"""Embedding gather, its deterministic weight gradient, and the LM head
(parity: rl_engine/reference/embedding/{embedding,lm_head,matmul}.py)."""
from __future__ import annotations

import torch

from rl_kernel_b200.reference.gemm.det_gemm import det_gemm_reference


class NativeEmbeddingOp:
    def __call__(self, ids: torch.Tensor, weight: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
        local = ids - vocab_start
        ok = (local >= 0) & (local < weight.shape[0])
        out = weight[local.clamp(0, weight.shape[0] - 1)]
        return out * ok.unsqueeze(-1).to(out.dtype)

    forward = __call__


def embedding_grad_weight_reference(ids: torch.Tensor, dy: torch.Tensor, vocab: int) -> torch.Tensor:
    """dW[v] = sum of dy rows with id v, added in ascending token order in fp32."""
    dw = torch.zeros(vocab, dy.shape[1], dtype=torch.float32, device=dy.device)
    order = torch.sort(ids.reshape(-1), stable=True).indices
    for t in order.tolist():
        dw[int(ids.reshape(-1)[t])] += dy[t].float()
    return dw


class NativeLMHeadOp:
    def __call__(self, hidden, weight, bias=None):
        out = det_gemm_reference(hidden, weight)
        return out if bias is None else out + bias

    forward = __call__

    def forward_fp32(self, hidden, weight, bias=None):
        out = det_gemm_reference(hidden, weight, out_dtype=torch.float32)
        return out if bias is None else out + bias.float()
