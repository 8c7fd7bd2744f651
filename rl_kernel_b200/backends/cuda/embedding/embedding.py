"""Embedding gather device operator with a deterministic weight gradient
(parity: SM90EmbeddingOp, rl_engine/backends/cuda/embedding/embedding.py:86-147).

Forward is ``rlk_embedding_fwd`` (16-byte row copies); the weight gradient sorts the token ids
(stable) and lets one warp own each vocabulary row, adding that row's occurrences in ascending
token order in fp32 (``rlk_embedding_bwd``), so it has no atomics and no dependence on the batch
layout.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.embedding.canonical_embedding import embedding


class SM100EmbeddingOp(torch.nn.Module):
    op_class = "gather"
    is_batch_invariant = True
    backward_impl = "native"
    backend_id = "b200"

    def __init__(self) -> None:
        super().__init__()

    @staticmethod
    def _can_use(token_ids: torch.Tensor, weight: torch.Tensor) -> bool:
        return bool(weight.is_cuda and token_ids.dtype in (torch.int32, torch.int64)
                    and weight.dtype in (torch.bfloat16, torch.float32) and weight.dim() == 2)

    _can_use_sm90 = _can_use

    def forward(self, token_ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        if not self._can_use(token_ids, weight):
            raise RuntimeError(f"{type(self).__name__} requires CUDA bf16 weights and integer ids; "
                               "a fallback to another implementation is forbidden")
        if weight.dtype != torch.bfloat16:
            return torch.nn.functional.embedding(token_ids.to(weight.device), weight)
        return embedding(token_ids.to(weight.device), weight)

    def forward_fp32(self, token_ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        return self.forward(token_ids, weight).float()          # a gather is exact: widening after it loses nothing


SM90EmbeddingOp = SM100EmbeddingOp
