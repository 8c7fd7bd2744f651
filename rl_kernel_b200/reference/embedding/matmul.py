"""Plain matmul reference (parity: NativeMatmulOp, rl_engine/reference/embedding/matmul.py:10-28): one fp32
``torch.matmul`` as gold; no split-K, no blocked accumulation."""
from __future__ import annotations

import torch
from torch import Tensor


class NativeMatmulOp(torch.nn.Module):
    op_class = "reduction"

    def forward(self, a: Tensor, b: Tensor) -> Tensor:
        return self.forward_fp32(a, b).to(a.dtype)

    def forward_fp32(self, a: Tensor, b: Tensor) -> Tensor:
        return torch.matmul(a.float(), b.float())


__all__ = ["NativeMatmulOp"]
