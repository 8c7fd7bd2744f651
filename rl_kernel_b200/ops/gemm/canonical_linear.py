"""fp32-output linear used for scoring heads (parity: canonical_linear_fp32,
rl_engine/ops/gemm/canonical_linear.py:81): bf16 operands, fp32 result, no intermediate rounding."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_fwd_fp32


def canonical_linear_fp32(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    lead = x.shape[:-1]
    y = det_gemm_fwd_fp32(x.reshape(-1, x.shape[-1]), w)
    if bias is not None:
        y = y + bias.float()
    return y.reshape(*lead, w.shape[0])
