"""LM head as the batch-invariant GEMM (parity: rl_engine/ops/embedding/canonical_lm_head.py; the
reference's one-CTA-per-logit SM90LMHeadOp is replaced by the tcgen05 GEMM whose rows are
independent by construction)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_fwd, det_gemm_linear


def lm_head_logits(hidden: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return det_gemm_linear(hidden, weight)


class LMHeadOp:
    backend_id = "b200"

    def __call__(self, hidden, weight, bias=None):
        y = det_gemm_linear(hidden, weight)
        return y if bias is None else y + bias

    forward = __call__

    def forward_fp32(self, hidden, weight, bias=None):
        y = det_gemm_fwd(hidden.reshape(-1, hidden.shape[-1]), weight, out_dtype=torch.float32)
        y = y.reshape(*hidden.shape[:-1], weight.shape[0])
        return y if bias is None else y + bias.float()
