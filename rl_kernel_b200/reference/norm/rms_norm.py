"""RMSNorm reference: y = x * rsqrt(mean(x^2) + eps) * w, all factors fp32, one rounding at the
store ("kernel order", rl_engine/reference/norm/rms_norm.py:160-171)."""
from __future__ import annotations

import torch


def rms_norm_reference(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6,
                       residual: torch.Tensor | None = None):
    if residual is not None:
        s = (x.float() + residual.float()).to(x.dtype)
    else:
        s = x
    sf = s.float()
    # row-local reduction over the last dim only: batch-invariant
    rstd = torch.rsqrt(sf.pow(2).sum(-1, keepdim=True) / sf.shape[-1] + eps)
    y = (sf * rstd * w.float()).to(x.dtype)
    return (y, s) if residual is not None else y


class NativeRMSNormOp:
    def __init__(self, eps: float = 1e-6):
        self.eps = eps

    def __call__(self, x, w, residual=None):
        return rms_norm_reference(x, w, self.eps, residual)

    forward = __call__

    def forward_fp32(self, x, w):
        return rms_norm_reference(x.float(), w.float(), self.eps)
