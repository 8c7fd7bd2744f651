"""RMSNorm device operator (parity: rl_engine/backends/cuda/norm/rmsnorm.py:19-116).

Forward and backward are ``rlk_rmsnorm_fwd`` / ``rlk_rmsnorm_bwd`` (one CTA per row block, fp32
row statistics, gain gradient reduced over fixed row blocks in a fixed tree), so the output of a
row never depends on the other rows of the call.  ``mask`` zeroes the rows it excludes, as the
reference's masked variant does.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.norm.canonical_rmsnorm import _RMSNormFn as RMSNormCuda
from rl_kernel_b200.ops.norm.canonical_rmsnorm import rms_norm


def rmsnorm_cuda(x, weight, eps: float = 1e-6, mask=None):
    y = rms_norm(x, weight, eps)
    if mask is not None:
        y = y * mask.to(y.dtype).reshape(*x.shape[:-1], 1)
    return y


class RMSNormCudaOp:
    op_class = "row_reduce"
    backend_id = "b200"
    backward_impl = "native"

    def forward(self, x, weight, *, eps: float = 1e-6):
        return rms_norm(x, weight, eps)

    __call__ = forward

    def forward_fp32(self, x, weight, *, eps: float = 1e-6):
        xf = x.float()
        return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()

    def parameter_vjp_contributions_fp32(self, *, x, weight, grad_output, eps: float = 1e-6):
        """Per-row contributions to d(weight): row r gives grad_output[r] * x[r] * rstd[r] (fp32)."""
        del weight
        xf = x.reshape(-1, x.shape[-1]).float()
        g = grad_output.reshape(-1, x.shape[-1]).float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return {"weight": g * xf * rstd}
