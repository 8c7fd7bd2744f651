"""RMSNorm entry point with native forward and backward (parity: rl_engine/ops/norm/
canonical_rmsnorm.py and RMSNormCudaOp, rl_engine/backends/cuda/norm/rmsnorm.py:97)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops._dispatch import use_native
from rl_kernel_b200.reference.norm.rms_norm import rms_norm_reference


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        from rl_kernel_b200.backends import native as nv

        y = torch.empty_like(x)
        nv.rmsnorm_fwd(x, w, y, eps)
        ctx.save_for_backward(x, w)
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, dy):
        from rl_kernel_b200.backends import native as nv

        x, w = ctx.saved_tensors
        rows, H = x.shape
        dx = torch.empty_like(x)
        dw = torch.zeros_like(w)
        scratch = torch.empty(nv.rmsnorm_bwd_scratch_elems(rows, H), device=x.device, dtype=torch.float32)
        nv.rmsnorm_bwd(x, w, dy.contiguous(), dx, scratch, ctx.eps, dw_bf16=dw)
        return dx, dw, None


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last dimension; differentiable."""
    if not use_native(x, w):
        return rms_norm_reference(x, w, eps)
    lead = x.shape[:-1]
    return _RMSNormFn.apply(x.reshape(-1, x.shape[-1]).contiguous(), w.contiguous(), eps).reshape(*lead, x.shape[-1])


class RMSNormOp:
    backend_id = "b200"
    backward_impl = "native"

    def __init__(self, eps: float = 1e-6):
        self.eps = eps

    def __call__(self, x, w):
        return rms_norm(x, w, self.eps)

    forward = __call__

    def forward_fp32(self, x, w):
        return rms_norm_reference(x.float(), w.float(), self.eps)
