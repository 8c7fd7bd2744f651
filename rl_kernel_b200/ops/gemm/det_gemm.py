"""Batch-invariant deterministic GEMM (parity: rl_engine/ops/gemm/det_gemm.py:9-31 and the
DetGemmOp/_DetLinearFn of rl_engine/backends/cuda/gemm/det_gemm.py:239-313).

``det_gemm_linear(x, w, nchunks)`` is y = x @ w^T with w stored [out, in] like nn.Linear; its
backward uses the same kernel family (dX = dY @ W through an MN-major B operand, dW = dY^T @ X
through MN-major A and B), so forward and backward are both deterministic and tile-invariant.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.ops._dispatch import use_native
from rl_kernel_b200.reference.gemm.det_gemm import det_gemm_reference


def det_gemm_fwd(a: torch.Tensor, b_t: torch.Tensor, *, nchunks: int = 1, out: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """a [M,K] @ b_t[N,K]^T ("rhs transposed": the weight layout)."""
    if not use_native(a, b_t):
        return det_gemm_reference(a, b_t, nchunks=nchunks, out_dtype=out_dtype)
    from rl_kernel_b200.backends import native as nv

    M, K = a.shape
    N = b_t.shape[0]
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=out_dtype or torch.bfloat16)
    return nv.det_gemm(a.contiguous(), b_t.contiguous(), out, M=M, N=N, K=K, nchunks=nchunks)


def det_gemm_fwd_fp32(a, b_t, *, nchunks: int = 1):
    return det_gemm_fwd(a, b_t, nchunks=nchunks, out_dtype=torch.float32)


def det_gemm(a: torch.Tensor, b: torch.Tensor, *, nchunks: int = 1) -> torch.Tensor:
    """a [M,K] @ b [K,N] (b physically [K,N])."""
    if not use_native(a, b):
        return det_gemm_reference(a, b.t(), nchunks=nchunks)
    from rl_kernel_b200.backends import native as nv

    M, K = a.shape
    N = b.shape[1]
    out = torch.empty(M, N, device=a.device, dtype=torch.bfloat16)
    return nv.det_gemm(a.contiguous(), b.contiguous(), out, M=M, N=N, K=K, b_mn=True, nchunks=nchunks)


def det_gemm_da(dy: torch.Tensor, w: torch.Tensor, *, nchunks: int = 1) -> torch.Tensor:
    """dX [M,K] = dY [M,N] @ W [N,K]."""
    if not use_native(dy, w):
        return det_gemm_reference(dy, w.t(), nchunks=nchunks)
    from rl_kernel_b200.backends import native as nv

    M, N = dy.shape
    K = w.shape[1]
    out = torch.empty(M, K, device=dy.device, dtype=torch.bfloat16)
    return nv.det_gemm(dy.contiguous(), w.contiguous(), out, M=M, N=K, K=N, b_mn=True, nchunks=nchunks)


def det_gemm_db(dy: torch.Tensor, x: torch.Tensor, *, out: torch.Tensor | None = None,
                accumulate: bool = False) -> torch.Tensor:
    """dW [N,K] = dY [T,N]^T @ X [T,K], tokens reduced in ascending order (canonical [out,in] layout)."""
    if not use_native(dy, x):
        r = det_gemm_reference(dy.t().contiguous(), x.t().contiguous())
        return r if out is None else (out.add_(r) if accumulate else out.copy_(r))
    from rl_kernel_b200.backends import native as nv

    T, N = dy.shape
    K = x.shape[1]
    if T % 8:                                   # the token contraction steps by 8 rows: zero rows add exact zeros at the end
        pad = 8 - T % 8
        dy, x, T = torch.cat([dy, dy.new_zeros(pad, N)]), torch.cat([x, x.new_zeros(pad, K)]), T + pad
    if out is None:
        out = torch.zeros(N, K, device=dy.device, dtype=torch.bfloat16)
        accumulate = False
    return nv.det_gemm(dy.contiguous(), x.contiguous(), out, M=N, N=K, K=T, a_mn=True, b_mn=True,
                       accumulate=accumulate)


class _DetLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, nchunks):
        ctx.save_for_backward(x, w)
        ctx.nchunks = nchunks
        return det_gemm_fwd(x, w, nchunks=nchunks)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = det_gemm_da(dy.contiguous(), w) if ctx.needs_input_grad[0] else None
        dw = det_gemm_db(dy.contiguous(), x) if ctx.needs_input_grad[1] else None
        return dx, dw, None


def det_gemm_linear(x: torch.Tensor, w: torch.Tensor, nchunks: int = 1) -> torch.Tensor:
    """y = x @ w^T for x [..., K]; differentiable."""
    lead = x.shape[:-1]
    y = _DetLinearFn.apply(x.reshape(-1, x.shape[-1]), w, nchunks)
    return y.reshape(*lead, w.shape[0])


class DetGemmOp:
    """Registry object for ``det_gemm`` (callable like the reference's DetGemmOp)."""
    backend_id = "b200-tcgen05"
    backward_impl = "native"

    def __call__(self, a, b):
        return det_gemm(a, b)

    forward = __call__

    def forward_rhs_transposed(self, a, b_t, nchunks: int = 1):
        return det_gemm_fwd(a, b_t, nchunks=nchunks)

    def forward_fp32(self, a, b):
        if not use_native(a, b):
            return det_gemm_reference(a, b.t(), out_dtype=torch.float32)
        from rl_kernel_b200.backends import native as nv

        out = torch.empty(a.shape[0], b.shape[1], device=a.device, dtype=torch.float32)
        return nv.det_gemm(a.contiguous(), b.contiguous(), out, M=a.shape[0], N=b.shape[1], K=a.shape[1], b_mn=True)

    def linear(self, x, w, nchunks: int = 1):
        return det_gemm_linear(x, w, nchunks)
