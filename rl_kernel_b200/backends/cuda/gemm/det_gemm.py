"""Deterministic GEMM device operator (parity: rl_engine/backends/cuda/gemm/det_gemm.py:34-406).

One backend exists here: the tcgen05 kernel family of csrc/gemm/det_gemm_sm100.cu.  Every output
element is one fp32 TMEM accumulation over K in ascending 16-wide steps (or a fixed tree over
canonical K chunks), whatever the tile shape, the row count or the neighbours of the row, so the
reference's choice between its SM90 kernel and a pinned no-split-K cuBLASLt call has no
counterpart: ``det_gemm_backend()`` always answers ``"sm100_tcgen05"`` and there is never a
fallback reason.

``DetGemmOp()(a, b)`` takes ``b`` as [K, N] (the reference's operand order) and is differentiable;
``DetGemmOp().linear(x, w)`` takes an nn.Linear-style [N, K] weight without transposing it.
"""
from __future__ import annotations

from typing import Callable

import torch

from rl_kernel_b200.ops.autograd.backward_runtime import record_backward
from rl_kernel_b200.ops.gemm.det_gemm import _DetLinearFn, det_gemm_da, det_gemm_db, det_gemm_fwd
from rl_kernel_b200.runtime.policy import route_report, route_report_enabled

_BACKEND = "sm100_tcgen05"
_ROUTE_REPORTED = False


def det_gemm_backend() -> str:
    return _BACKEND


def det_gemm_fallback_reason() -> str | None:
    return None


def det_gemm_backend_id() -> str:
    return "rlkernel.det_gemm.sm100_tcgen05.v1"


def _report_route_once() -> None:
    global _ROUTE_REPORTED
    if _ROUTE_REPORTED or not route_report_enabled():
        return
    _ROUTE_REPORTED = True
    route_report("gemm", requested=_BACKEND, actual=det_gemm_backend_id(), fallback=False)


def _need_cuda_bf16(*ts: torch.Tensor) -> None:
    for t in ts:
        if t.dtype != torch.bfloat16:
            raise TypeError("BF16 only")
        if not t.is_cuda:
            raise RuntimeError("Inputs must be on CUDA device")


def det_gemm_linear(a: torch.Tensor, weight: torch.Tensor, *,
                    native_op: Callable[[torch.Tensor, torch.Tensor], torch.Tensor] | None = None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """``a [M, K] @ weight[N, K]^T`` (inference form; ``out`` receives the result in place)."""
    _report_route_once()
    if native_op is not None:
        return native_op(a, weight)
    return det_gemm_fwd(a, weight, out=out)


def det_gemm_linear_input_gradient(grad_output: torch.Tensor, weight: torch.Tensor, *,
                                   native_op: Callable | None = None) -> torch.Tensor:
    """``dX = dY @ weight`` (weight [N, K] read as the MN-major B operand; no transpose is made)."""
    _report_route_once()
    if native_op is not None:
        return native_op(grad_output, weight)
    return det_gemm_da(grad_output.contiguous(), weight)


def det_gemm_linear_weight_gradient(a: torch.Tensor, grad_output: torch.Tensor, *,
                                    native_op: Callable | None = None) -> torch.Tensor:
    """``dWeight [N, K] = dY^T @ X`` with the rows (tokens) reduced in ascending order."""
    _report_route_once()
    if native_op is not None:
        return native_op(a, grad_output)
    return det_gemm_db(grad_output.contiguous(), a.contiguous())


class _DetGemmFn(torch.autograd.Function):
    """c = a [M, K] @ b [K, N]; da = dc @ b^T and db = a^T @ dc through the same kernel family."""

    @staticmethod
    def forward(ctx, a, b, output_fp32=False):
        from rl_kernel_b200.backends import native as nv

        ctx.save_for_backward(a, b)
        M, K = a.shape
        N = b.shape[1]
        out = torch.empty(M, N, device=a.device, dtype=torch.float32 if output_fp32 else torch.bfloat16)
        return nv.det_gemm(a.contiguous(), b.contiguous(), out, M=M, N=N, K=K, b_mn=True)

    @staticmethod
    def backward(ctx, grad_out):
        from rl_kernel_b200.backends import native as nv

        a, b = ctx.saved_tensors
        g = grad_out.contiguous()
        if g.dtype != torch.bfloat16:
            g = g.to(torch.bfloat16)
        M, K = a.shape
        N = b.shape[1]
        da = db = None
        if ctx.needs_input_grad[0]:       # [M, K] = g [M, N] @ b[K, N]^T : b is the K-major "weight" operand
            da = nv.det_gemm(g, b.contiguous(), torch.empty(M, K, device=a.device, dtype=a.dtype), M=M, N=K, K=N)
        if ctx.needs_input_grad[1]:       # [K, N] = a[M, K]^T @ g [M, N] : both operands MN-major
            db = nv.det_gemm(a.contiguous(), g, torch.empty(K, N, device=a.device, dtype=b.dtype), M=K, N=N, K=M,
                             a_mn=True, b_mn=True)
        record_backward("det_gemm", kernel_id="rlk_det_gemm(dA)+rlk_det_gemm(dB)", impl="b200_det_gemm", family="cuda")
        return da, db, None


class DetGemmOp:
    """Batch-invariant deterministic GEMM on the 5th-generation tensor cores."""

    backend_id = "b200-tcgen05"
    backward_impl = "native"
    has_hardware_op = True

    def __init__(self):
        from rl_kernel_b200.backends import extension

        self.has_hardware_op = extension.load(required=False) is not None and torch.cuda.is_available()

    def __call__(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        _need_cuda_bf16(a, b)
        if a.device != b.device:
            raise ValueError("GEMM operands must be on the same device")
        _report_route_once()
        return _DetGemmFn.apply(a, b, False)

    forward = __call__

    def linear(self, a: torch.Tensor, weight: torch.Tensor, *, out: torch.Tensor | None = None) -> torch.Tensor:
        """Apply a native [N, K] linear weight without materialising ``weight.T``."""
        _need_cuda_bf16(a, weight)
        if out is not None:
            if torch.is_grad_enabled() and (a.requires_grad or weight.requires_grad):
                raise RuntimeError("direct-output deterministic GEMM is inference-only")
            return det_gemm_linear(a, weight, out=out)
        lead = a.shape[:-1]
        return _DetLinearFn.apply(a.reshape(-1, a.shape[-1]), weight, 1).reshape(*lead, weight.shape[0])

    def forward_fp32(self, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        _need_cuda_bf16(a, b)
        return _DetGemmFn.apply(a, b, True)

    forward_accum_fp32 = forward_fp32

    def parameter_vjp_contributions_fp32(self, *, a, b, grad_output):
        """Per-row contributions to d(b): row r gives outer(a[r], grad_output[r]) in fp32 ([rows, K, N])."""
        del b
        return {"b": a.float()[:, :, None] * grad_output.float()[:, None, :]}


def deterministic_gemm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    return _DetGemmFn.apply(a, b, False)
