"""LM-head device operator (parity: SM90LMHeadOp, rl_engine/backends/cuda/embedding/lm_head.py:81-168).

The reference launches one CTA per logit so that a row's logits cannot depend on the batch.  Here
the same property comes from the GEMM contract (each output element is one ordered fp32
accumulation over K in tensor memory), so the head is the tcgen05 GEMM at full tensor throughput.
Backward uses the same kernel family; the optional bias gradient adds rows in ascending order.
"""
from __future__ import annotations

from typing import Optional

import torch

from rl_kernel_b200.ops.autograd.backward_runtime import record_backward
from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_da, det_gemm_db, det_gemm_fwd


class _LMHeadFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, bias, output_fp32):
        h2 = hidden.reshape(-1, hidden.shape[-1])
        ctx.save_for_backward(hidden, weight)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = None if bias is None else bias.dtype
        y = det_gemm_fwd(h2, weight, out_dtype=torch.float32 if output_fp32 else torch.bfloat16)
        if bias is not None:
            y = (y.float() + bias.float()).to(y.dtype)
        return y.reshape(*hidden.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad_output):
        hidden, weight = ctx.saved_tensors
        g2 = grad_output.reshape(-1, weight.shape[0]).contiguous()
        gb = g2 if g2.dtype == torch.bfloat16 else g2.to(torch.bfloat16)
        h2 = hidden.reshape(-1, hidden.shape[-1]).contiguous()
        gh = gw = gbias = None
        if ctx.needs_input_grad[0]:
            gh = det_gemm_da(gb, weight).reshape_as(hidden).to(hidden.dtype)
        if ctx.needs_input_grad[1]:
            gw = det_gemm_db(gb, h2).to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            acc = torch.zeros(g2.shape[1], device=g2.device, dtype=torch.float32)
            for r in range(g2.shape[0]):                 # ascending row order, like the reference
                acc = acc + g2[r].float()
            gbias = acc.to(ctx.bias_dtype)
        record_backward("lm_head", kernel_id="rlk_det_gemm", impl="b200_det_gemm", family="cuda")
        return gh, gw, gbias, None


class SM100LMHeadOp:
    op_class = "reduction"
    is_batch_invariant = True
    backward_impl = "b200_det_gemm"
    backend_id = "b200-tcgen05"

    def __init__(self) -> None:
        pass

    @staticmethod
    def _can_use(hidden: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> bool:
        return bool(hidden.is_cuda and weight.is_cuda and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                    and weight.dim() == 2 and hidden.shape[-1] == weight.shape[1]
                    and (bias is None or (bias.is_cuda and bias.shape == (weight.shape[0],))))

    _can_use_sm90 = _can_use

    def _check(self, hidden, weight, bias):
        if not self._can_use(hidden, weight, bias):
            raise RuntimeError(f"{type(self).__name__} requires CUDA bf16 inputs; a fallback to another implementation "
                               "is forbidden")

    def forward(self, hidden: torch.Tensor, weight: torch.Tensor, *, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        self._check(hidden, weight, bias)
        return _LMHeadFunction.apply(hidden, weight, bias, False)

    __call__ = forward

    def forward_fp32(self, hidden: torch.Tensor, weight: torch.Tensor, *, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        self._check(hidden, weight, bias)
        return _LMHeadFunction.apply(hidden, weight, bias, True)

    def parameter_vjp_contributions_fp32(self, *, hidden, weight, grad_output, bias=None):
        del weight, bias
        rows_h = hidden.reshape(-1, hidden.size(-1)).float()
        rows_g = grad_output.reshape(-1, grad_output.size(-1)).float()
        return {"weight": rows_g[:, :, None] * rows_h[:, None, :]}


SM90LMHeadOp = SM100LMHeadOp
