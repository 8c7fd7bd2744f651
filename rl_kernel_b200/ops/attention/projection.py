"""Tensor-parallel attention projections: column-parallel QKV and row-parallel output projection
with the canonical chunk tree finished by the fixed-order collective (parity:
AttentionProjectionOp, rl_engine/ops/attention/projection.py:138 and the Megatron-side
_CanonicalColumnProjection / _DeterministicTPOutputProjection)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_linear


class _TPAllReduce(torch.autograd.Function):
    """Forward: fixed-tree all-reduce; backward: identity (the gradient is replicated)."""

    @staticmethod
    def forward(ctx, x, collective):
        return collective.all_reduce(x.contiguous()) if collective is not None else x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _TPCopy(torch.autograd.Function):
    """Forward: identity; backward: fixed-tree all-reduce of the partial input gradients."""

    @staticmethod
    def forward(ctx, x, collective):
        ctx.collective = collective
        return x

    @staticmethod
    def backward(ctx, g):
        c = ctx.collective
        return (c.all_reduce(g.contiguous()) if c is not None else g), None


class AttentionProjectionOp:
    def __init__(self, canonical_tp: int = 8, tp_size: int = 1, collective=None):
        if canonical_tp % tp_size:
            raise ValueError("tp_size must divide canonical_tp")
        self.nchunks = canonical_tp // tp_size
        self.collective = collective if tp_size > 1 else None

    def qkv(self, hidden: torch.Tensor, w_qkv_local: torch.Tensor) -> torch.Tensor:
        return det_gemm_linear(_TPCopy.apply(hidden, self.collective), w_qkv_local)

    def output(self, attn_local: torch.Tensor, w_o_local: torch.Tensor) -> torch.Tensor:
        partial = det_gemm_linear(attn_local, w_o_local, self.nchunks)
        return _TPAllReduce.apply(partial, self.collective)
