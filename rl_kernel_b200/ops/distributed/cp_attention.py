"""Context-parallel causal attention as a differentiable operator on the sm_100a kernels.

Each rank holds 1/cp of every sequence (zigzag or contiguous shards); the attention kernels fetch
the remote K/V blocks (forward, dQ) and the remote Q / dO / lse / delta blocks (dK, dV) themselves
through peer-mapped buffers, in the canonical 128-key block order, so output and gradients are
bitwise equal to the single-GPU kernels for every cp (rl_kernel_b200/distributed/cp_attention.py).
The reference computes the same by gathering Q/K/V and running the whole sequence on every rank
(rl_engine/backends/cuda/attention/cp_comm.py:444-566).
"""
from __future__ import annotations

import torch


class _CPAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, op, nseq, seq_len):
        o, lse = op.cp.forward(q, k, v, nseq, seq_len)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.op, ctx.geom = op, (nseq, seq_len)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ctx.op.cp.backward(q, k, v, o, lse, do.contiguous(), *ctx.geom)
        return dq, dk, dv, None, None, None


class CPAttentionOp:
    """``op(q, k, v, nseq=, seq_len=)`` with q [nseq * S_local, Hq * 128], k / v [nseq * S_local, Hkv * 128]
    (this rank's tokens of ``nseq`` sequences of global length ``seq_len``, in ``local_positions``
    order) -> (out, lse)."""

    backend_id = "b200-tcgen05-cp"
    schedule = "remote_kv_in_kernel_no_splitkv"

    def __init__(self, collective, device, *, num_q_heads: int, num_kv_heads: int, max_local_tokens: int,
                 layout: str = "zigzag"):
        from rl_kernel_b200.distributed.cp_attention import CPAttention

        self.cp = CPAttention(collective, torch.device(device), num_q_heads=num_q_heads, num_kv_heads=num_kv_heads,
                              max_local_tokens=max_local_tokens, layout=layout)
        self.layout = layout

    def local_positions(self, seq_len: int) -> torch.Tensor:
        return self.cp.local_positions(seq_len)

    def __call__(self, q, k, v, *, nseq: int, seq_len: int):
        return _CPAttentionFn.apply(q.contiguous(), k.contiguous(), v.contiguous(), self, nseq, seq_len)

    forward = __call__
