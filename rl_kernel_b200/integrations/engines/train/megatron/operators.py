"""Operator objects for the Megatron binding (parity: rl_engine/integrations/engines/train/megatron/
operators.py:102-665).

``MegatronAttentionOperator`` takes core-attention inputs in Megatron's [S_local, B, H, D] layout.
Without context parallelism the packed kernel runs.  With it every rank holds Megatron's zigzag
shard of each sequence (chunks r and 2 cp - 1 - r of 2 cp); two paths serve it:

* ``CPAttentionOp`` (NVLink, the product path): the kernel reads the other ranks' K/V blocks over
  peer memory while computing this rank's rows only; forward and backward are the single-GPU bits.
* a gather communication object (``CUDAAGRSAttentionCPCommunication`` over any transport, Gloo
  included): the strict runtime gathers Q/K/V and positions, runs the shared core on the logical
  sequence and returns the local rows -- the reference's graph, cp-fold redundant.

``MegatronFFNOperator`` / ``MegatronLogpOperator`` route the MLP and the output layer's selected
log-probs; under CP their weight gradients go through ``canonical_cp.weight_gradient``.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.distributed.algorithms import canonical_cp
from rl_kernel_b200.ops.attention.attention import causal_attention
from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn
from rl_kernel_b200.ops.logprob import linear_logp
from rl_kernel_b200.reference.attention.blockwise import zigzag_chunks


def megatron_zigzag_positions(seq_len: int, cp_size: int, cp_rank: int) -> torch.Tensor:
    """Global positions of the tokens a CP rank holds under Megatron's zigzag split."""
    if cp_size == 1:
        return torch.arange(seq_len)
    return torch.cat([torch.arange(a, b) for a, b in zigzag_chunks(seq_len, cp_size)[cp_rank]])


def packed_local_sequence_layout(cu_seqlens, cp_size: int, cp_rank: int) -> tuple[list[int], torch.Tensor]:
    """For a packed batch with global boundaries ``cu_seqlens`` (every length divisible by 2 cp): the local
    boundaries of this rank's shards and the global position of every local token."""
    cu = [int(x) for x in (cu_seqlens.tolist() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens)]
    local_cu, pos = [0], []
    for a, b in zip(cu, cu[1:]):
        n = b - a
        if n % (2 * cp_size):
            raise ValueError(f"packed sequence of {n} tokens is not divisible by 2 * cp = {2 * cp_size}")
        local_cu.append(local_cu[-1] + n // cp_size)
        pos.append(megatron_zigzag_positions(n, cp_size, cp_rank))
    return local_cu, torch.cat(pos)


class MegatronAttentionOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, cp_size: int = 1, cp_rank: int = 0, cp_collective=None, *, cp_op=None, communication=None,
                 core=None, tp_size: int = 1, tp_rank: int = 0):
        self.cp_size, self.cp_rank, self.cp_collective = cp_size, cp_rank, cp_collective
        self.cp_op, self.communication, self.core = cp_op, communication, core
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self._runtime = None

    def _native(self, device, hq: int, hkv: int, tokens: int):
        if self.cp_op is None:
            from rl_kernel_b200.ops.distributed import CPAttentionOp

            self.cp_op = CPAttentionOp(self.cp_collective, device, num_q_heads=hq, num_kv_heads=hkv,
                                       max_local_tokens=tokens, layout="zigzag")
        return self.cp_op

    def __call__(self, layer, q, k, v, cu_seqlens=None, **kw):
        """q [S_local, B, Hq, D], k / v [S_local, B, Hkv, D] -> [S_local, B, Hq * D]."""
        S, B, hq, d = q.shape
        hkv = k.shape[2]
        pack = lambda t, h: t.permute(1, 0, 2, 3).reshape(B * S, h, d)  # noqa: E731
        if self.cp_size == 1:
            cu = [i * S for i in range(B + 1)]
            o = causal_attention(pack(q, hq), pack(k, hkv), pack(v, hkv), cu)
            return o.view(B, S, hq, d).permute(1, 0, 2, 3).reshape(S, B, hq * d)
        seq_len = S * self.cp_size
        if self.communication is None and q.is_cuda and self.cp_collective is not None and hasattr(self.cp_collective, "frame_tensor"):
            op = self._native(q.device, hq, hkv, B * S)
            o, _ = op(pack(q, hq).reshape(B * S, hq * d), pack(k, hkv).reshape(B * S, hkv * d),
                      pack(v, hkv).reshape(B * S, hkv * d), nseq=B, seq_len=seq_len)
            return o.view(B, S, hq, d).permute(1, 0, 2, 3).reshape(S, B, hq * d)
        # gather path (any transport): the strict runtime on [B, H, S_local, D]
        from rl_kernel_b200.backends.cuda.attention.cp_comm import CUDAAGRSAttentionCPCommunication
        from rl_kernel_b200.backends.cuda.attention.strict_runtime import ReferenceAttentionCore, StrictCUDAAttentionRuntime
        from rl_kernel_b200.contracts.operators.attention import AttentionContract

        if self._runtime is None:
            comm = self.communication or CUDAAGRSAttentionCPCommunication(collective=self.cp_collective)
            core = self.core or (None if q.is_cuda else ReferenceAttentionCore())
            self._runtime = StrictCUDAAttentionRuntime(core=core, communication=comm)
        contract = AttentionContract.for_layout(hq * self.tp_size, hkv * self.tp_size, head_dim=d, seq_len=seq_len,
                                                batch_size=B, tp_rank=self.tp_rank, tp_world_size=self.tp_size,
                                                cp_rank=self.cp_rank, cp_world_size=self.cp_size, layout="zigzag")
        pos = megatron_zigzag_positions(seq_len, self.cp_size, self.cp_rank).to(q.device).expand(B, S)
        res = self._runtime.forward_with_lse(q.permute(1, 2, 0, 3), k.permute(1, 2, 0, 3), v.permute(1, 2, 0, 3),
                                             contract=contract, causal=True, scale=None, cp_world_size=self.cp_size,
                                             query_position_ids=pos, key_position_ids=pos)
        return res.out.permute(2, 0, 1, 3).reshape(S, B, hq * d)


class _CanonicalLinear(torch.autograd.Function):
    """y = x W^T with the weight gradient in logical token order under the active CP layout."""

    @staticmethod
    def forward(ctx, x, weight, nchunks):
        from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_fwd

        ctx.save_for_backward(x, weight)
        ctx.layout = canonical_cp.current_layout()
        return det_gemm_fwd(x, weight, nchunks=nchunks)

    @staticmethod
    def backward(ctx, dy):
        from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_da

        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = det_gemm_da(dy, w) if ctx.needs_input_grad[0] else None
        dw = canonical_cp.weight_gradient(x, dy, ctx.layout) if ctx.needs_input_grad[1] else None
        return dx, dw, None


class MegatronFFNOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, canonical_tp: int = 8, tp_size: int = 1, collective=None, sequence_parallel: bool = False):
        self.canonical_tp, self.tp_size, self.collective = canonical_tp, tp_size, collective
        self.sequence_parallel = sequence_parallel

    def __call__(self, layer, x):
        if canonical_cp.current_layout() is not None and torch.is_grad_enabled():
            # context-parallel training: the same three GEMMs with canonical weight gradients
            from rl_kernel_b200.ops.activation import swiglu_packed
            from rl_kernel_b200.ops.attention.projection import _TPAllReduce, _TPCopy

            nchunks = self.canonical_tp // self.tp_size
            coll = self.collective if self.tp_size > 1 else None
            lead = x.shape[:-1]
            gu = _CanonicalLinear.apply(_TPCopy.apply(x.reshape(-1, x.shape[-1]), coll), layer.rlk_w_gu, 1)
            act = swiglu_packed(gu, layer.rlk_w_down.shape[1] // nchunks)
            y = _TPAllReduce.apply(_CanonicalLinear.apply(act, layer.rlk_w_down, nchunks), coll)
            return y.reshape(*lead, y.shape[-1])
        return qwen3_ffn(x, layer.rlk_w_gu, layer.rlk_w_down, canonical_tp=self.canonical_tp, tp_size=self.tp_size,
                         collective=self.collective, sequence_parallel=self.sequence_parallel)


class MegatronLogpOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, temperature: float = 1.0):
        self.temperature = temperature

    def __call__(self, layer, hidden, targets, min_keep=None):
        return linear_logp(hidden, layer.weight, targets, self.temperature, min_keep=min_keep)
