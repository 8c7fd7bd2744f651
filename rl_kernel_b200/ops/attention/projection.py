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


class _SPAllGather(torch.autograd.Function):
    """Sequence parallelism, entering a column-parallel GEMM.  Forward: rank-ordered all-gather of the token
    rows [T / tp, H] -> [T, H]; backward: fixed-tree reduce-scatter of the partial input gradients, which is
    the all-reduce of ``_TPCopy`` with every rank keeping only its rows."""

    @staticmethod
    def forward(ctx, x, collective):
        ctx.collective = collective
        if collective is None:
            return x
        return collective.all_gather(x.contiguous()).reshape(-1, *x.shape[1:])

    @staticmethod
    def backward(ctx, g):
        c = ctx.collective
        return (c.reduce_scatter(g.contiguous()) if c is not None else g), None


class _SPReduceScatter(torch.autograd.Function):
    """Sequence parallelism, leaving a row-parallel GEMM.  Forward: fixed-tree reduce-scatter of the partial
    outputs (each rank keeps its [T / tp, H] rows of the sum ``_TPAllReduce`` would give); backward: all-gather."""

    @staticmethod
    def forward(ctx, x, collective):
        ctx.collective = collective
        return collective.reduce_scatter(x.contiguous()) if collective is not None else x

    @staticmethod
    def backward(ctx, g):
        c = ctx.collective
        return (c.all_gather(g.contiguous()).reshape(-1, *g.shape[1:]) if c is not None else g), None


class _SPGemmReduceScatter(torch.autograd.Function):
    """Row-parallel GEMM and its reduce-scatter as ONE kernel (``gemm_reduce_scatter`` of the symmetric-memory
    collective): a rank pulls and reduces only the 128-row tiles of its own token rows from inside the GEMM epilogue.
    Backward is that of ``_SPReduceScatter`` after ``det_gemm_linear``: all-gather dy, then the two gradient GEMMs."""

    @staticmethod
    def forward(ctx, x, w, nchunks, collective):
        ctx.save_for_backward(x, w)
        ctx.nchunks, ctx.collective = nchunks, collective
        out = torch.empty(x.shape[0] // collective.world, w.shape[0], device=x.device, dtype=x.dtype)
        return collective.gemm_reduce_scatter(x.contiguous(), w.contiguous(), out, nchunks)

    @staticmethod
    def backward(ctx, g):
        from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_da, det_gemm_db

        x, w = ctx.saved_tensors
        dy = ctx.collective.all_gather(g.contiguous()).reshape(-1, g.shape[-1])
        dx = det_gemm_da(dy, w, nchunks=1) if ctx.needs_input_grad[0] else None
        dw = det_gemm_db(dy, x) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def sp_row_parallel_linear(x: torch.Tensor, w: torch.Tensor, nchunks: int, collective, *, fused: bool | None = None) -> torch.Tensor:
    """Sequence-parallel exit of a row-parallel projection: ``reduce_scatter(x @ w^T)`` over token rows.  ``fused``
    (default: whenever the collective and the shape allow) runs GEMM and reduce-scatter as one kernel; both forms give
    the same bits."""
    can = (hasattr(collective, "gemm_reduce_scatter") and x.is_cuda and x.dtype == torch.bfloat16
           and x.shape[0] % (128 * collective.world) == 0)
    if fused is None:
        fused = can
    if fused:
        if not can:
            raise ValueError("the fused GEMM + reduce-scatter needs the symmetric-memory collective, bf16 CUDA operands and "
                             "a token count that is a multiple of 128 x tp")
        return _SPGemmReduceScatter.apply(x, w, nchunks, collective)
    return _SPReduceScatter.apply(det_gemm_linear(x, w, nchunks), collective)


# Identity of the projections around attention, as reported to the rollout / training binding.
PROJECTION_POLICY_ID = "rl_kernel_b200.attention_projection.canonical_k_chunk_tree.v1"
DETERMINISTIC_PROJECTION_BACKEND_ID = "rl_kernel_b200.det_gemm.tcgen05"
REFERENCE_PROJECTION_BACKEND_ID = "rl_kernel_b200.reference.det_gemm"
QKV_COLLECTIVE_CONTRACT = {"tp_forward": "none", "tp_backward_dgrad": "fixed_tree_all_reduce", "sp_forward": "rank_order_all_gather",
                           "sp_backward": "fixed_tree_reduce_scatter"}
O_PROJ_COLLECTIVE_CONTRACT = {"tp_forward": "fixed_tree_all_reduce", "tp_backward_dgrad": "none",
                              "sp_forward": "fixed_tree_reduce_scatter", "sp_backward": "rank_order_all_gather"}


class AttentionProjectionOp:
    """``sequence_parallel``: activations outside the projections are sharded by token rows over the TP group
    (all-gather before the QKV GEMM, reduce-scatter after the output GEMM; parity: the SP branches of
    rl_engine/ops/attention/projection.py:35-130).  The sums are the same trees as without it, so the bits of
    every token row are unchanged."""

    def __init__(self, canonical_tp: int = 8, tp_size: int = 1, collective=None, sequence_parallel: bool = False):
        if canonical_tp % tp_size:
            raise ValueError("tp_size must divide canonical_tp")
        if sequence_parallel and (tp_size == 1 or collective is None):
            raise ValueError("sequence parallelism needs a tensor-parallel group")
        self.nchunks = canonical_tp // tp_size
        self.collective = collective if tp_size > 1 else None
        self.sequence_parallel = sequence_parallel

    def qkv(self, hidden: torch.Tensor, w_qkv_local: torch.Tensor) -> torch.Tensor:
        enter = _SPAllGather if self.sequence_parallel else _TPCopy
        return det_gemm_linear(enter.apply(hidden, self.collective), w_qkv_local)

    def output(self, attn_local: torch.Tensor, w_o_local: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            return sp_row_parallel_linear(attn_local.reshape(-1, attn_local.shape[-1]), w_o_local, self.nchunks, self.collective)
        return _TPAllReduce.apply(det_gemm_linear(attn_local, w_o_local, self.nchunks), self.collective)

    def runtime_readback(self, *, device_type: str = "cuda") -> dict:
        """Plans of the two projections (name -> facts) for the rollout / training binding."""
        backend = DETERMINISTIC_PROJECTION_BACKEND_ID if device_type == "cuda" else REFERENCE_PROJECTION_BACKEND_ID
        mode = "sp" if self.sequence_parallel else "tp"
        tp = 1 if self.collective is None else int(getattr(self.collective, "world", 1))
        common = {"backend": backend, "policy_id": PROJECTION_POLICY_ID, "fallback": False, "split_k": False, "k_order": "ascending",
                  "acc_dtype": "fp32", "tp_world_size": tp, "sequence_parallel": self.sequence_parallel}
        return {"qkv": {**common, "canonical_k_chunks": 1, "forward_collective": QKV_COLLECTIVE_CONTRACT[f"{mode}_forward"] if tp > 1 else "none"},
                "o_proj": {**common, "canonical_k_chunks": self.nchunks * tp, "local_k_chunks": self.nchunks,
                           "forward_collective": O_PROJ_COLLECTIVE_CONTRACT[f"{mode}_forward"] if tp > 1 else "none"}}
