"""Qwen3 SwiGLU FFN with tensor parallelism and the canonical down-projection tree (parity:
qwen3_ffn / Qwen3FFNOp, rl_engine/ops/ffn/qwen3.py:10-25 and rl_engine/backends/cuda/ffn/ffn.py:
211-999).  Weights are in the engine layout: ``w_gu`` [2*I_local, H] with gate/up interleaved per
canonical shard, ``w_down`` [H, I_local]."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.activation import swiglu_packed
from rl_kernel_b200.ops.attention.projection import _SPAllGather, _TPAllReduce, _TPCopy, sp_row_parallel_linear
from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_linear


def qwen3_ffn(x: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, *, canonical_tp: int = 8, tp_size: int = 1,
              collective=None, sequence_parallel: bool = False) -> torch.Tensor:
    """``sequence_parallel``: ``x`` holds this rank's token rows [T / tp, H]; they are all-gathered before the
    gate/up GEMM and the down projection's sum is reduce-scattered back to rows (reference: ffn.py:601-603,
    648-651).  Same trees, same bits per row as the all-reduce form."""
    nchunks = canonical_tp // tp_size
    blk = w_down.shape[1] // nchunks          # columns of one canonical shard
    coll = collective if tp_size > 1 else None
    if sequence_parallel and coll is None:
        raise ValueError("sequence parallelism needs a tensor-parallel group")
    enter = _SPAllGather if sequence_parallel else _TPCopy
    lead = x.shape[:-1]
    gu = det_gemm_linear(enter.apply(x.reshape(-1, x.shape[-1]), coll), w_gu)
    act = swiglu_packed(gu, blk)
    if sequence_parallel:       # GEMM + reduce-scatter in one kernel where the collective has it
        return sp_row_parallel_linear(act, w_down, nchunks, coll)
    y = _TPAllReduce.apply(det_gemm_linear(act, w_down, nchunks), coll)
    return y.reshape(*lead, y.shape[-1])


class Qwen3FFNOp:
    backend_id = "b200-tcgen05"
    backward_impl = "native"

    def __init__(self, canonical_tp: int = 8, tp_size: int = 1, collective=None, sequence_parallel: bool = False):
        self.canonical_tp, self.tp_size, self.collective = canonical_tp, tp_size, collective
        self.sequence_parallel = sequence_parallel

    def __call__(self, x, w_gu, w_down):
        return qwen3_ffn(x, w_gu, w_down, canonical_tp=self.canonical_tp, tp_size=self.tp_size,
                         collective=self.collective, sequence_parallel=self.sequence_parallel)

    forward = __call__

    @torch.no_grad()
    def packed_inference(self, x, w_gu, w_down):
        return self(x, w_gu, w_down)
