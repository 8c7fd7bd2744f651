"""Qwen3 SwiGLU FFN with tensor parallelism and the canonical down-projection tree (parity:
qwen3_ffn / Qwen3FFNOp, rl_engine/ops/ffn/qwen3.py:10-25 and rl_engine/backends/cuda/ffn/ffn.py:
211-999).  Weights are in the engine layout: ``w_gu`` [2*I_local, H] with gate/up interleaved per
canonical shard, ``w_down`` [H, I_local]."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.activation import swiglu_packed
from rl_kernel_b200.ops.attention.projection import _TPAllReduce, _TPCopy
from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_linear


def qwen3_ffn(x: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, *, canonical_tp: int = 8, tp_size: int = 1,
              collective=None) -> torch.Tensor:
    nchunks = canonical_tp // tp_size
    blk = w_down.shape[1] // nchunks          # columns of one canonical shard
    coll = collective if tp_size > 1 else None
    gu = det_gemm_linear(_TPCopy.apply(x, coll), w_gu)
    act = swiglu_packed(gu, blk)
    return _TPAllReduce.apply(det_gemm_linear(act, w_down, nchunks), coll)


class Qwen3FFNOp:
    backend_id = "b200-tcgen05"
    backward_impl = "native"

    def __init__(self, canonical_tp: int = 8, tp_size: int = 1, collective=None):
        self.canonical_tp, self.tp_size, self.collective = canonical_tp, tp_size, collective

    def __call__(self, x, w_gu, w_down):
        return qwen3_ffn(x, w_gu, w_down, canonical_tp=self.canonical_tp, tp_size=self.tp_size,
                         collective=self.collective)

    forward = __call__

    @torch.no_grad()
    def packed_inference(self, x, w_gu, w_down):
        return self(x, w_gu, w_down)
