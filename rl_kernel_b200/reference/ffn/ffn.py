"""Qwen3 SwiGLU FFN reference with the canonical tensor-parallel tree: the down projection's K
dimension is cut into ``canonical_tp`` chunks combined by a balanced tree, so splitting the chunks
over TP ranks and finishing the tree in the collective reproduces the single-rank bits
(parity: rl_engine/reference/ffn/ffn.py and the canonical-TP scheme of
rl_engine/backends/cuda/ffn/ffn.py:338-368)."""
from __future__ import annotations

import torch

from rl_kernel_b200.reference.activation.swiglu import swiglu_reference
from rl_kernel_b200.reference.gemm.det_gemm import det_gemm_reference, tree_reduce


def qwen3_ffn_reference(x, w_gate, w_up, w_down, *, canonical_tp: int = 8, tp: int = 1):
    """Full-weight inputs; ``tp`` simulates the physical split in one process."""
    inter = w_gate.shape[0]
    per = inter // tp
    chunks_per_rank = canonical_tp // tp
    partials = []
    for r in range(tp):
        sl = slice(r * per, (r + 1) * per)
        act = swiglu_reference(det_gemm_reference(x, w_gate[sl]), det_gemm_reference(x, w_up[sl]))
        partials.append(det_gemm_reference(act, w_down[:, sl], nchunks=chunks_per_rank))
    return tree_reduce(partials, x.dtype) if tp > 1 else partials[0]


class NativeQwen3FFNOp:
    def __init__(self, canonical_tp: int = 8):
        self.canonical_tp = canonical_tp

    def __call__(self, x, w_gate, w_up, w_down, tp: int = 1):
        return qwen3_ffn_reference(x, w_gate, w_up, w_down, canonical_tp=self.canonical_tp, tp=tp)

    forward = __call__
