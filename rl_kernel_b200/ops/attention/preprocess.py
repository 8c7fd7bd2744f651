"""Attention input preprocessing: split the fused QKV activation, per-head QK-RMSNorm, RoPE —
one fused kernel on the GPU (parity: H100AttentionPreprocessor, rl_engine/ops/attention/
preprocess.py:180-345, which chains TE/own RMSNorm and the rope kernel)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.rope import qk_norm_rope
from rl_kernel_b200.reference.rope.rope import rope_tables


class AttentionPreprocessor:
    def __init__(self, num_q_heads: int, num_kv_heads: int, head_dim: int = 128, rope_theta: float = 1e6,
                 eps: float = 1e-6, max_positions: int = 40960, device="cpu"):
        self.hq, self.hkv, self.d, self.eps = num_q_heads, num_kv_heads, head_dim, eps
        self.cos, self.sin = rope_tables(head_dim, rope_theta, max_positions, device)

    def to(self, device):
        self.cos, self.sin = self.cos.to(device), self.sin.to(device)
        return self

    def __call__(self, qkv: torch.Tensor, q_norm_weight: torch.Tensor, k_norm_weight: torch.Tensor,
                 positions: torch.Tensor):
        """qkv [T, (hq+2hkv)*D] GQA-group-major -> q [T,hq,D], k [T,hkv,D], v [T,hkv,D]."""
        if self.cos.device != qkv.device:
            self.to(qkv.device)
        q, k, v = qk_norm_rope(qkv, q_norm_weight, k_norm_weight, self.cos, self.sin, positions, hq=self.hq,
                               hkv=self.hkv, eps=self.eps)
        T = qkv.shape[0]
        return q.view(T, self.hq, self.d), k.view(T, self.hkv, self.d), v.view(T, self.hkv, self.d)
