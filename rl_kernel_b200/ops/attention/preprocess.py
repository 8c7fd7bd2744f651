"""Attention input preprocessing: split the fused QKV activation, per-head QK-RMSNorm, RoPE —
one fused kernel on the GPU (parity: H100AttentionPreprocessor, rl_engine/ops/attention/
preprocess.py:180-345, which chains TE/own RMSNorm and the rope kernel)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.rope import qk_norm_rope
from rl_kernel_b200.reference.rope.rope import rope_tables

# What an engine reports about the input boundary of attention (QK-RMSNorm and RoPE) and what a strict
# rollout / training pair may report.  The fused kernel and the PyTorch definition compute the same expression
# (fp32 math on bf16-rounded inputs, one rounding at the end) from the same cos / sin table, so either may serve
# both steps; an engine's own kernels may not.
PREPROCESS_POLICY_ID = "rl_kernel_b200.attention_preprocess.fp32_table_rope.v1"
FUSED_PREPROCESS_BACKEND_ID = "rl_kernel_b200.fused_qk_norm_rope"
REFERENCE_PREPROCESS_BACKEND_ID = "rl_kernel_b200.reference.qk_norm_rope"
MANDATED_ATTENTION_PREPROCESS_BACKENDS = {"qk_rmsnorm": FUSED_PREPROCESS_BACKEND_ID, "rope": FUSED_PREPROCESS_BACKEND_ID}
ALLOWED_ATTENTION_PREPROCESS_BACKENDS = {
    "qk_rmsnorm": frozenset({FUSED_PREPROCESS_BACKEND_ID, REFERENCE_PREPROCESS_BACKEND_ID, "rl_kernel_b200.rms_norm"}),
    "rope": frozenset({FUSED_PREPROCESS_BACKEND_ID, REFERENCE_PREPROCESS_BACKEND_ID, "rl_kernel_b200.rope"}),
}


class AttentionPreprocessor:
    def __init__(self, num_q_heads: int, num_kv_heads: int, head_dim: int = 128, rope_theta: float = 1e6,
                 eps: float = 1e-6, max_positions: int = 40960, device="cpu"):
        self.hq, self.hkv, self.d, self.eps = num_q_heads, num_kv_heads, head_dim, eps
        self.rope_theta, self.max_positions = float(rope_theta), int(max_positions)
        self.cos, self.sin = rope_tables(head_dim, rope_theta, max_positions, device)
        self._last_backend: str | None = None

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
        self._last_backend = FUSED_PREPROCESS_BACKEND_ID if qkv.is_cuda else REFERENCE_PREPROCESS_BACKEND_ID
        T = qkv.shape[0]
        return q.view(T, self.hq, self.d), k.view(T, self.hkv, self.d), v.view(T, self.hkv, self.d)

    def runtime_readback(self) -> dict:
        """What ran on the last call, in the shape the rollout / training binding consumes."""
        backend = self._last_backend
        return {"backends": {} if backend is None else {"qk_rmsnorm": backend, "rope": backend}, "fallback": False,
                "fallback_reason": None, "policy_id": PREPROCESS_POLICY_ID,
                "probe_id": f"theta={self.rope_theta:g};positions={self.max_positions};eps={self.eps:g};head_dim={self.d}"}
