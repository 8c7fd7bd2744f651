"""NeoX (rotate-half) RoPE and the fused per-head QK-RMSNorm + RoPE reference
(parity: rl_engine/reference/rope/rope.py:9; fused form = csrc/norm/rmsnorm.cu here)."""
from __future__ import annotations

import torch


def rope_tables(head_dim: int, theta: float, max_pos: int, device="cpu"):
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv_freq[None]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def apply_rope(x: torch.Tensor, pos: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [..., T, heads, D] fp32; pos [T]."""
    half = x.shape[-1] // 2
    c = cos[pos.long()].unsqueeze(-2)
    s = sin[pos.long()].unsqueeze(-2)
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1)


def qk_norm_rope_reference(x: torch.Tensor, w: torch.Tensor, pos: torch.Tensor, cos, sin, eps: float):
    """x [T, heads, D] -> RMSNorm over D with gain w, then RoPE; fp32 math, one rounding."""
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) / xf.shape[-1] + eps) * w.float()
    return apply_rope(n, pos, cos, sin).to(x.dtype)


class NativeRoPEOp:
    def __init__(self, head_dim: int, theta: float = 1e6, max_pos: int = 4096):
        self.cos, self.sin = rope_tables(head_dim, theta, max_pos)

    def __call__(self, x, pos):
        return apply_rope(x.float(), pos, self.cos.to(x.device), self.sin.to(x.device)).to(x.dtype)

    forward = __call__
