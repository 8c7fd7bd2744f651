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
    """PyTorch NeoX RoPE with the call shape ``op(x [..., S, D], positions [S] | [B, S], theta=...)``
    (parity: NativeRoPEOp, rl_engine/reference/rope/rope.py:10).  Angles are computed in fp64 and stored
    in fp32, like every other RoPE in this package; no table is accepted or returned."""

    op_class = "elementwise"

    def __init__(self, head_dim: int | None = None, theta: float = 1_000_000.0, max_pos: int = 4096):
        self.theta = theta

    @staticmethod
    def _cos_sin(x, positions, theta):
        D, S = x.shape[-1], x.shape[-2]
        pos = positions.to(x.device).long()
        cos, sin = rope_tables(D, theta, int(pos.max().item()) + 1 if pos.numel() else 1, x.device)
        shape = [1] * (x.dim() - 2) + [S, D // 2]
        if pos.dim() == 2:
            shape[0] = pos.shape[0]
        return cos[pos].view(shape), sin[pos].view(shape)

    def forward_fp32(self, x, positions, *, theta: float | None = None):
        c, s = self._cos_sin(x, positions, self.theta if theta is None else theta)
        half = x.shape[-1] // 2
        a, b = x.float()[..., :half], x.float()[..., half:]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    def forward(self, x, positions, *, theta: float | None = None):
        return self.forward_fp32(x, positions, theta=theta).to(x.dtype)

    __call__ = forward
