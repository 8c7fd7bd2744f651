"""RoPE / fused QK-norm+RoPE entry points."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops._dispatch import use_native
from rl_kernel_b200.reference.rope.rope import qk_norm_rope_reference, rope_tables


class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, q_w, k_w, cos, sin, pos, hq, hkv, eps):
        from rl_kernel_b200.backends import native as nv

        T = qkv.shape[0]
        q = torch.empty(T, hq * 128, device=qkv.device, dtype=qkv.dtype)
        k = torch.empty(T, hkv * 128, device=qkv.device, dtype=qkv.dtype)
        v = torch.empty(T, hkv * 128, device=qkv.device, dtype=qkv.dtype)
        nv.qk_norm_rope_fwd(qkv, q_w, k_w, cos, sin, pos, q, k, v, Hq=hq, Hkv=hkv, eps=eps)
        ctx.save_for_backward(qkv, q_w, k_w, cos, sin, pos)
        ctx.meta = (hq, hkv, eps)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        from rl_kernel_b200.backends import native as nv

        qkv, q_w, k_w, cos, sin, pos = ctx.saved_tensors
        hq, hkv, eps = ctx.meta
        T = qkv.shape[0]
        dqkv = torch.empty_like(qkv)
        dqw, dkw = torch.zeros_like(q_w), torch.zeros_like(k_w)
        scr = torch.empty(nv.qk_norm_rope_bwd_scratch_elems(T), device=qkv.device, dtype=torch.float32)
        nv.qk_norm_rope_bwd(qkv, q_w, k_w, cos, sin, pos, dq.contiguous(), dk.contiguous(), dv.contiguous(), dqkv,
                            scr, dqw, dkw, Hq=hq, Hkv=hkv, eps=eps, accumulate_dw=False)
        return dqkv, dqw, dkw, None, None, None, None, None, None


def qk_norm_rope(qkv: torch.Tensor, q_w, k_w, cos, sin, pos, *, hq: int, hkv: int, eps: float = 1e-6):
    """Fused per-head RMSNorm + NeoX RoPE over a GQA-group-major QKV activation [T, (hq+2hkv)*128].
    Returns (q [T, hq*128], k [T, hkv*128], v [T, hkv*128])."""
    if use_native(qkv):
        return _QKNormRopeFn.apply(qkv, q_w, k_w, cos, sin, pos.to(torch.int32), hq, hkv, eps)
    T, g, d = qkv.shape[0], hq // hkv, 128 if qkv.shape[1] % 128 == 0 and qkv.shape[1] // (hq + 2 * hkv) == 128 else qkv.shape[1] // (hq + 2 * hkv)
    grp = qkv.view(T, hkv, g + 2, d)
    q = qk_norm_rope_reference(grp[:, :, :g].reshape(T, hq, d), q_w, pos, cos, sin, eps).reshape(T, hq * d)
    k = qk_norm_rope_reference(grp[:, :, g], k_w, pos, cos, sin, eps).reshape(T, hkv * d)
    return q, k, grp[:, :, g + 1].reshape(T, hkv * d)


class RoPEOp:
    backend_id = "b200"

    def __init__(self, head_dim: int = 128, theta: float = 1e6, max_pos: int = 4096, device="cpu"):
        self.cos, self.sin = rope_tables(head_dim, theta, max_pos, device)

    def __call__(self, x, pos):
        from rl_kernel_b200.reference.rope.rope import apply_rope

        return apply_rope(x.float(), pos, self.cos.to(x.device), self.sin.to(x.device)).to(x.dtype)

    forward = __call__
