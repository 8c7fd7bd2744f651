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


_TABLES: dict = {}


def _tables_for(head_dim: int, theta: float, max_pos: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables [max_pos, head_dim/2], cached per (head_dim, theta, device) and grown in powers of two."""
    key = (int(head_dim), float(theta), str(device))
    have = _TABLES.get(key)
    if have is None or have[0].shape[0] < max_pos:
        n = 4096
        while n < max_pos:
            n *= 2
        cos, sin = rope_tables(head_dim, theta, n, device)
        have = (cos.contiguous(), sin.contiguous())
        _TABLES[key] = have
    return have


class _RopeFn(torch.autograd.Function):
    """y = rotate(x, pos); dx = rotate(dy, -pos) through the same kernel."""

    @staticmethod
    def forward(ctx, x2, pos, cos, sin, heads, d):
        from rl_kernel_b200.backends import native as nv

        ctx.save_for_backward(pos, cos, sin)
        ctx.meta = (heads, d)
        return nv.rope(x2, pos, cos, sin, torch.empty_like(x2), heads=heads, head_dim=d)

    @staticmethod
    def backward(ctx, dy):
        from rl_kernel_b200.backends import native as nv

        pos, cos, sin = ctx.saved_tensors
        heads, d = ctx.meta
        dy = dy.contiguous()
        return nv.rope(dy, pos, cos, sin, torch.empty_like(dy), heads=heads, head_dim=d, inverse=True), None, None, None, None, None


def rope(x: torch.Tensor, positions: torch.Tensor, *, theta: float = 1_000_000.0, out_fp32: bool = False,
         max_position: int | None = None) -> torch.Tensor:
    """NeoX RoPE of ``x`` [..., S, D] at ``positions`` [S] or [B, S] (x then is [B, ..., S, D]); differentiable
    in ``x``.  Angles come from the shared fp32 table, the math is fp32 and the result is rounded once
    (``out_fp32`` keeps it in fp32).  ``max_position`` (an upper bound on the positions, exclusive) saves the
    device-to-host read that sizes the table otherwise.  A head-major view of token-major storage
    (``x.transpose(-3, -2)`` contiguous, the layout a QKV projection leaves) is rotated in place of a copy: the
    kernel walks the token rows and the result has the strides of ``x``.
    Parity: RoPESM90Op / NativeRoPEOp.forward(_fp32)."""
    D = x.shape[-1]
    S = x.shape[-2]
    pos = positions.to(x.device)
    if pos.shape[-1] != S:
        raise ValueError(f"positions {tuple(pos.shape)} do not match the sequence axis {S} of x")
    if pos.dim() == 2 and (x.dim() < 3 or x.shape[0] != pos.shape[0]):
        raise ValueError("positions [B, S] need x [B, ..., S, D]")
    max_pos = int(max_position) if max_position is not None else (int(pos.max().item()) + 1 if pos.numel() else 1)
    cos, sin = _tables_for(D, theta, max_pos, x.device)
    if not use_native(x):
        xf = x.float()
        half = D // 2
        shape = [1] * (x.dim() - 2) + [S, half]
        if pos.dim() == 2:
            shape[0] = pos.shape[0]
        c, s = cos[pos.long()].view(shape), sin[pos.long()].view(shape)
        a, b = xf[..., :half], xf[..., half:]
        y = torch.cat([a * c - b * s, b * c + a * s], dim=-1)
        return y if out_fp32 else y.to(x.dtype)
    xin = x.float() if (out_fp32 or x.dtype not in (torch.bfloat16, torch.float32)) else x
    p32 = pos.to(torch.int32)
    if xin.dim() >= 3 and xin.shape[-3] > 1 and not xin.is_contiguous() and xin.transpose(-3, -2).is_contiguous():
        # [..., H, S, D] view of [..., S, H, D] storage: rows are tokens, the heads of a token are adjacent
        xt = xin.transpose(-3, -2)
        H, lead = xt.shape[-2], xt.shape[:-2]              # lead = [..., S]
        prow = p32.expand(lead) if pos.dim() == 1 else p32.view(pos.shape[0], *([1] * (len(lead) - 2)), S).expand(lead)
        y = _RopeFn.apply(xt.reshape(-1, H * D), prow.reshape(-1).contiguous(), cos, sin, H, D).view(xt.shape).transpose(-3, -2)
    else:
        lead = xin.shape[:-1]                              # [..., S]
        prow = p32.expand(lead) if pos.dim() == 1 else p32.view(pos.shape[0], *([1] * (xin.dim() - 3)), S).expand(lead)
        y = _RopeFn.apply(xin.reshape(-1, D).contiguous(), prow.reshape(-1).contiguous(), cos, sin, 1, D).view(xin.shape)
    return y if (out_fp32 or y.dtype == x.dtype) else y.to(x.dtype)


class RoPEOp:
    """Registry object ``rope`` with the reference's call shape ``op(x, positions, theta=...)``."""
    backend_id = "b200"
    backward_impl = "native"
    op_class = "elementwise"

    def __call__(self, x, positions, *, theta: float = 1_000_000.0):
        return rope(x, positions, theta=theta)

    forward = __call__

    def forward_fp32(self, x, positions, *, theta: float = 1_000_000.0):
        return rope(x, positions, theta=theta, out_fp32=True)
