"""SwiGLU entry point (packed gate|up layout, native forward and backward)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops._dispatch import use_native
from rl_kernel_b200.reference.activation.swiglu import swiglu_packed_reference, swiglu_reference


class _SwiGLUPackedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, blk):
        from rl_kernel_b200.backends import native as nv

        rows, two_i = gu.shape
        out = torch.empty(rows, two_i // 2, device=gu.device, dtype=gu.dtype)
        nv.swiglu_fwd(gu, out, two_i // 2, blk)
        ctx.save_for_backward(gu)
        ctx.blk = blk
        return out

    @staticmethod
    def backward(ctx, dout):
        from rl_kernel_b200.backends import native as nv

        (gu,) = ctx.saved_tensors
        dgu = torch.empty_like(gu)
        nv.swiglu_bwd(gu, dout.contiguous(), dgu, gu.shape[1] // 2, ctx.blk)
        return dgu, None


def swiglu_packed(gu: torch.Tensor, blk: int | None = None) -> torch.Tensor:
    """gu [..., 2I] with gate/up interleaved in blocks of ``blk`` columns -> silu(gate) * up [..., I]."""
    if not use_native(gu):
        lead = gu.shape[:-1]
        return swiglu_packed_reference(gu.reshape(-1, gu.shape[-1]), blk).reshape(*lead, gu.shape[-1] // 2)
    lead = gu.shape[:-1]
    return _SwiGLUPackedFn.apply(gu.reshape(-1, gu.shape[-1]).contiguous(), blk).reshape(*lead, gu.shape[-1] // 2)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if not use_native(gate, up):
        return swiglu_reference(gate, up)
    return swiglu_packed(torch.cat([gate, up], dim=-1))


class SwiGLUOp:
    backend_id = "b200"

    def __call__(self, gate, up):
        return swiglu(gate, up)

    forward = __call__
