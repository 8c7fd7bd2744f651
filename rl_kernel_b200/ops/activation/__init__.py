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


class _SwiGLUSplitFn(torch.autograd.Function):
    """silu(gate) * up with gate and up read where they are (no packed copy); both gradients from one kernel."""

    @staticmethod
    def forward(ctx, gate, up):
        from rl_kernel_b200.backends import native as nv

        out = torch.empty(gate.shape, device=gate.device, dtype=gate.dtype)
        nv.swiglu_split_fwd(gate, up, out)
        ctx.save_for_backward(gate, up)
        return out

    @staticmethod
    def backward(ctx, dout):
        from rl_kernel_b200.backends import native as nv

        gate, up = ctx.saved_tensors
        dgate, dup = torch.empty(gate.shape, device=gate.device, dtype=gate.dtype), torch.empty(up.shape, device=up.device, dtype=up.dtype)
        nv.swiglu_split_bwd(gate, up, _rows16(dout), dgate, dup)
        return dgate, dup


def _rows16(t: torch.Tensor) -> torch.Tensor:
    """``t`` [rows, I] as the kernels want it: unit inner stride, row stride a multiple of 8 elements, 16-byte aligned."""
    ok = t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    if not use_native(gate, up):
        return swiglu_reference(gate, up)
    if gate.shape != up.shape:
        raise ValueError(f"swiglu: gate {tuple(gate.shape)} and up {tuple(up.shape)} differ")
    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16 or gate.shape[-1] % 8:
        return swiglu_packed(torch.cat([gate, up], dim=-1))
    lead, I = gate.shape[:-1], gate.shape[-1]
    return _SwiGLUSplitFn.apply(_rows16(gate.reshape(-1, I)), _rows16(up.reshape(-1, I))).reshape(*lead, I)


class SwiGLUOp:
    backend_id = "b200"

    def __call__(self, gate, up):
        return swiglu(gate, up)

    forward = __call__
