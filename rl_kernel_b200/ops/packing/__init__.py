"""Varlen packing (compaction by mask, cu_seqlens) and its inverse.

On a CUDA tensor whose rows are a multiple of 16 bytes the rows move with one gather / scatter
kernel (csrc/packing/pack.cu); the order of the packed tokens is the row-major order of the kept
positions on every path, so packing never changes a reduction order downstream.
"""
from __future__ import annotations

import ctypes

import torch

from rl_kernel_b200.reference.packing.pack import NativePackOp, cu_seqlens_from_lengths  # noqa: F401


def _native_ok(x: torch.Tensor) -> bool:
    if not x.is_cuda or x.dim() < 2:
        return False
    row_bytes = x[0, 0].numel() * x.element_size() if x.dim() > 2 else x.element_size()
    return row_bytes % 16 == 0 and x.is_contiguous()


def _move(src2d: torch.Tensor, idx: torch.Tensor, dst2d: torch.Tensor, scatter: bool) -> None:
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.backends import native as nv

    row_bytes = src2d.shape[1] * src2d.element_size()
    limit = dst2d.shape[0] if scatter else src2d.shape[0]
    rc = ext.load().rlk_move_rows(ext.ptr(src2d), ctypes.c_longlong(src2d.stride(0) * src2d.element_size()), ext.ptr(idx),
                                  ext.ptr(dst2d), ctypes.c_longlong(dst2d.stride(0) * dst2d.element_size()),
                                  ctypes.c_int(idx.numel()), ctypes.c_int(row_bytes), ctypes.c_longlong(limit),
                                  ctypes.c_int(int(scatter)), ext.stream_ptr(src2d.device))
    ext.check(rc, "move_rows")
    nv._count()


class PackOp(NativePackOp):
    backend_id = "b200"

    def pack(self, x: torch.Tensor, mask: torch.Tensor):
        m = mask.bool()
        if not _native_ok(x):
            return super().pack(x, mask)
        B, S = m.shape
        idx = torch.nonzero(m.reshape(-1)).reshape(-1).contiguous()          # kept positions, row-major order
        src = x.reshape(B * S, -1)
        out = torch.empty((idx.numel(),) + tuple(x.shape[2:]), dtype=x.dtype, device=x.device)
        _move(src, idx, out.reshape(idx.numel(), -1), scatter=False)
        return out, cu_seqlens_from_lengths(m.sum(1))

    def unpack(self, packed: torch.Tensor, mask: torch.Tensor, fill: float = 0.0) -> torch.Tensor:
        m = mask.bool()
        probe = packed.reshape(packed.shape[0], -1) if packed.dim() > 1 else packed.reshape(-1, 1)
        if not (packed.is_cuda and packed.is_contiguous() and (probe.shape[1] * packed.element_size()) % 16 == 0):
            return super().unpack(packed, mask, fill)
        B, S = m.shape
        out = packed.new_full((B, S) + tuple(packed.shape[1:]), fill)
        idx = torch.nonzero(m.reshape(-1)).reshape(-1).contiguous()
        _move(probe, idx, out.reshape(B * S, -1), scatter=True)
        return out

    __call__ = pack
