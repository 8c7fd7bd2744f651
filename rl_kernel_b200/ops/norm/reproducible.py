"""Partition-independent L2 norm for gradient clipping (parity: rl_engine/ops/norm/reproducible.py:
17-202, which NVRTC-compiles an integer-bin kernel from a Python string; here the kernel is part
of librlk_b200.so).

A finite bf16 value is ``mant * 2^e`` with ``mant < 2^8``; squares are summed as integers in one
64-bit bin per exponent, so the result does not depend on how the tensors are split over
parameters, blocks or ranks.  fp32 values are ``m * 2^(e-150)`` with a 24-bit integer ``m``: the
48-bit square is split into three 16-bit limbs, one bin per (exponent, limb) -- 768 bins
(``sumsq_bins_f32``), the scheme of the reference's NVRTC kernel.
"""
from __future__ import annotations

from typing import Iterable

import torch

_EXP = torch.arange(256).clamp(min=1).double()
_W = torch.pow(2.0, 2.0 * (_EXP - 134.0))
_W[255] = 0.0


def _bins_cpu(t: torch.Tensor) -> torch.Tensor:
    h = t.detach().to(torch.bfloat16).contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
    e = (h >> 7) & 0xFF
    mant = h & 0x7F
    mant = torch.where(e != 0, mant | 0x80, mant)
    sq = (mant.to(torch.int64) * mant.to(torch.int64))
    finite = e != 0xFF
    bins = torch.zeros(256, dtype=torch.int64)
    bins.index_add_(0, e[finite].reshape(-1).long(), sq[finite].reshape(-1))
    bins[255] = int((~finite).sum())
    return bins


def sumsq_bins(tensors: Iterable[torch.Tensor]) -> torch.Tensor:
    """256 int64 bins (bin 255 counts non-finite values) accumulated over all tensors."""
    total = None
    for t in tensors:
        if t.dtype != torch.bfloat16:
            raise TypeError("exact sum of squares is defined for bf16 tensors")
        if t.is_cuda:
            from rl_kernel_b200.backends import native as nv

            b = torch.zeros(256, dtype=torch.int64, device=t.device) if total is None else total
            nv.sumsq_bins(t.contiguous().view(-1), b)
            total = b
        else:
            b = _bins_cpu(t)
            total = b if total is None else total + b
    if total is None:
        total = torch.zeros(256, dtype=torch.int64)
    return total


_W32 = (torch.pow(2.0, 2.0 * (_EXP - 150.0))[:, None] * torch.tensor([1.0, 65536.0, 4294967296.0], dtype=torch.float64)[None])
_W32[255] = 0.0


def _bins_f32_cpu(t: torch.Tensor) -> torch.Tensor:
    u = t.detach().float().contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    e = (u >> 23) & 0xFF
    m = u & 0x7FFFFF
    m = torch.where(e != 0, m | 0x800000, m)
    sq = m * m
    finite = (e != 0xFF).reshape(-1)
    bins = torch.zeros(256, 3, dtype=torch.int64)
    ee = e.reshape(-1)[finite]
    sqf = sq.reshape(-1)[finite]
    for l in range(3):
        bins[:, l].index_add_(0, ee, (sqf >> (16 * l)) & (0xFFFF if l < 2 else 0xFFFFFFFF))
    bins[255, 0] = int((~finite).sum())
    return bins.reshape(-1)


def sumsq_bins_f32(tensors: Iterable[torch.Tensor]) -> torch.Tensor:
    """768 int64 bins (three limbs per exponent) accumulated over fp32 tensors; exact."""
    total = None
    for t in tensors:
        if t.dtype != torch.float32:
            raise TypeError("sumsq_bins_f32 takes fp32 tensors")
        if t.is_cuda:
            from rl_kernel_b200.backends import native as nv

            b = torch.zeros(768, dtype=torch.int64, device=t.device) if total is None else total
            nv.sumsq_bins_f32(t.contiguous().view(-1), b)
            total = b
        else:
            b = _bins_f32_cpu(t)
            total = b if total is None else total + b
    return total if total is not None else torch.zeros(768, dtype=torch.int64)


def norm_from_bins_f32(bins: torch.Tensor) -> torch.Tensor:
    w = _W32.reshape(-1).to(bins.device)
    return (bins.double() * w).sum().sqrt()


def norm_from_bins(bins: torch.Tensor) -> torch.Tensor:
    return (bins.double().cpu() * _W).sum().sqrt() if not bins.is_cuda else \
        (bins.double() * _W.to(bins.device)).sum().sqrt()


def reproducible_grad_norm(tensors: Iterable[torch.Tensor], group=None) -> torch.Tensor:
    """Exact global L2 norm; with ``group`` the integer bins are summed over ranks first."""
    tensors = list(tensors)
    fp32 = bool(tensors) and all(t.dtype == torch.float32 for t in tensors)
    bins = sumsq_bins_f32(tensors) if fp32 else sumsq_bins(tensors)
    if group is not None:
        import torch.distributed as dist

        dist.all_reduce(bins, group=group)
    return norm_from_bins_f32(bins) if fp32 else norm_from_bins(bins)


def clip_grad_norm_(parameters: Iterable[torch.nn.Parameter], max_norm: float, group=None) -> torch.Tensor:
    params = [p for p in parameters if p.grad is not None]
    total = reproducible_grad_norm([p.grad for p in params], group)
    scale = float(min(1.0, max_norm / (float(total) + 1e-6)))
    if scale < 1.0:
        for p in params:
            p.grad.mul_(scale)
    return total


_INSTALLED = False


def install() -> None:
    """Route ``torch.nn.utils.clip_grad_norm_`` through the exact norm for bf16 gradients
    (parity: reproducible.install(), rl_engine/ops/norm/reproducible.py:177)."""
    global _INSTALLED
    if _INSTALLED:
        return
    orig = torch.nn.utils.clip_grad_norm_

    def patched(parameters, max_norm, norm_type=2.0, **kw):
        ps = [parameters] if isinstance(parameters, torch.Tensor) else list(parameters)
        dts = {p.grad.dtype for p in ps if p.grad is not None}
        if norm_type == 2.0 and ps and (dts <= {torch.bfloat16} or dts <= {torch.float32}):
            return clip_grad_norm_(ps, max_norm)
        return orig(ps, max_norm, norm_type, **kw)

    torch.nn.utils.clip_grad_norm_ = patched
    _INSTALLED = True
