"""Raw-bit comparison of tensors.

The reference's invariance comparator is ``allclose(atol=0, rtol=0)`` after an upcast, which
treats +0/-0 as equal and leaves NaN unspecified
(docs/contracts/ws1-numerical-precision-standard.md:404-421).  The checks here compare the
stored bit patterns, so "bitwise equal" means exactly that.
"""
from __future__ import annotations

import torch

_INT_VIEW = {
    torch.float32: torch.int32,
    torch.bfloat16: torch.int16,
    torch.float16: torch.int16,
    torch.float64: torch.int64,
}


def raw_bits(t: torch.Tensor) -> torch.Tensor:
    """Reinterpret a floating tensor as the integer tensor of its bit patterns."""
    t = t.detach().contiguous()
    view = _INT_VIEW.get(t.dtype)
    return t.view(view) if view is not None else t


def bit_mismatch_count(a: torch.Tensor, b: torch.Tensor, mask: torch.Tensor | None = None) -> int:
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError(f"shape/dtype differ: {tuple(a.shape)}/{a.dtype} vs {tuple(b.shape)}/{b.dtype}")
    diff = raw_bits(a) != raw_bits(b.to(a.device))
    if mask is not None:
        diff = diff & mask.to(diff.device).bool()
    return int(diff.sum().item())


def bit_equal(a: torch.Tensor, b: torch.Tensor, mask: torch.Tensor | None = None) -> bool:
    return bit_mismatch_count(a, b, mask) == 0
