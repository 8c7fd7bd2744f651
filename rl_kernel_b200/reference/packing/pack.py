"""Varlen packing: [B, S] padded -> [T] packed with cu_seqlens, and back
(parity: NativePackOp, rl_engine/reference/packing/pack.py:95)."""
from __future__ import annotations

import torch


def cu_seqlens_from_lengths(lengths: torch.Tensor) -> torch.Tensor:
    return torch.cat([lengths.new_zeros(1), lengths.cumsum(0)]).to(torch.int32)


class NativePackOp:
    def pack(self, x: torch.Tensor, mask: torch.Tensor):
        """x [B, S, ...], mask [B, S] (True = keep, row-major order) -> packed [T, ...], cu_seqlens."""
        m = mask.bool()
        return x[m], cu_seqlens_from_lengths(m.sum(1))

    def unpack(self, packed: torch.Tensor, mask: torch.Tensor, fill: float = 0.0) -> torch.Tensor:
        m = mask.bool()
        out = packed.new_full(m.shape + packed.shape[1:], fill)
        out[m] = packed
        return out

    __call__ = pack
