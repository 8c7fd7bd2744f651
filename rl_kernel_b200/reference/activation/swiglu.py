"""SiLU / SwiGLU references (parity: rl_engine/reference/activation/swiglu.py)."""
from __future__ import annotations

import torch


def swiglu_reference(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    g = gate.float()
    return (g / (1.0 + torch.exp(-g)) * up.float()).to(gate.dtype)


def swiglu_packed_reference(gu: torch.Tensor, blk: int | None = None) -> torch.Tensor:
    """gu [rows, 2I] with gate/up interleaved in blocks of ``blk`` columns (blk=I: [gate|up])."""
    rows, two_i = gu.shape
    i = two_i // 2
    blk = blk or i
    g3 = gu.reshape(rows, i // blk, 2, blk)
    return swiglu_reference(g3[:, :, 0].reshape(rows, i), g3[:, :, 1].reshape(rows, i))


class NativeSwiGLUOp:
    def __call__(self, gate, up):
        return swiglu_reference(gate, up)

    forward = __call__
