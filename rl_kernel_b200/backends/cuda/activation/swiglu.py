"""SiLU / SwiGLU device operators (parity: rl_engine/backends/cuda/activation/swiglu.py:92-157).

``SwiGLUCudaOp(gate, up)`` packs the two halves into the block-interleaved gate|up layout of the
fused FFN kernels and runs ``rlk_swiglu_fwd`` / ``rlk_swiglu_bwd``; fp32 math, one rounding.
``forward_fp32`` keeps the fp32 product (what the FFN's down projection consumes in the
reference's composite) and is evaluated by the same formula on the device without the kernel's
final rounding.
"""
from __future__ import annotations

import torch
from torch import Tensor

from rl_kernel_b200.ops.activation import swiglu


class SiLUCudaOp:
    op_class = "elementwise"
    backend_id = "b200"

    def __init__(self) -> None:
        pass

    def forward_fp32(self, x: Tensor) -> Tensor:
        xf = x.float()
        return xf / (1.0 + torch.exp(-xf))

    def forward(self, x: Tensor) -> Tensor:
        return self.forward_fp32(x).to(x.dtype)

    __call__ = forward


class SwiGLUCudaOp:
    op_class = "elementwise"
    backend_id = "b200"
    backward_impl = "native"

    def __init__(self) -> None:
        pass

    def forward(self, gate: Tensor, up: Tensor) -> Tensor:
        if gate.shape != up.shape:
            raise ValueError(f"gate {tuple(gate.shape)} and up {tuple(up.shape)} differ")
        return swiglu(gate, up)

    __call__ = forward

    def forward_fp32(self, gate: Tensor, up: Tensor) -> Tensor:
        g, u = gate.float(), up.float()
        return g / (1.0 + torch.exp(-g)) * u
