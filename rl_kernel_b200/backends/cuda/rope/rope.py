"""RoPE device operator (parity: RoPESM90Op, rl_engine/backends/cuda/rope/rope.py:98-160).

``op(x [..., S, D], positions [S] | [B, S], theta=1e6)``, differentiable in ``x``; the rotation
runs in ``rlk_rope`` (csrc/rope/rope.cu) from the shared fp32 angle tables and the backward is the
same kernel with the angle negated.
"""
from __future__ import annotations

from torch import Tensor

from rl_kernel_b200.ops.rope import rope


class RoPESM100Op:
    op_class = "elementwise"
    backend_id = "b200"
    backward_impl = "native"

    def __init__(self) -> None:
        pass

    def forward(self, x: Tensor, positions: Tensor, *, theta: float = 1_000_000.0) -> Tensor:
        if x.device.type != "cuda":
            raise RuntimeError(f"{type(self).__name__} requires a CUDA tensor, got device '{x.device}'.")
        return rope(x, positions, theta=theta)

    __call__ = forward

    def forward_fp32(self, x: Tensor, positions: Tensor, *, theta: float = 1_000_000.0) -> Tensor:
        return rope(x, positions, theta=theta, out_fp32=True)


RoPESM90Op = RoPESM100Op
