"""Shared dispatch helper: CUDA tensors -> native kernels (required), CPU tensors -> references."""
from __future__ import annotations

import torch

from rl_kernel_b200.backends import extension


def use_native(*tensors: torch.Tensor) -> bool:
    cuda = [t.is_cuda for t in tensors if isinstance(t, torch.Tensor)]
    if not cuda or not any(cuda):
        return False
    if not all(cuda):
        raise ValueError("all tensor arguments must live on the same kind of device")
    extension.load(required=True)   # raises with build instructions when the library is absent
    return True
