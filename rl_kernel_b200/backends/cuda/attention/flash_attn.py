"""Flash attention device operators (parity: rl_engine/backends/cuda/attention/flash_attn.py:27-663).

The reference binds FlashAttention-4 with ``num_splits=1`` as its strict production core and
flash-attn 2 as the plain operator.  Both names map to the one tcgen05 kernel here (no split-KV,
ascending 128-key blocks), so "strict" and "fast" are the same code.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from rl_kernel_b200.backends.cuda.attention.deterministic_attn import (STRICT_ATTENTION_CORE_ID,
                                                                         STRICT_ATTENTION_SCHEDULE_ID)
from rl_kernel_b200.ops.attention.attention import AttentionOp, causal_attention

STRICT_ATTENTION_PRODUCTION_CORE_ID = STRICT_ATTENTION_CORE_ID


class StrictFlashAttentionUnavailable(RuntimeError):
    """The sm_100a library is missing or the device is not a B200."""


class StrictFlashAttention4Core:
    """Strict production core over packed (varlen) or padded inputs; no split-KV, one schedule."""

    core_id = STRICT_ATTENTION_PRODUCTION_CORE_ID
    schedule = STRICT_ATTENTION_SCHEDULE_ID
    num_splits = 1

    def __init__(self, *, softmax_scale: Optional[float] = None) -> None:
        from rl_kernel_b200.runtime.registry import KernelRegistry

        ok, why = KernelRegistry.native_ready()
        if not ok:
            raise StrictFlashAttentionUnavailable(why)
        self.softmax_scale = softmax_scale

    def forward_varlen(self, q, k, v, cu_seqlens, *, return_lse: bool = False):
        """q [T, Hq, D], k/v [T, Hkv, D] packed with boundaries ``cu_seqlens``."""
        return causal_attention(q, k, v, cu_seqlens, scale=self.softmax_scale, return_lse=return_lse)

    def __call__(self, q, k, v, *, causal: bool = True, key_padding_mask=None, return_lse: bool = False):
        """Padded q [B, S, Hq, D], k/v [B, S, Hkv, D]."""
        return AttentionOp()(q, k, v, causal=causal, key_padding_mask=key_padding_mask, scale=self.softmax_scale,
                             return_lse=return_lse)


class FlashAttentionOp:
    """``op(q, k, v, dropout_p=0, softmax_scale=None, causal=False)`` on [B, S, H, D] tensors."""

    backend_id = "b200-tcgen05"
    backward_impl = "native"

    def __init__(self):
        self.op = AttentionOp()

    def __call__(self, q, k, v, dropout_p: float = 0.0, softmax_scale: Optional[float] = None, causal: bool = False):
        if dropout_p:
            raise ValueError("dropout is not part of the deterministic attention contract")
        if not causal:
            raise NotImplementedError("the deterministic kernels implement causal attention")
        scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(q.shape[-1])
        return self.op(q, k, v, causal=True, scale=scale)

    forward = __call__
