"""Deterministic attention device operator with the reference's [B, H, S, D] surface
(parity: rl_engine/backends/cuda/attention/deterministic_attn.py:29-360).

The reference materialises fp32 scores for a batch-invariant softmax.  Here the operator runs
the tcgen05 flash kernel whose per-row program is fixed (128-key blocks in ascending order, one
running max / sum per row, fp32 accumulators in tensor memory), which gives the same property at
tensor-core speed: a row's output depends only on that row's query and its keys.
``RLKernelDeterministicAttentionCore`` is the strict core the runtime binds: padded [B, S, H, D]
inputs with explicit positions, returning output and fp32 LSE.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from rl_kernel_b200.ops.attention.attention import AttentionOp

STRICT_ATTENTION_CORE_ID = "rlkernel.attention.b200_tcgen05.canonical_128_key_blocks.v1"
STRICT_ATTENTION_SCHEDULE_ID = "canonical_128_key_blocks_no_splitkv"


@dataclass(frozen=True)
class DeterministicAttentionCoreResult:
    out: torch.Tensor
    lse: torch.Tensor
    core_id: str = STRICT_ATTENTION_CORE_ID
    schedule: str = STRICT_ATTENTION_SCHEDULE_ID


class DeterministicAttentionOp:
    core_id = STRICT_ATTENTION_CORE_ID
    strict_schedule = STRICT_ATTENTION_SCHEDULE_ID
    backend_id = "rlkernel.b200.deterministic_attention"
    backward_impl = "native"

    def __init__(self) -> None:
        self._op = AttentionOp()

    @staticmethod
    def _validate_inputs(q, k, v, key_padding_mask) -> None:
        if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
            raise ValueError("q, k, v must be [B, H, S, D]")
        if k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[-1] != k.shape[-1]:
            raise ValueError(f"incompatible shapes q={tuple(q.shape)} k={tuple(k.shape)} v={tuple(v.shape)}")
        if q.shape[1] % k.shape[1]:
            raise ValueError("query heads must be a multiple of key/value heads (GQA)")
        if key_padding_mask is not None and key_padding_mask.shape != (k.shape[0], k.shape[2]):
            raise ValueError("key_padding_mask must be [B, S_kv]")

    def forward_with_lse(self, q, k, v, *, causal: bool = True, scale: Optional[float] = None,
                         key_padding_mask: Optional[torch.Tensor] = None):
        """(out [B, Hq, S, D], lse [B, Hq, S] fp32); differentiable in q, k, v."""
        self._validate_inputs(q, k, v, key_padding_mask)
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        o, lse = self._op(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), causal=causal,
                          key_padding_mask=key_padding_mask, scale=scale, return_lse=True)
        return o.transpose(1, 2), lse.transpose(1, 2)

    def forward(self, q, k, v, *, causal: bool = True, scale: Optional[float] = None,
                key_padding_mask: Optional[torch.Tensor] = None):
        return self.forward_with_lse(q, k, v, causal=causal, scale=scale, key_padding_mask=key_padding_mask)[0]

    __call__ = forward

    def forward_fp32(self, q, k, v, *, causal: bool = True, scale: Optional[float] = None,
                     key_padding_mask: Optional[torch.Tensor] = None):
        """The same program with the output widened; the kernel's one rounding (bf16 out) is kept, as
        the production path has it."""
        return self.forward(q, k, v, causal=causal, scale=scale, key_padding_mask=key_padding_mask).float()


class RLKernelDeterministicAttentionCore:
    """Strict attention core: q [B, Sq, Hq, D], k/v [B, Skv, Hkv, D], explicit query positions."""

    core_id = STRICT_ATTENTION_CORE_ID
    schedule = STRICT_ATTENTION_SCHEDULE_ID

    def __init__(self, *, scale: Optional[float] = None, causal: bool = True) -> None:
        if not causal:
            raise ValueError("the strict core is causal")
        self.scale = scale
        self._op = AttentionOp()

    @staticmethod
    def _validate_positions(q, k, q_positions) -> None:
        if q_positions is None:
            return
        if q_positions.shape != q.shape[:2]:
            raise ValueError("q_positions must be [B, Sq]")
        if q.shape[1] == k.shape[1]:
            want = torch.arange(q.shape[1], device=q_positions.device).expand_as(q_positions)
            if not torch.equal(q_positions.long(), want):
                raise ValueError("prefill positions must be 0..S-1; use the decode entry for other offsets")

    def forward_with_lse(self, q, k, v, *, q_positions=None, key_padding_mask=None) -> DeterministicAttentionCoreResult:
        self._validate_positions(q, k, q_positions)
        if q.shape[1] == 1 and k.shape[1] > 1:                     # decode: one query per sequence
            from rl_kernel_b200.ops.attention.attention import decode_attention

            pos = q_positions[:, 0] if q_positions is not None else torch.full((q.shape[0],), k.shape[1] - 1,
                                                                              device=q.device)
            o = decode_attention(q[:, 0], k, v, pos, scale=self.scale)
            return DeterministicAttentionCoreResult(o.unsqueeze(1), torch.empty(0, device=q.device))
        o, lse = self._op(q, k, v, causal=True, key_padding_mask=key_padding_mask, scale=self.scale, return_lse=True)
        return DeterministicAttentionCoreResult(o, lse)

    def __call__(self, q, k, v, **kw):
        return self.forward_with_lse(q, k, v, **kw).out
