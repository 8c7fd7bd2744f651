"""Prefix-shared attention device operator (parity: PrefixSharedAttentionOp,
rl_engine/backends/cuda/attention/prefix_shared_attn.py:11-70).

Accepts the reference's single-head shapes (q [bs, G, Lq, D]; k, v [bs, Lkv, D]) as well as the
multi-head GQA shapes of ``ops.attention.prefix_shared`` (q [bs, G, Lq, Hq, D]).  The G samples'
query rows share 128-row tiles, so the prompt's K/V blocks are fetched once per tile.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.attention.prefix_shared import prefix_shared_attention


class PrefixSharedAttentionOp:
    backend_id = "b200-tcgen05"

    def __init__(self):
        self.has_hardware_op = torch.cuda.is_available()

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        if q.dim() == 4:                                   # [bs, G, Lq, D] with a single head
            if q.dtype != torch.bfloat16:
                raise TypeError("Only BF16 is supported for this kernel.")
            return prefix_shared_attention(q.unsqueeze(3), k.unsqueeze(2), v.unsqueeze(2)).squeeze(3)
        return prefix_shared_attention(q, k, v)
