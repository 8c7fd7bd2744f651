"""Operator objects for the Megatron binding, including the zigzag context-parallel layout helpers
(parity: rl_engine/integrations/engines/train/megatron/operators.py:102-601)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.attention.attention import causal_attention
from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn
from rl_kernel_b200.ops.logprob import linear_logp
from rl_kernel_b200.reference.attention.blockwise import zigzag_chunks


def megatron_zigzag_positions(seq_len: int, cp_size: int, cp_rank: int) -> torch.Tensor:
    """Global positions of the tokens a CP rank holds under Megatron's zigzag split."""
    if cp_size == 1:
        return torch.arange(seq_len)
    return torch.cat([torch.arange(a, b) for a, b in zigzag_chunks(seq_len, cp_size)[cp_rank]])


class MegatronAttentionOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, cp_size: int = 1, cp_collective=None):
        self.cp_size, self.cp_collective = cp_size, cp_collective

    def __call__(self, layer, q, k, v, cu_seqlens=None, **kw):
        """q/k/v in Megatron's [S, B, H, D] layout (B sequences of equal length S)."""
        S, B, hq, d = q.shape
        hkv = k.shape[2]
        if self.cp_size > 1:
            raise NotImplementedError("context-parallel training attention goes through CPAttention "
                                      "(rl_kernel_b200.distributed.cp_attention), bound by the engine")
        pack = lambda t, h: t.permute(1, 0, 2, 3).reshape(B * S, h, d)  # noqa: E731
        cu = [i * S for i in range(B + 1)]
        o = causal_attention(pack(q, hq), pack(k, hkv), pack(v, hkv), cu)
        return o.view(B, S, hq, d).permute(1, 0, 2, 3).reshape(S, B, hq * d)


class MegatronFFNOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, canonical_tp: int = 8, tp_size: int = 1, collective=None):
        self.canonical_tp, self.tp_size, self.collective = canonical_tp, tp_size, collective

    def __call__(self, layer, x):
        return qwen3_ffn(x, layer.rlk_w_gu, layer.rlk_w_down, canonical_tp=self.canonical_tp, tp_size=self.tp_size,
                         collective=self.collective)


class MegatronLogpOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, temperature: float = 1.0):
        self.temperature = temperature

    def __call__(self, layer, hidden, targets):
        return linear_logp(hidden, layer.weight, targets, self.temperature)
