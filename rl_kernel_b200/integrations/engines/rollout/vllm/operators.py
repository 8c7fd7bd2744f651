"""Operator objects the vLLM binding installs (parity: VllmAttentionOperator / VllmFFNOperator /
VllmLogpOperator, rl_engine/integrations/engines/rollout/vllm/operators.py:209-1455)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.attention.attention import causal_attention, decode_attention
from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn
from rl_kernel_b200.ops.logprob import linear_logp


class VllmAttentionOperator:
    backend_id = "b200-tcgen05"

    def __call__(self, layer, q, k, v, kv_cache=None, positions=None, cu_seqlens=None, **kw):
        """Prefill (``cu_seqlens`` given, q/k/v packed [T, H, D]) or single-token decode
        (``kv_cache`` = (k_cache, v_cache) [B, S_max, Hkv, D] already holding the new token)."""
        hq, hkv, d = layer.num_heads, layer.num_kv_heads, layer.head_dim
        if kv_cache is not None and cu_seqlens is None:
            kc, vc = kv_cache
            return decode_attention(q.view(-1, hq, d), kc, vc, positions).reshape(q.shape[0], hq * d)
        T = q.shape[0]
        cu = cu_seqlens if cu_seqlens is not None else [0, T]
        o = causal_attention(q.view(T, hq, d), k.view(T, hkv, d), v.view(T, hkv, d), cu)
        return o.reshape(T, hq * d)


class VllmFFNOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, canonical_tp: int = 8, tp_size: int = 1, collective=None):
        self.canonical_tp, self.tp_size, self.collective = canonical_tp, tp_size, collective

    def __call__(self, layer, x):
        """``layer`` carries ``rlk_w_gu`` / ``rlk_w_down`` in the engine layout (set at weight load)."""
        return qwen3_ffn(x, layer.rlk_w_gu, layer.rlk_w_down, canonical_tp=self.canonical_tp, tp_size=self.tp_size,
                         collective=self.collective)


class VllmLogpOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, temperature: float = 1.0, real_vocab: int | None = None):
        self.temperature, self.real_vocab = temperature, real_vocab

    def __call__(self, hidden: torch.Tensor, lm_head_weight: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        w = lm_head_weight if self.real_vocab is None else lm_head_weight[: self.real_vocab]
        return linear_logp(hidden, w, token_ids, self.temperature)
