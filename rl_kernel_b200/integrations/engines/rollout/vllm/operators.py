"""Operator objects the vLLM binding installs (parity: VllmAttentionOperator / VllmFFNOperator /
VllmLogpOperator, rl_engine/integrations/engines/rollout/vllm/operators.py:209-1455).

``VllmAttentionOperator`` consumes what a serving engine hands an attention layer: the new tokens'
Q/K/V, the layer's block KV cache ``[2, num_blocks, block_size, Hkv, D]``, and per-step metadata
(``slot_mapping``, ``block_table``, ``seq_lens``, ``query_start_loc``).  It stores the new K/V rows at
their slots and runs the paged kernel, whose producer walks the block table; the cache block must
be the canonical 128-key block (``--block-size 128``) because a page is the unit the per-row
program is defined on.  A legacy dense call (``kv_cache=(k, v)`` as [B, S_max, Hkv, D] tensors, or
packed prefill with ``cu_seqlens``) is still accepted.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from rl_kernel_b200.ops.attention.attention import causal_attention, decode_attention
from rl_kernel_b200.ops.attention.paged import PAGE, paged_attention_block_table, write_kv_slots
from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn
from rl_kernel_b200.ops.logprob import linear_logp


@dataclass
class VllmKVCacheView:
    """One layer's block cache as the two row pools the kernels address."""
    k_pool: torch.Tensor            # [num_blocks * 128, Hkv * D]
    v_pool: torch.Tensor
    num_blocks: int
    num_kv_heads: int
    head_dim: int

    @classmethod
    def from_tensor(cls, kv_cache: torch.Tensor) -> "VllmKVCacheView":
        if kv_cache.dim() != 5 or kv_cache.shape[0] != 2:
            raise ValueError(f"expected a [2, num_blocks, block_size, Hkv, D] cache, got {tuple(kv_cache.shape)}")
        _, nb, bs, hkv, d = kv_cache.shape
        if bs != PAGE:
            raise ValueError(f"the deterministic paged kernel needs a KV block of {PAGE} tokens (got {bs}); start the "
                             f"engine with --block-size {PAGE}")
        if not kv_cache[0].is_contiguous():
            raise ValueError("the K and V halves of the cache must be contiguous")
        return cls(kv_cache[0].view(nb * bs, hkv * d), kv_cache[1].view(nb * bs, hkv * d), nb, hkv, d)


def _host_list(x) -> list[int]:
    return [int(v) for v in (x.tolist() if isinstance(x, torch.Tensor) else x)]


class VllmAttentionOperator:
    backend_id = "b200-tcgen05"
    schedule = "canonical_128_key_blocks_no_splitkv"

    def __init__(self, peer_pools=None):
        self.peer_pools = peer_pools            # (k_pools, v_pools) of every PCP rank when pages live on other GPUs
        self.calls = {"paged": 0, "dense_decode": 0, "packed_prefill": 0}

    def forward_paged(self, layer, query, key, value, kv_cache: torch.Tensor, attn_metadata: Any,
                      output: torch.Tensor | None = None) -> torch.Tensor:
        """query [T, Hq * D] (or [T, Hq, D]); returns [T, Hq * D].  ``attn_metadata`` needs ``slot_mapping``,
        ``block_table``, ``seq_lens`` (``seq_lens_cpu`` is preferred when present) and ``query_start_loc``
        (``query_start_loc_cpu``), ``num_actual_tokens``."""
        hq, hkv, d = layer.num_heads, layer.num_kv_heads, getattr(layer, "head_dim", None) or layer.head_size
        view = VllmKVCacheView.from_tensor(kv_cache)
        n = int(getattr(attn_metadata, "num_actual_tokens", query.shape[0]))
        q = query[:n].reshape(n, hq, d)
        if key is not None:                                   # forward_includes_kv_cache_update
            write_kv_slots(view.k_pool, view.v_pool, key[:n].reshape(n, hkv * d), value[:n].reshape(n, hkv * d),
                           attn_metadata.slot_mapping[:n])
        lens = _host_list(getattr(attn_metadata, "seq_lens_cpu", None) if getattr(attn_metadata, "seq_lens_cpu", None)
                          is not None else attn_metadata.seq_lens)
        qsl = _host_list(getattr(attn_metadata, "query_start_loc_cpu", None)
                         if getattr(attn_metadata, "query_start_loc_cpu", None) is not None else attn_metadata.query_start_loc)
        out3 = None if output is None else output[:n].view(n, hq, d)
        o = paged_attention_block_table(q, view.k_pool, view.v_pool, attn_metadata.block_table[: len(lens)], lens, qsl,
                                        num_kv_heads=hkv, scale=getattr(layer, "scale", None), out=out3,
                                        peer_pools=self.peer_pools)
        self.calls["paged"] += 1
        if output is not None:
            return output
        return o.reshape(n, hq * d)

    def __call__(self, layer, q, k, v, kv_cache=None, positions=None, cu_seqlens=None, attn_metadata=None, output=None,
                 **kw):
        if attn_metadata is not None and isinstance(kv_cache, torch.Tensor) and kv_cache.dim() == 5:
            return self.forward_paged(layer, q, k, v, kv_cache, attn_metadata, output)
        hq, hkv, d = layer.num_heads, layer.num_kv_heads, layer.head_dim
        if kv_cache is not None and cu_seqlens is None:
            kc, vc = kv_cache                                  # dense [B, S_max, Hkv, D] caches already holding the token
            self.calls["dense_decode"] += 1
            return decode_attention(q.view(-1, hq, d), kc, vc, positions).reshape(q.shape[0], hq * d)
        T = q.shape[0]
        cu = cu_seqlens if cu_seqlens is not None else [0, T]
        self.calls["packed_prefill"] += 1
        return causal_attention(q.view(T, hq, d), k.view(T, hkv, d), v.view(T, hkv, d), cu).reshape(T, hq * d)


class VllmFFNOperator:
    backend_id = "b200-tcgen05"

    def __init__(self, canonical_tp: int = 8, tp_size: int = 1, collective=None):
        self.canonical_tp, self.tp_size, self.collective = canonical_tp, tp_size, collective

    def __call__(self, layer, x):
        """``layer`` carries ``rlk_w_gu`` / ``rlk_w_down`` in the engine layout (set at weight load)."""
        return qwen3_ffn(x, layer.rlk_w_gu, layer.rlk_w_down, canonical_tp=self.canonical_tp, tp_size=self.tp_size,
                         collective=self.collective)


class VllmLogpOperator:
    """Sampled-token log-prob with the trainer's operator; ``min_keep`` replays the sampler's top-k / top-p support."""
    backend_id = "b200-tcgen05"

    def __init__(self, temperature: float = 1.0, real_vocab: int | None = None):
        self.temperature, self.real_vocab = temperature, real_vocab

    def __call__(self, hidden: torch.Tensor, lm_head_weight: torch.Tensor, token_ids: torch.Tensor,
                 min_keep: torch.Tensor | None = None) -> torch.Tensor:
        w = lm_head_weight if self.real_vocab is None else lm_head_weight[: self.real_vocab]
        return linear_logp(hidden, w, token_ids, self.temperature, min_keep=min_keep)
