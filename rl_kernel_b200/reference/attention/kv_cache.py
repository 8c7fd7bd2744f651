"""KV-cache attention reference: append K/V at a position, attend over the filled prefix with
the canonical block schedule (parity: NativeKVCacheAttnOp / StatefulKVCache,
rl_engine/reference/attention/{kv_cache,stateful_kv}.py)."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from rl_kernel_b200.reference.attention.blockwise import blockwise_attention_reference


@dataclass
class StatefulKVCache:
    k: torch.Tensor  # [layers, batch, max_len, Hkv, D]
    v: torch.Tensor
    lengths: torch.Tensor  # [batch]

    @classmethod
    def allocate(cls, n_layers, batch, n_kv_heads, max_seq_len, head_dim, dtype, device="cpu"):
        shape = (n_layers, batch, max_seq_len, n_kv_heads, head_dim)
        return cls(torch.zeros(shape, dtype=dtype, device=device), torch.zeros(shape, dtype=dtype, device=device),
                   torch.zeros(batch, dtype=torch.long, device=device))

    def append(self, layer: int, k_new: torch.Tensor, v_new: torch.Tensor, start: torch.Tensor) -> None:
        """k_new/v_new [batch, n, Hkv, D] written at positions start[b] .. start[b]+n."""
        n = k_new.shape[1]
        for b in range(k_new.shape[0]):
            s = int(start[b])
            self.k[layer, b, s:s + n] = k_new[b]
            self.v[layer, b, s:s + n] = v_new[b]


class NativeKVCacheAttnOp:
    def __init__(self, p_dtype: torch.dtype | None = None):
        self.p_dtype = p_dtype

    def __call__(self, q, cache: StatefulKVCache, layer: int, q_pos: torch.Tensor, scale=None):
        """q [batch, n, Hq, D]; q_pos [batch, n] absolute positions -> out [batch, n, Hq, D]."""
        outs = []
        for b in range(q.shape[0]):
            kv_len = int(q_pos[b].max()) + 1
            o, _ = blockwise_attention_reference(q[b], cache.k[layer, b, :kv_len], cache.v[layer, b, :kv_len],
                                                 q_pos[b], scale=scale, p_dtype=self.p_dtype)
            outs.append(o)
        return torch.stack(outs)

    forward = __call__
