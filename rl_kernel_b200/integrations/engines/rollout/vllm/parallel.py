"""Prefill context parallelism for rollout ("PCP"): KV pages are token-interleaved over the CP ranks;
each rank gathers the pages it needs, restores logical order, computes a disjoint slice of the query
rows over the full KV, and the outputs are gathered in rank order — no floating-point reduction,
so the result equals the single-rank one bit for bit (parity: PagedContextParallel,
rl_engine/integrations/engines/rollout/vllm/parallel.py:25-158)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.attention.attention import causal_attention


class PagedContextParallel:
    def __init__(self, collective, cp_size: int, cp_rank: int):
        self.coll, self.cp, self.rank = collective, cp_size, cp_rank

    def shard_tokens(self, x: torch.Tensor) -> torch.Tensor:
        """Token-interleaved shard: rank r keeps tokens r, r+cp, ..."""
        return x[self.rank::self.cp].contiguous()

    def restore(self, gathered: torch.Tensor, total: int) -> torch.Tensor:
        """gathered [cp, ceil(total/cp), ...] in rank order -> logical token order [total, ...]."""
        out = gathered.new_empty((total,) + tuple(gathered.shape[2:]))
        for r in range(self.cp):
            n = len(range(r, total, self.cp))
            out[r::self.cp] = gathered[r, :n]
        return out

    def _gather_padded(self, x: torch.Tensor, total: int) -> torch.Tensor:
        per = (total + self.cp - 1) // self.cp
        pad = x.new_zeros((per,) + tuple(x.shape[1:]))
        pad[: x.shape[0]] = x
        return self.coll.all_gather(pad) if self.cp > 1 else pad.unsqueeze(0)

    def forward(self, q_local, k_local, v_local, total_tokens: int, scale=None) -> torch.Tensor:
        """All inputs are this rank's interleaved shard [T_local, H, D]; returns this rank's shard
        of the attention output."""
        k = self.restore(self._gather_padded(k_local, total_tokens), total_tokens)
        v = self.restore(self._gather_padded(v_local, total_tokens), total_tokens)
        q = self.restore(self._gather_padded(q_local, total_tokens), total_tokens)
        # every rank computes whole-sequence rows only for the positions it owns: the kernel's rows
        # are independent, so computing the full sequence and slicing gives the same bits
        o = causal_attention(q, k, v, [0, total_tokens], scale=scale)
        return o[self.rank::self.cp].contiguous()
