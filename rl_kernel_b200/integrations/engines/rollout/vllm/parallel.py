"""Prefill context parallelism for rollout ("PCP", parity: PagedContextParallel,
rl_engine/integrations/engines/rollout/vllm/parallel.py:25-158).

The reference gathers Q, K and V on every CP rank and computes the whole sequence everywhere.  Here
the KV pages stay where they were written: block b of a sequence lives in the pool of rank
``b % cp`` and every rank's page table names the owner of each block, so the paged kernel reads
remote pages over NVLink while it computes only this rank's slice of the query rows.  Nothing is
gathered and no floating-point value is reduced, hence the rows equal the single-rank ones bit for
bit.  ``forward_gathered`` keeps the reference's gather-everything graph for transports without
peer memory (Gloo on CPU) and as the definition the native path is tested against.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.attention.attention import causal_attention
from rl_kernel_b200.ops.attention.paged import PAGE, PagedKVCache, paged_attention


class PagedContextParallel:
    def __init__(self, collective, cp_size: int, cp_rank: int):
        self.coll, self.cp, self.rank = collective, cp_size, cp_rank
        self._pm = None
        self.cache: PagedKVCache | None = None

    # ---- native path: page pool spread over the CP ranks, remote pages read in the kernel
    def attach_pools(self, num_pages: int, num_kv_heads: int, head_dim: int, device) -> PagedKVCache:
        """Allocate this rank's pool in peer-mapped memory and exchange the mappings (collective)."""
        from rl_kernel_b200.distributed.cp_attention import PeerMappedBuffers

        shape = (num_pages * PAGE, num_kv_heads * head_dim)
        self._pm = PeerMappedBuffers(getattr(self.coll, "group", None), device, {"k": (shape, torch.bfloat16),
                                                                                   "v": (shape, torch.bfloat16)})
        self.cache = PagedKVCache(num_pages, num_kv_heads, head_dim, device, rank=self.rank,
                                  k_pool=self._pm.local("k"), v_pool=self._pm.local("v"))
        return self.cache

    def owner_of_block(self, block: int) -> int:
        return block % self.cp

    def query_slice(self, total_tokens: int) -> tuple[int, int]:
        per = (total_tokens + self.cp - 1) // self.cp
        return min(total_tokens, self.rank * per), min(total_tokens, (self.rank + 1) * per)

    def write_owned_blocks(self, seq: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v [total, Hkv, D] of the whole sequence (every rank computed or received them); this rank stores the
        blocks it owns and learns the page ids of the others."""
        import torch.distributed as dist

        total = k.shape[0]
        self.cache.reserve(seq, total, owner_of_block=self.owner_of_block)
        for b in range((total + PAGE - 1) // PAGE):
            if self.owner_of_block(b) == self.rank:
                lo, hi = b * PAGE, min(total, (b + 1) * PAGE)
                self.cache.write(seq, torch.arange(lo, hi), k[lo:hi].reshape(hi - lo, -1), v[lo:hi].reshape(hi - lo, -1))
        tables = [None] * self.cp
        dist.all_gather_object(tables, self.cache.tables[seq], group=getattr(self.coll, "group", None))
        for b in range(len(self.cache.tables[seq])):
            o = self.owner_of_block(b)
            if o != self.rank:
                self.cache.set_remote_page(seq, b, o, tables[o][b] & 0xFFFFFF)
        self.coll.barrier()                       # every rank's pages are written before anyone reads them

    def forward(self, q_slice: torch.Tensor, seq: int, total_tokens: int, scale=None) -> torch.Tensor:
        """q_slice [hi - lo, Hq, D]: this rank's contiguous slice ``query_slice(total_tokens)`` of the query rows;
        returns the matching output rows."""
        if self.cache is None:
            raise RuntimeError("call attach_pools() and write_owned_blocks() first")
        lo, hi = self.query_slice(total_tokens)
        if hi == lo:
            return q_slice.new_empty(0, *q_slice.shape[1:])
        out = paged_attention(q_slice.contiguous(), self.cache, [seq], [torch.arange(lo, hi)], scale=scale,
                              peer_pools=(self._pm["k"], self._pm["v"]))
        return out

    def release(self, seq: int) -> None:
        self.coll.barrier()                       # nobody frees a page a peer still reads
        self.cache.release(seq)

    # ---- gather-everything graph (any transport)
    def shard_tokens(self, x: torch.Tensor) -> torch.Tensor:
        """Token-interleaved shard: rank r keeps tokens r, r + cp, ..."""
        return x[self.rank::self.cp].contiguous()

    def restore(self, gathered: torch.Tensor, total: int) -> torch.Tensor:
        """gathered [cp, ceil(total / cp), ...] in rank order -> logical token order [total, ...]."""
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

    def forward_gathered(self, q_local, k_local, v_local, total_tokens: int, scale=None) -> torch.Tensor:
        """Inputs are this rank's interleaved shards [T_local, H, D]; returns this rank's shard of the output.  Every
        rank computes the whole sequence (cp-fold redundant work): use ``forward`` where peer memory exists."""
        k = self.restore(self._gather_padded(k_local, total_tokens), total_tokens)
        v = self.restore(self._gather_padded(v_local, total_tokens), total_tokens)
        q = self.restore(self._gather_padded(q_local, total_tokens), total_tokens)
        o = causal_attention(q, k, v, [0, total_tokens], scale=scale)
        return o[self.rank::self.cp].contiguous()
