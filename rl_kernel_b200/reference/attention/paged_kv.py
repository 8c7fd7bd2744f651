"""Paged KV cache reference: a pool of 128-token pages plus per-sequence page tables, scored by
materialising each sequence's keys in logical order and running the blockwise reference (parity:
StatefulKVCache / PagedKVScoringBaseline, rl_engine/reference/attention/stateful_kv.py:20 and
paged_kv.py:85).  The page size equals the canonical KV block, so paging changes where a block is
read from and nothing about the arithmetic."""
from __future__ import annotations

import torch

from rl_kernel_b200.reference.attention.blockwise import blockwise_attention_reference

PAGE = 128


class PagedKVReference:
    def __init__(self, num_pages: int, num_kv_heads: int, head_dim: int, dtype=torch.bfloat16):
        self.k = torch.zeros(num_pages, PAGE, num_kv_heads, head_dim, dtype=dtype)
        self.v = torch.zeros_like(self.k)
        self.free = list(range(num_pages - 1, -1, -1))
        self.tables: dict[int, list[int]] = {}
        self.lengths: dict[int, int] = {}

    def append(self, seq: int, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v [n, Hkv, D]: the next n tokens of sequence ``seq``."""
        table = self.tables.setdefault(seq, [])
        n0 = self.lengths.get(seq, 0)
        for i in range(k.shape[0]):
            pos = n0 + i
            if pos // PAGE >= len(table):
                if not self.free:
                    raise RuntimeError("page pool exhausted")
                table.append(self.free.pop())
            self.k[table[pos // PAGE], pos % PAGE] = k[i]
            self.v[table[pos // PAGE], pos % PAGE] = v[i]
        self.lengths[seq] = n0 + k.shape[0]

    def release(self, seq: int) -> None:
        self.free.extend(reversed(self.tables.pop(seq, [])))
        self.lengths.pop(seq, None)

    def gather(self, seq: int) -> tuple[torch.Tensor, torch.Tensor]:
        n, table = self.lengths[seq], self.tables[seq]
        k = torch.cat([self.k[p] for p in table])[:n]
        v = torch.cat([self.v[p] for p in table])[:n]
        return k, v

    def score(self, seq: int, q: torch.Tensor, positions: torch.Tensor, scale: float | None = None):
        """q [n, Hq, D] at ``positions`` [n] of sequence ``seq`` -> (out, lse)."""
        k, v = self.gather(seq)
        return blockwise_attention_reference(q, k, v, positions, scale=scale, strict=False)
