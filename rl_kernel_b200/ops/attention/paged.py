"""Paged KV cache attention on the sm_100a kernel: a page is one canonical 128-key block, the
kernel's TMA producer looks the page of every block up in a device page table, so decode and
chunked prefill over a fragmented pool execute the per-row program of contiguous KV bit for bit.
Page-table entries also carry the owning rank, which turns the same call into rollout context
parallelism over a page pool that is spread over several GPUs ("PCP"): every rank computes a
disjoint slice of the query rows and reads remote pages directly over NVLink instead of gathering
them first.  Parity: FA4 paged varlen path and PagedContextParallel
(rl_engine/backends/cuda/attention/flash_attn.py:404-517,
rl_engine/integrations/engines/rollout/vllm/parallel.py:25-158).
"""
from __future__ import annotations

import math

import torch

PAGE = 128


class PagedKVCache:
    """Page pool [num_pages * 128, Hkv * D] for K and V (one layer) with host-side page tables."""

    def __init__(self, num_pages: int, num_kv_heads: int, head_dim: int, device, *, rank: int = 0,
                 k_pool: torch.Tensor | None = None, v_pool: torch.Tensor | None = None):
        if head_dim != 128:
            raise ValueError("head_dim must be 128")
        self.hkv, self.d, self.dev, self.rank = num_kv_heads, head_dim, device, rank
        shape = (num_pages * PAGE, num_kv_heads * head_dim)
        self.k = k_pool if k_pool is not None else torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.v = v_pool if v_pool is not None else torch.zeros(shape, dtype=torch.bfloat16, device=device)
        self.free = list(range(num_pages - 1, -1, -1))
        self.tables: dict[int, list[int]] = {}       # entries: (rank << 24) | page
        self.lengths: dict[int, int] = {}

    def reserve(self, seq: int, new_len: int, *, owner_of_block=None) -> None:
        """Make sure sequence ``seq`` has pages for ``new_len`` tokens.  ``owner_of_block(b)`` names
        the rank whose pool holds block b (default: this rank); only blocks owned here take a page
        from this pool, the others must be filled in with ``set_remote_page``."""
        table = self.tables.setdefault(seq, [])
        while len(table) * PAGE < new_len:
            b = len(table)
            owner = self.rank if owner_of_block is None else owner_of_block(b)
            if owner == self.rank:
                if not self.free:
                    raise RuntimeError("page pool exhausted")
                table.append((owner << 24) | self.free.pop())
            else:
                table.append(-1)
        self.lengths[seq] = max(self.lengths.get(seq, 0), new_len)

    def set_remote_page(self, seq: int, block: int, owner: int, page: int) -> None:
        self.tables[seq][block] = (owner << 24) | page

    def slots(self, seq: int, positions: torch.Tensor) -> torch.Tensor:
        """Pool rows for tokens of ``seq`` at ``positions`` (all in blocks this rank owns)."""
        table = torch.tensor([e & 0xFFFFFF for e in self.tables[seq]], dtype=torch.long)
        pos = positions.long().cpu()
        return (table[pos // PAGE] * PAGE + pos % PAGE).to(torch.int32).to(self.dev)

    def write(self, seq: int, positions: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
        """k, v [n, Hkv * D] for tokens at ``positions`` (the engine's fused QK-norm+RoPE kernel
        writes straight into the pool through ``slots`` instead)."""
        s = self.slots(seq, positions).long()
        self.k[s] = k
        self.v[s] = v

    def release(self, seq: int) -> None:
        for e in self.tables.pop(seq, []):
            if e >= 0 and (e >> 24) == self.rank:
                self.free.append(e & 0xFFFFFF)
        self.lengths.pop(seq, None)

    def table_tensor(self, seqs: list[int]) -> tuple[torch.Tensor, list[int]]:
        flat, offs = [], []
        for s in seqs:
            offs.append(len(flat))
            if any(e < 0 for e in self.tables[s]):
                raise RuntimeError(f"sequence {s} has blocks without a page")
            flat += self.tables[s]
        return torch.tensor(flat, dtype=torch.int32, device=self.dev), offs


def paged_attention(q: torch.Tensor, cache: PagedKVCache, seqs: list[int], q_positions: list[torch.Tensor], *,
                    scale: float | None = None, peer_pools: tuple[list[torch.Tensor], list[torch.Tensor]] | None = None,
                    return_lse: bool = False):
    """q [T, Hq, D]: the query tokens of the listed sequences back to back; ``q_positions[i]`` are
    the (ascending, consecutive) positions of sequence i's queries.  One token per sequence is
    decode, several are chunked prefill.  ``peer_pools = (k_pools, v_pools)`` lists every rank's
    pools (this rank's own at its index) when page tables point at other GPUs."""
    from rl_kernel_b200.backends import native as nv

    T, hq, d = q.shape
    hkv, g = cache.hkv, hq // cache.hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    table, offs = cache.table_tensor(seqs)
    rows, t0 = [], 0
    single = all(p.numel() == 1 for p in q_positions)
    for i, s in enumerate(seqs):
        pos = q_positions[i]
        n, p0 = pos.numel(), int(pos[0])
        kv_cap = p0 + n
        if single:
            # decode: the GQA group's heads become the rows of one tile (q viewed as [T*Hq, D])
            for hk in range(hkv):
                r0 = t0 * hq + hk * g
                rows.append([r0, 0, g, 0, hk * d, p0, 0, kv_cap, r0, 1, 0, offs[i] + 1])
        else:
            for qt in range((n + 127) // 128 - 1, -1, -1):
                for h in range(hq):
                    r0 = t0 + qt * 128
                    rows.append([r0, h * d, min(128, n - qt * 128), 0, (h // g) * d, p0 + qt * 128, 1, kv_cap,
                                 r0 * hq + h, hq, 0, offs[i] + 1])
        t0 += n
    tiles = torch.tensor(rows, dtype=torch.int32, device=q.device).contiguous()
    k_list, v_list = peer_pools if peer_pools is not None else ([cache.k], [cache.v])
    lse = torch.empty(T, hq, device=q.device, dtype=torch.float32)
    if single:
        q2 = torch.zeros(T * hq + 128, d, device=q.device, dtype=q.dtype)
        q2[: T * hq] = q.reshape(T * hq, d)
        o2 = torch.empty_like(q2)
        nv.attn_fwd(q2, k_list, v_list, o2, lse, tiles, scale, decode=g <= 8, page_table=table)
        out = o2[: T * hq].view(T, hq, d)
    else:
        q2 = q.reshape(T, hq * d).contiguous()
        o2 = torch.empty_like(q2)
        nv.attn_fwd(q2, k_list, v_list, o2, lse, tiles, scale, page_table=table)
        out = o2.view(T, hq, d)
    return (out, lse) if return_lse else out


def write_kv_slots(k_pool: torch.Tensor, v_pool: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                   slot_mapping: torch.Tensor) -> None:
    """Store the new tokens' K/V rows [T, Hkv * D] at flat pool rows ``slot_mapping`` [T] (negative = padding token:
    skipped).  Pools are [num_pages * 128, Hkv * D] views of the cache."""
    slots = slot_mapping.reshape(-1).long()
    key, value = key.reshape(key.shape[0], -1), value.reshape(value.shape[0], -1)
    if key.is_cuda and (key.shape[1] * key.element_size()) % 16 == 0 and key.stride(1) == 1 and value.stride(1) == 1:
        from rl_kernel_b200.ops.packing import _move

        _move(key, slots.contiguous(), k_pool, True)       # the kernel skips indices outside [0, rows)
        _move(value, slots.contiguous(), v_pool, True)
        return
    ok = slots >= 0
    k_pool[slots[ok]] = key[ok]
    v_pool[slots[ok]] = value[ok]


def paged_attention_block_table(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                                seq_lens, query_start_loc, *, num_kv_heads: int, scale: float | None = None,
                                out: torch.Tensor | None = None, return_lse: bool = False,
                                peer_pools: tuple[list[torch.Tensor], list[torch.Tensor]] | None = None):
    """Causal attention of a continuous batch over a block-table KV cache (the metadata a serving engine keeps).

    q [T, Hq, D]: the new tokens of all requests back to back; request i owns rows
    ``query_start_loc[i]:query_start_loc[i+1]`` and its cache (new tokens included) holds ``seq_lens[i]`` tokens, so its
    queries sit at positions ``seq_lens[i] - n_i .. seq_lens[i] - 1``.  ``block_table`` [B, max_blocks] int32 lists the
    128-token pages of every request (-1 padded; entries may carry an owner rank in bits 24+ together with
    ``peer_pools``).  ``seq_lens`` / ``query_start_loc`` are host sequences (a serving engine has them on the CPU).
    Decode rows (one new token) and prefill chunks may be mixed in one call."""
    T, hq, d = q.shape
    hkv, g = num_kv_heads, hq // num_kv_heads
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    lens = [int(x) for x in (seq_lens.tolist() if isinstance(seq_lens, torch.Tensor) else seq_lens)]
    qsl = [int(x) for x in (query_start_loc.tolist() if isinstance(query_start_loc, torch.Tensor) else query_start_loc)]
    B, maxb = block_table.shape
    if len(lens) != B or len(qsl) != B + 1:
        raise ValueError("seq_lens needs one entry and query_start_loc one boundary more than the block table has rows")
    if not q.is_cuda:
        return _paged_reference(q, k_pool, v_pool, block_table, lens, qsl, hkv, scale, out, return_lse)
    from rl_kernel_b200.backends import native as nv

    if d != 128:
        raise ValueError("head_dim must be 128")
    table = block_table.to(torch.int32).contiguous().view(-1)          # row i starts at i * max_blocks
    decode_rows, prefill_rows = [], []
    for i in range(B):
        n, t0 = qsl[i + 1] - qsl[i], qsl[i]
        if n == 0:
            continue
        p0 = lens[i] - n
        if p0 < 0:
            raise ValueError(f"request {i}: {n} query tokens but only {lens[i]} cached")
        if n == 1:
            for hk in range(hkv):
                r0 = t0 * hq + hk * g
                decode_rows.append([r0, 0, g, 0, hk * d, p0, 0, lens[i], r0, 1, 0, i * maxb + 1])
        else:
            for qt in range((n + 127) // 128 - 1, -1, -1):
                for h in range(hq):
                    r0 = t0 + qt * 128
                    prefill_rows.append([r0, h * d, min(128, n - qt * 128), 0, (h // g) * d, p0 + qt * 128, 1, lens[i],
                                         r0 * hq + h, hq, 0, i * maxb + 1])
    k_list, v_list = peer_pools if peer_pools is not None else ([k_pool], [v_pool])
    o = out.view(T, hq, d) if out is not None else torch.empty_like(q)
    lse = torch.empty(T, hq, device=q.device, dtype=torch.float32)
    if decode_rows:                      # the GQA group's heads are the rows of one tile: q viewed as [T * Hq, D]
        tiles = torch.tensor(decode_rows, dtype=torch.int32, device=q.device)
        q2 = torch.zeros(T * hq + 128, d, device=q.device, dtype=q.dtype)
        q2[: T * hq] = q.reshape(T * hq, d)
        o2 = torch.empty_like(q2)
        nv.attn_fwd(q2, k_list, v_list, o2, lse, tiles, scale, decode=g <= 8, page_table=table)
        if prefill_rows:
            sel = torch.tensor(sorted({r[0] // hq for r in decode_rows}), device=q.device)
            o[sel] = o2[: T * hq].view(T, hq, d)[sel]
        else:
            o.copy_(o2[: T * hq].view(T, hq, d))
    if prefill_rows:
        tiles = torch.tensor(prefill_rows, dtype=torch.int32, device=q.device)
        q2 = q.reshape(T, hq * d).contiguous()
        o2 = torch.empty_like(q2) if decode_rows else o.view(T, hq * d)
        lse2 = torch.empty_like(lse) if decode_rows else lse
        nv.attn_fwd(q2, k_list, v_list, o2, lse2, tiles, scale, page_table=table)
        if decode_rows:
            rows = torch.cat([torch.arange(qsl[i], qsl[i + 1]) for i in range(B) if qsl[i + 1] - qsl[i] > 1]).to(q.device)
            o[rows] = o2.view(T, hq, d)[rows]
            lse[rows] = lse2[rows]
    return (o, lse) if return_lse else o


def _paged_reference(q, k_pool, v_pool, block_table, lens, qsl, hkv, scale, out, return_lse):
    """The same semantics with gathered pages on the CPU: the block-wise reference with per-row products, whose
    result for a query row does not depend on which other rows (chunk, batch) it is computed with."""
    from rl_kernel_b200.reference.attention.blockwise import blockwise_attention_reference

    T, hq, d = q.shape
    o = out.view(T, hq, d) if out is not None else torch.empty_like(q)
    lse = torch.zeros(T, hq)
    for i in range(len(lens)):
        n = qsl[i + 1] - qsl[i]
        if n == 0:
            continue
        pages = (block_table[i, : (lens[i] + PAGE - 1) // PAGE].long() & 0xFFFFFF)
        rows = (pages[:, None] * PAGE + torch.arange(PAGE)[None]).reshape(-1)[: lens[i]]
        k = k_pool[rows].view(lens[i], hkv, d)
        v = v_pool[rows].view(lens[i], hkv, d)
        oi, li = blockwise_attention_reference(q[qsl[i]:qsl[i + 1]], k, v, torch.arange(lens[i] - n, lens[i]), scale=scale,
                                               strict=True)
        o[qsl[i]:qsl[i + 1]] = oi
        lse[qsl[i]:qsl[i + 1]] = li
    return (o, lse) if return_lse else o
