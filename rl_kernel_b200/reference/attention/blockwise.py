"""Blockwise attention with the canonical schedule of the sm_100a kernels, and the
context-parallel reference built on it.

Contract (csrc/attention/attn_fwd_sm100.cu): keys are consumed in blocks of 128 counted from the
first key of the sequence, in ascending order, with an online softmax per query row; a block
that is fully masked for a row leaves its (m, l, acc) state untouched.  Because a row's program
depends only on its own position, any split of the QUERY rows over batches, chunks or
context-parallel ranks gives the same bits: CP changes where K/V blocks are read from, not the
arithmetic.  The reference's PyTorch CP op defines the same property with (out, lse) partial
states merged in global block order (rl_engine/reference/attention/cp_attention.py:378-411,
1661-1672); ``merge_two_states`` is kept for API parity and for checking the equivalence.
"""
from __future__ import annotations

import math

import torch

BLOCK = 128


def merge_two_states(o1, lse1, o2, lse2):
    """Combine two partial attention results over disjoint key sets (fp32, logaddexp weights)."""
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse).unsqueeze(-1)
    w2 = torch.exp(lse2 - lse).unsqueeze(-1)
    return torch.nan_to_num(w1) * o1 + torch.nan_to_num(w2) * o2, lse


def _row_block_products(qf, kf, vf, k0, block, strict):
    """Scores of every query row against the zero-padded key block and the padded value block."""
    nb = min(block, kf.shape[1] - k0)
    kb = kf.new_zeros(kf.shape[0], block, kf.shape[2])
    vb = vf.new_zeros(vf.shape[0], block, vf.shape[2])
    kb[:, :nb], vb[:, :nb] = kf[:, k0:k0 + nb], vf[:, k0:k0 + nb]
    if not strict:
        return qf @ kb.transpose(-1, -2), vb
    # one matrix-vector product per (head, row), always against a full [block, D] operand, so a
    # row's bits cannot depend on the batch, on the chunking or on how much of the block is filled
    s = torch.stack([torch.stack([torch.mv(kb[h], qf[h, i]) for i in range(qf.shape[1])])
                     for h in range(qf.shape[0])]) if qf.shape[1] else qf.new_zeros(qf.shape[0], 0, block)
    return s, vb


def blockwise_attention_reference(q, k, v, q_pos, *, scale=None, block: int = BLOCK,
                                  p_dtype: torch.dtype | None = None, strict: bool = True):
    """q [Sq, Hq, D], k/v [Skv, Hkv, D], q_pos [Sq] (key position of each query row).
    Returns (out [Sq, Hq, D] in q.dtype, lse [Sq, Hq] fp32). ``p_dtype`` rounds the probabilities
    before P·V the way the kernel does (bf16).  ``strict`` computes every row with its own
    matrix-vector products (bitwise batch/chunk invariant on any BLAS); ``strict=False`` uses
    batched matmuls and is only tolerance-equal."""
    Sq, Hq, D = q.shape
    Skv, Hkv = k.shape[0], k.shape[1]
    g = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(1, 0, 2).contiguous()          # [Hq, Sq, D]
    kf = k.float().permute(1, 0, 2).repeat_interleave(g, dim=0).contiguous()
    vf = v.float().permute(1, 0, 2).repeat_interleave(g, dim=0).contiguous()
    m = torch.full((Hq, Sq), float("-inf"))
    l = torch.zeros(Hq, Sq)
    acc = torch.zeros(Hq, Sq, D)
    kv_len = (q_pos.long() + 1).clamp(max=Skv)            # [Sq]
    nblk = (int(kv_len.max().item()) + block - 1) // block if Sq else 0
    for b in range(nblk):
        k0 = b * block
        s, vb = _row_block_products(qf, kf, vf, k0, block, strict)
        idx = torch.arange(k0, k0 + block)
        vis = idx[None, :] < kv_len[:, None]              # [Sq, block]
        s = s.masked_fill(~vis[None], float("-inf"))
        m_blk = s.max(dim=-1).values
        m_new = torch.maximum(m, m_blk)
        m_use = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
        alpha = torch.exp((m - m_use) * scale)
        p = torch.exp((s - m_use.unsqueeze(-1)) * scale)
        p = torch.where(vis[None], p, torch.zeros_like(p))
        psum = p.new_zeros(Hq, Sq)
        for j in range(block):                            # fixed ascending order
            psum = psum + p[..., j]
        l = l * alpha + psum
        pr = p.to(p_dtype).float() if p_dtype is not None else p
        if strict:
            vt = vb.transpose(-1, -2).contiguous()        # [Hq, D, block]
            pv = torch.stack([torch.stack([torch.mv(vt[h], pr[h, i]) for i in range(Sq)])
                              for h in range(Hq)])
        else:
            pv = pr @ vb
        acc = acc * alpha.unsqueeze(-1) + pv
        m = m_new
    out = acc / l.clamp_min(1e-38).unsqueeze(-1)
    out = torch.where((l > 0).unsqueeze(-1), out, torch.zeros_like(out))
    lse = torch.where(l > 0, m * scale + torch.log(l.clamp_min(1e-38)), torch.full_like(l, float("-inf")))
    return out.permute(1, 0, 2).to(q.dtype), lse.permute(1, 0)


def zigzag_chunks(seq_len: int, cp: int) -> list[list[tuple[int, int]]]:
    """Megatron zigzag: 2*cp equal chunks; rank c owns chunks c and 2*cp-1-c (load balance)."""
    n = 2 * cp
    if seq_len % n:
        raise ValueError("sequence length must be divisible by 2*cp")
    c = seq_len // n
    return [[(r * c, (r + 1) * c), ((n - 1 - r) * c, (n - r) * c)] for r in range(cp)]


class DeterministicCPAttentionReferenceOp:
    """Context-parallel attention simulated in one process: the sequence is sharded over ``cp``
    ranks (contiguous or zigzag), every rank computes its own query rows against the full K/V
    with the canonical block schedule, and the shards are stitched back.  The result is bitwise
    equal to ``cp = 1`` for every cp and layout."""

    def __init__(self, cp: int = 1, layout: str = "zigzag", scale: float | None = None,
                 p_dtype: torch.dtype | None = None):
        if layout not in ("zigzag", "contiguous"):
            raise ValueError(layout)
        self.cp, self.layout, self.scale, self.p_dtype = cp, layout, scale, p_dtype

    def shard_positions(self, seq_len: int) -> list[torch.Tensor]:
        if self.cp == 1:
            return [torch.arange(seq_len)]
        if self.layout == "contiguous":
            c = seq_len // self.cp
            return [torch.arange(r * c, (r + 1) * c) for r in range(self.cp)]
        return [torch.cat([torch.arange(a, b) for a, b in chunks]) for chunks in zigzag_chunks(seq_len, self.cp)]

    def __call__(self, q, k, v):
        """q [S, Hq, D], k/v [S, Hkv, D] (one causal sequence) -> (out, lse)."""
        S = q.shape[0]
        out = torch.empty_like(q)
        lse = torch.empty(S, q.shape[1])
        for pos in self.shard_positions(S):
            o, l = blockwise_attention_reference(q[pos], k, v, pos, scale=self.scale, p_dtype=self.p_dtype)
            out[pos], lse[pos] = o, l
        return out, lse

    forward = __call__
