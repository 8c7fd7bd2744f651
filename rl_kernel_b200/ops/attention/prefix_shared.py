"""Prefix-shared attention for GRPO: the G samples of a prompt attend to the prompt's K/V, which is
stored once.  Two forms:

* ``prefix_shared_attention`` -- the stand-alone operator (parity: PrefixSharedAttentionOp /
  csrc/cuda/attention/prefix_shared_attention.cu:85-331 in the reference: Q [bs, G, Lq, Hq, 128]
  against shared K/V [bs, Lkv, Hkv, 128], no causal mask, forward only).  Query rows of different
  samples are packed into the same 128-row tiles of the sm_100a attention kernel, so a K/V block
  is fetched once per tile of up to 128 (sample, position) rows instead of once per sample.
* page sharing during decode (``rl_kernel_b200.models.qwen3.grpo``): the page tables of a group's
  sequences point at the same physical prompt pages, so the shared blocks are read from HBM once
  and served to the other samples from L2; a sequence still runs the canonical per-row program,
  so the bits equal unshared decode and training.
"""
from __future__ import annotations

import math

import torch

from rl_kernel_b200.ops._dispatch import use_native


def prefix_shared_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float | None = None,
                            return_lse: bool = False):
    """q [bs, G, Lq, Hq, D]; k, v [bs, Lkv, Hkv, D] -> out like q (and lse [bs, G, Lq, Hq])."""
    bs, G, Lq, hq, d = q.shape
    Lkv, hkv = k.shape[1], k.shape[2]
    g = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if not use_native(q, k, v):
        kk = k.float().repeat_interleave(g, dim=2)                       # [bs, Lkv, Hq, D]
        vv = v.float().repeat_interleave(g, dim=2)
        s = torch.einsum("bgqhd,bkhd->bgqhk", q.float(), kk) * scale
        lse = torch.logsumexp(s, -1)
        o = torch.einsum("bgqhk,bkhd->bgqhd", torch.softmax(s, -1), vv).to(q.dtype)
        return (o, lse) if return_lse else o
    from rl_kernel_b200.backends import native as nv

    if d != 128:
        raise ValueError("head_dim must be 128")
    rows_per_b = G * Lq
    q2 = q.reshape(bs * rows_per_b, hq * d).contiguous()
    k2 = k.reshape(bs * Lkv, hkv * d).contiguous()
    v2 = v.reshape(bs * Lkv, hkv * d).contiguous()
    tiles = []
    for b in range(bs):
        for r0 in range(0, rows_per_b, 128):
            n = min(128, rows_per_b - r0)
            row0 = b * rows_per_b + r0
            for h in range(hq):
                # pos_step 0: every row of the tile sees all Lkv keys (no causal mask)
                tiles.append([row0, h * d, n, b * Lkv, (h // g) * d, Lkv - 1, 0, Lkv, row0 * hq + h, hq, 0, 0])
    t = torch.tensor(tiles, dtype=torch.int32, device=q.device).contiguous()
    o2 = torch.empty_like(q2)
    lse = torch.empty(bs * rows_per_b, hq, device=q.device, dtype=torch.float32)
    nv.attn_fwd(q2, [k2], [v2], o2, lse, t, scale)
    out = o2.view(bs, G, Lq, hq, d)
    return (out, lse.view(bs, G, Lq, hq)) if return_lse else out


class PrefixSharedAttentionOp:
    backend_id = "b200-tcgen05"
    backward_impl = "none"

    def __init__(self, scale: float | None = None):
        self.scale = scale

    def __call__(self, q, k, v, return_lse: bool = False):
        return prefix_shared_attention(q, k, v, scale=self.scale, return_lse=return_lse)
