"""Vocabulary-parallel fused linear -> selected log-prob on the sm_100a kernels, differentiable.

Every rank holds a row shard of the LM head.  Forward: the GEMM epilogue reduces its logits tile
to per-(row, 128-id tile) softmax statistics (the [N, V] logits are never written); the tile
statistics and the owner's target logit travel through the group's fixed-order collective (no
floating-point all-reduce: every tile has exactly one owner) and every rank merges the complete
tile list in ascending tile order -- the same bits for 1, 2, 4 or 8 shards.  Backward: logits of
the local shard are recomputed per row chunk, turned into dlogits in place, and multiplied into
dH (canonical vocabulary chunks + tree all-reduce) and dW (local).
(parity: CudaVocabParallelLogprobOp / sm90_deterministic_linear_logp_tp,
rl_engine/backends/cuda/logprob/vocab_parallel_logp.py:116, linear_logp.py:1078-1690).
"""
from __future__ import annotations

import torch

from rl_kernel_b200.reference.logprob.tile_logp import TILE


def _stats(nv, hidden, weight, targets, vocab_start, inv_temp, ntile, collective, rank, world):
    n = hidden.shape[0]
    dev = hidden.device
    stats = torch.empty(n, ntile, 2, device=dev, dtype=torch.float32)
    stats[..., 0] = float("-inf")
    stats[..., 1] = 0
    tl = torch.zeros(n, device=dev, dtype=torch.float32)
    if weight.shape[0] > 0:
        nv.lmhead_logp_stats(hidden, weight, targets, stats, tl, vocab_start=vocab_start, inv_temp=inv_temp)
    if world > 1:
        per = ntile // world
        mine = stats[:, rank * per:(rank + 1) * per].contiguous()
        g = collective.all_gather(mine)                       # [world, n, per, 2], bits unchanged
        stats = g.permute(1, 0, 2, 3).reshape(n, ntile, 2).contiguous()
        tl = collective.all_gather(tl).sum(0)                 # exactly one rank holds a non-zero entry per row
    return stats, tl


class _VPLinearLogpFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, op):
        from rl_kernel_b200.backends import native as nv

        rows = hidden.shape[0]
        logp = torch.empty(rows, device=hidden.device, dtype=torch.float32)
        lse = torch.empty(rows, device=hidden.device, dtype=torch.float32)
        for r0 in range(0, rows, op.chunk):
            r1 = min(rows, r0 + op.chunk)
            st, tl = _stats(nv, hidden[r0:r1], weight[:op.real_rows], targets[r0:r1], op.vocab_start, op.inv_temp,
                            op.ntile, op.collective, op.rank, op.world)
            nv.logp_merge(st, tl, logp[r0:r1], lse[r0:r1])
        ctx.save_for_backward(hidden, weight, targets, lse)
        ctx.op = op
        return logp

    @staticmethod
    def backward(ctx, g):
        from rl_kernel_b200.backends import native as nv

        hidden, weight, targets, lse = ctx.saved_tensors
        op = ctx.op
        rows, H = hidden.shape
        vloc, vpad = op.real_rows, weight.shape[0]
        g = g.float().contiguous()
        dh = torch.empty_like(hidden)
        dw = torch.zeros_like(weight)
        # GEMM extents step by 8: the real ids round up into the (zero) padding rows of the shard, whose logits are 0 and
        # whose gradient is set to 0; the token contraction of dW rounds up with zero rows
        v8 = min(vpad, (vloc + 7) // 8 * 8)
        cap = (min(rows, op.chunk) + 7) // 8 * 8
        logits = torch.zeros(cap, vpad, device=hidden.device, dtype=hidden.dtype)
        for r0 in range(0, rows, op.chunk):
            r1 = min(rows, r0 + op.chunk)
            n = r1 - r0
            n8 = (n + 7) // 8 * 8
            lg, hrows = logits[:n], hidden[r0:r1]
            if vloc > 0:
                nv.det_gemm(hrows, weight[:v8], lg[:, :v8], M=n, N=v8, K=H)
                nv.dlogits_(lg[:, :v8], targets[r0:r1], lse[r0:r1], g[r0:r1], vocab_start=op.vocab_start,
                            inv_temp=op.inv_temp)
                if v8 != vloc:
                    lg[:, vloc:v8].zero_()
                # canonical vocabulary chunks: the padded shard splits into equal pieces, the padding
                # columns are zero, and the tree over the ranks finishes the same sum for every world
                nv.det_gemm(lg, weight, dh[r0:r1], M=n, N=H, K=vpad, b_mn=True, nchunks=op.nchunks)
                if n8 != n:
                    logits[n:n8].zero_()
                    hrows = torch.cat([hrows, hrows.new_zeros(n8 - n, H)])
                nv.det_gemm(logits[:n8, :v8], hrows, dw[:v8], M=v8, N=H, K=n8, a_mn=True, b_mn=True, accumulate=True)
            else:
                dh[r0:r1].zero_()
        if op.world > 1:
            op.collective.all_reduce_(dh)
        return dh, dw, None, None


class VocabParallelLinearLogpOp:
    """``op(hidden [N, H], weight_shard [V_pad / world, H], targets [N])`` -> fp32 log-prob [N].

    ``padded_vocab`` must be a multiple of ``8 * 128`` (so that no 128-id tile straddles a shard);
    ``real_vocab`` ids beyond it are padding: their rows of the weight shard must be zero and they
    take no part in the softmax."""

    backend_id = "b200-tcgen05-vocab-parallel"
    is_fused_logp = True
    backward_impl = "native"

    def __init__(self, *, real_vocab: int, padded_vocab: int, collective=None, temperature: float = 1.0,
                 canonical_shards: int = 8, chunk: int = 4096):
        self.collective = collective
        self.world = getattr(collective, "world", 1) if collective is not None else 1
        self.rank = getattr(collective, "rank", 0) if collective is not None else 0
        if padded_vocab % (canonical_shards * TILE) or canonical_shards % self.world:
            raise ValueError(f"padded vocabulary {padded_vocab} must split into {canonical_shards} x 128-id tiles and "
                             f"{self.world} ranks must divide {canonical_shards}")
        v_local = padded_vocab // self.world
        self.vocab_start = self.rank * v_local
        self.real_rows = max(0, min(v_local, real_vocab - self.vocab_start))
        self.v_local, self.ntile = v_local, padded_vocab // TILE
        self.nchunks = canonical_shards // self.world
        self.inv_temp, self.chunk = 1.0 / temperature, chunk

    def __call__(self, hidden, weight_shard, targets):
        if weight_shard.shape[0] != self.v_local:
            raise ValueError(f"weight shard has {weight_shard.shape[0]} rows, expected {self.v_local}")
        shp = targets.shape
        h = hidden.reshape(-1, hidden.shape[-1]).contiguous()
        return _VPLinearLogpFn.apply(h, weight_shard.contiguous(), targets.reshape(-1).contiguous(), self).view(shp)

    forward = __call__
