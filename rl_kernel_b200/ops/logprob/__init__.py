"""Selected-token log-prob operators: from logits (batch-invariant, tile contract) and fused
linear->logp (hidden @ W^T never materialised), both differentiable with native backward."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops._dispatch import use_native
from rl_kernel_b200.reference.logprob.tile_logp import (NativeBatchInvariantLogpOp, NativeLinearLogpOp, TILE)


def _ntiles(vocab: int) -> int:
    return (vocab + TILE - 1) // TILE


class _LogpFromLogitsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, inv_temp, min_keep=None):
        from rl_kernel_b200.backends import native as nv

        rows, V = logits.shape
        stats = torch.empty(rows, _ntiles(V), 2, device=logits.device, dtype=torch.float32)
        tl = torch.zeros(rows, device=logits.device, dtype=torch.float32)
        nv.logits_tile_stats(logits, targets, stats, tl, vocab_start=0, inv_temp=inv_temp, min_keep=min_keep)
        logp = torch.empty(rows, device=logits.device, dtype=torch.float32)
        lse = torch.empty(rows, device=logits.device, dtype=torch.float32)
        nv.logp_merge(stats, tl, logp, lse)
        ctx.save_for_backward(logits, targets, lse, min_keep)
        ctx.inv_temp = inv_temp
        return logp

    @staticmethod
    def backward(ctx, g):
        from rl_kernel_b200.backends import native as nv

        logits, targets, lse, min_keep = ctx.saved_tensors
        d = logits.clone()
        nv.dlogits_(d, targets, lse, g.float().contiguous(), vocab_start=0, inv_temp=ctx.inv_temp, min_keep=min_keep)
        return d, None, None, None


def _keep_rows(min_keep, rows: int, device):
    if min_keep is None:
        return None
    mk = min_keep.reshape(-1).to(device=device, dtype=torch.float32).contiguous()
    if mk.numel() != rows:
        raise ValueError(f"min_keep must hold one threshold per token ({rows}), got {mk.numel()}")
    return mk


def logp_from_logits(logits: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0,
                     min_keep: torch.Tensor | None = None) -> torch.Tensor:
    """logits [..., V] bf16, targets [...] -> fp32 selected log-prob (batch-invariant, differentiable).

    ``min_keep`` [...] restricts the softmax to the sampling support of each token: scaled logits
    (logit / temperature) below the token's threshold count as -inf, which is what the rollout sampler
    drew from under top-k / top-p (``ops.sampling.policy.keep_threshold``)."""
    shp = targets.shape
    lg = logits.reshape(-1, logits.shape[-1])
    mk = _keep_rows(min_keep, lg.shape[0], lg.device)
    if not use_native(lg):
        return NativeBatchInvariantLogpOp(temperature).apply_fp32(lg, targets.reshape(-1), min_keep=mk).view(shp)
    return _LogpFromLogitsFn.apply(lg.contiguous(), targets.reshape(-1).contiguous(), 1.0 / temperature, mk).view(shp)


def replay_logp_from_logits(logits: torch.Tensor, targets: torch.Tensor, replay_ids: torch.Tensor,
                            temperature: float = 1.0, *, vocab_start: int = 0, return_lse: bool = False,
                            collective=None):
    """Selected log-prob over the compact support ``replay_ids`` [..., K<=64] (global ids; duplicates
    allowed) instead of the whole vocabulary -- bit-equal to ``logp_from_logits`` on logits masked to
    -inf outside those ids, at a cost of K loads per token instead of V.  Inference only.
    With ``collective`` (vocabulary-parallel shards; ``vocab_start`` = first id of this shard) the
    shards' compact tile lists are gathered in rank order before the merge.
    (parity: sm90_deterministic_top_p_logp_from_local_logits_tp, rl_engine/backends/cuda/logprob/
    linear_logp.py:1417-1494.)"""
    shp = targets.shape
    lg = logits.reshape(-1, logits.shape[-1])
    ids = replay_ids.reshape(-1, replay_ids.shape[-1]).to(device=lg.device, dtype=torch.long).contiguous()
    tg = targets.reshape(-1).to(device=lg.device, dtype=torch.long).contiguous()
    rows, K = ids.shape
    if rows != lg.shape[0] or tg.numel() != rows:
        raise ValueError("replay ids, targets and logits rows must align")
    if K > 64:
        raise ValueError("replay width exceeds the compact kernel limit of 64")
    world = getattr(collective, "world", 1) if collective is not None else 1
    if not use_native(lg):
        keep = torch.zeros(rows, lg.shape[1], dtype=torch.bool)
        local = ids - vocab_start
        ok = (local >= 0) & (local < lg.shape[1])
        keep[torch.arange(rows)[:, None].expand_as(local)[ok], local[ok]] = True
        op = NativeBatchInvariantLogpOp(temperature)
        if world == 1:
            lp, lse = op.apply_fp32(lg, tg, keep_mask=keep, return_lse=True)
        else:
            from rl_kernel_b200.reference.logprob.tile_logp import _target_z, merge_tile_stats, tile_stats_reference

            z = lg.float().masked_fill(~keep, float("-inf"))
            st = tile_stats_reference(z, vocab_start=0, inv_temp=op.inv_temp)
            tz, own = _target_z(z, tg, vocab_start, op.inv_temp)
            st = collective.all_gather(st).permute(1, 0, 2, 3).reshape(rows, -1, 2)
            lp, lse = merge_tile_stats(st, collective.all_gather(torch.where(own, tz, torch.zeros_like(tz))).sum(0))
        return (lp.view(shp), lse.view(shp)) if return_lse else lp.view(shp)
    from rl_kernel_b200.backends import native as nv

    with torch.no_grad():
        stats = torch.empty(rows, K, 2, device=lg.device, dtype=torch.float32)
        tl = torch.zeros(rows, device=lg.device, dtype=torch.float32)
        nv.replay_tile_stats(lg.contiguous(), tg, ids, stats, tl, vocab_start=vocab_start, inv_temp=1.0 / temperature)
        if world > 1:
            stats = collective.all_gather(stats).permute(1, 0, 2, 3).reshape(rows, world * K, 2).contiguous()
            tl = collective.all_gather(tl).sum(0)             # exactly one shard owns the target
        lp = torch.empty(rows, device=lg.device, dtype=torch.float32)
        lse = torch.empty(rows, device=lg.device, dtype=torch.float32)
        nv.logp_merge(stats, tl, lp, lse)
    return (lp.view(shp), lse.view(shp)) if return_lse else lp.view(shp)


class _IndexedLogpLseFn(torch.autograd.Function):
    """(logp, lse) of the rows listed in ``row_indices``; both outputs are differentiable."""

    @staticmethod
    def forward(ctx, logits, targets, row_indices, inv_temp):
        from rl_kernel_b200.backends import native as nv

        V = logits.shape[1]
        rows = row_indices.numel()
        stats = torch.empty(rows, _ntiles(V), 2, device=logits.device, dtype=torch.float32)
        tl = torch.zeros(rows, device=logits.device, dtype=torch.float32)
        nv.logits_tile_stats(logits, targets, stats, tl, vocab_start=0, inv_temp=inv_temp, row_indices=row_indices)
        logp = torch.empty(rows, device=logits.device, dtype=torch.float32)
        lse = torch.empty(rows, device=logits.device, dtype=torch.float32)
        nv.logp_merge(stats, tl, logp, lse)
        ctx.save_for_backward(logits, targets, row_indices, lse)
        ctx.inv_temp = inv_temp
        return logp, lse

    @staticmethod
    def backward(ctx, g_logp, g_lse):
        from rl_kernel_b200.backends import native as nv

        logits, targets, row_indices, lse = ctx.saved_tensors
        sel = logits.index_select(0, row_indices).contiguous()
        nv.dlogits_(sel, targets, lse, g_logp.float().contiguous(), vocab_start=0, inv_temp=ctx.inv_temp,
                    g_lse=g_lse.float().contiguous())
        d = torch.zeros_like(logits)
        d.index_add_(0, row_indices, sel)        # an index may repeat: its gradients add up
        return d, None, None, None


def logp_from_logits_indexed(logits: torch.Tensor, targets: torch.Tensor, row_indices: torch.Tensor,
                             temperature: float = 1.0, return_lse: bool = False):
    """Selected log-prob of ``targets[i]`` under row ``row_indices[i]`` of ``logits`` [R, V] (scoring
    a subset of positions without gathering the logits first; parity: the row_indices variants of
    csrc/cuda/logprob/fused_logp_kernel.cu:125-220).  With ``return_lse`` also the log-sum-exp,
    whose gradient is g_lse * softmax."""
    if not use_native(logits):
        lg = logits.index_select(0, row_indices)
        lp = NativeBatchInvariantLogpOp(temperature).apply_fp32(lg, targets)
        if not return_lse:
            return lp
        return lp, torch.logsumexp(lg.float() / temperature, -1)
    lp, lse = _IndexedLogpLseFn.apply(logits.contiguous(), targets.contiguous(), row_indices.contiguous().long(),
                                      1.0 / temperature)
    return (lp, lse) if return_lse else lp


class _LinearLogpFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, targets, inv_temp, chunk, min_keep=None):
        from rl_kernel_b200.backends import native as nv

        rows, V = hidden.shape[0], weight.shape[0]
        logp = torch.empty(rows, device=hidden.device, dtype=torch.float32)
        lse = torch.empty(rows, device=hidden.device, dtype=torch.float32)
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            stats = torch.empty(r1 - r0, _ntiles(V), 2, device=hidden.device, dtype=torch.float32)
            tl = torch.zeros(r1 - r0, device=hidden.device, dtype=torch.float32)
            nv.lmhead_logp_stats(hidden[r0:r1], weight, targets[r0:r1], stats, tl, vocab_start=0, inv_temp=inv_temp,
                                 min_keep=None if min_keep is None else min_keep[r0:r1])
            nv.logp_merge(stats, tl, logp[r0:r1], lse[r0:r1])
        ctx.save_for_backward(hidden, weight, targets, lse, min_keep)
        ctx.meta = (inv_temp, chunk)
        return logp

    @staticmethod
    def backward(ctx, g):
        from rl_kernel_b200.backends import native as nv

        hidden, weight, targets, lse, min_keep = ctx.saved_tensors
        inv_temp, chunk = ctx.meta
        rows, H = hidden.shape
        V = weight.shape[0]
        v8 = (V + 7) // 8 * 8                    # GEMM extents step by 8: a vocabulary that is not a multiple (rare) is padded with zero rows
        wmat = weight if v8 == V else torch.cat([weight, weight.new_zeros(v8 - V, H)])
        g = g.float().contiguous()
        dh = torch.empty_like(hidden)
        dw = torch.zeros_like(wmat)
        for r0 in range(0, rows, chunk):
            r1 = min(rows, r0 + chunk)
            n = r1 - r0
            npad = (n + 7) // 8 * 8           # the dW contraction runs over rows: zero rows pad it to the GEMM's K step
            buf = torch.empty(npad, v8, device=hidden.device, dtype=hidden.dtype)
            logits, hrows = buf[:n], hidden[r0:r1]
            nv.det_gemm(hrows, wmat, logits, M=n, N=v8, K=H)
            nv.dlogits_(logits, targets[r0:r1], lse[r0:r1], g[r0:r1], vocab_start=0, inv_temp=inv_temp,
                        min_keep=None if min_keep is None else min_keep[r0:r1])
            if v8 != V:
                logits[:, V:].zero_()          # padding ids are outside the softmax: no gradient
            nv.det_gemm(logits, wmat, dh[r0:r1], M=n, N=H, K=v8, b_mn=True)
            if npad != n:
                buf[n:].zero_()
                hrows = torch.cat([hrows, hrows.new_zeros(npad - n, H)])
            nv.det_gemm(buf, hrows, dw, M=v8, N=H, K=npad, a_mn=True, b_mn=True, accumulate=True)
        dw = dw if v8 == V else dw[:V].contiguous()
        return dh, dw, None, None, None, None


def linear_logp(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, temperature: float = 1.0,
                chunk: int = 4096, min_keep: torch.Tensor | None = None) -> torch.Tensor:
    """logp[n] = log_softmax(hidden[n] @ weight^T / T)[targets[n]] without keeping [N, V] logits
    (parity: FusedLinearLogpSM90Op, rl_engine/backends/cuda/logprob/linear_logp.py:802).
    ``min_keep`` [...]: per-token sampling-support threshold, applied in the GEMM epilogue (see
    ``logp_from_logits``); the train side replays the rollout's top-k / top-p support with it."""
    shp = targets.shape
    h = hidden.reshape(-1, hidden.shape[-1])
    mk = _keep_rows(min_keep, h.shape[0], h.device)
    if not use_native(h, weight):
        return NativeLinearLogpOp(temperature)(h, weight, targets.reshape(-1), min_keep=mk).view(shp)
    return _LinearLogpFn.apply(h.contiguous(), weight.contiguous(), targets.reshape(-1).contiguous(),
                               1.0 / temperature, chunk, mk).view(shp)


class BatchInvariantLogpOp:
    backend_id = "b200"
    is_fused_logp = True
    backward_impl = "native"

    def __init__(self, temperature: float = 1.0):
        self.temperature = temperature

    def __call__(self, logits, token_ids, *, min_keep=None):
        return logp_from_logits(logits, token_ids, self.temperature, min_keep=min_keep)

    forward = apply_fp32 = __call__

    def replay(self, logits, token_ids, replay_ids, **kw):
        return replay_logp_from_logits(logits, token_ids, replay_ids, self.temperature, **kw)


class LinearLogpOp:
    backend_id = "b200-tcgen05"
    is_fused_logp = True
    backward_impl = "native"

    def __init__(self, temperature: float = 1.0):
        self.temperature = temperature

    def __call__(self, hidden, weight, targets, *, min_keep=None):
        return linear_logp(hidden, weight, targets, self.temperature, min_keep=min_keep)

    forward = __call__
