"""The 128-id vocab-tile log-prob contract in PyTorch (csrc/include/rlk/logp_contract.cuh):

  tile t covers GLOBAL ids [128 t, 128 t + 128); per (row, tile): m = max z, s = sum exp(z - m) with
  the 128 terms added as four interleaved sequential chains combined as (c0+c1)+(c2+c3);
  per row: M = max_t m_t, S = sum_t s_t * exp(m_t - M) in ascending t, lse = M + log S,
  logp = min(z_target - lse, 0).

Tiles never straddle a vocab-parallel shard, so gathering the per-shard tile statistics in rank
order and merging gives the same bits for TP = 1, 2, 4, 8.  (The reference's version of this idea
is its 64-tile contract, rl_engine/reference/logprob/vocab_parallel_logp.py:4-36,194-363.)
"""
from __future__ import annotations

import torch

from rl_kernel_b200.reference.gemm.det_gemm import det_gemm_reference

TILE = 128


def tile_stats_reference(logits: torch.Tensor, *, vocab_start: int = 0, inv_temp: float = 1.0,
                         n_tiles_total: int | None = None) -> torch.Tensor:
    """logits [rows, n_local] (local shard starting at global id ``vocab_start``) ->
    stats [rows, n_tiles_total, 2] with untouched tiles = (-inf, 0)."""
    if vocab_start % TILE:
        raise ValueError("vocab_start must be a multiple of 128")
    rows, n_local = logits.shape
    nt_local = (n_local + TILE - 1) // TILE
    t0 = vocab_start // TILE
    total = n_tiles_total if n_tiles_total is not None else t0 + nt_local
    z = logits.float() * torch.tensor(inv_temp, dtype=torch.float32, device=logits.device)
    pad = nt_local * TILE - n_local
    if pad:
        z = torch.cat([z, z.new_full((rows, pad), float("-inf"))], dim=1)
    z = z.view(rows, nt_local, TILE)
    m = z.max(dim=-1).values
    e = torch.exp(z - torch.where(torch.isinf(m), torch.zeros_like(m), m).unsqueeze(-1))
    e = torch.where(torch.isinf(m).unsqueeze(-1), torch.zeros_like(e), e)
    chains = e.view(rows, nt_local, TILE // 4, 4)
    c = torch.zeros(rows, nt_local, 4, device=logits.device)
    for j in range(TILE // 4):          # four sequential chains, ascending
        c = c + chains[:, :, j]
    s = (c[..., 0] + c[..., 1]) + (c[..., 2] + c[..., 3])
    stats = torch.zeros(rows, total, 2, device=logits.device)
    stats[..., 0] = float("-inf")
    stats[:, t0:t0 + nt_local, 0] = m
    stats[:, t0:t0 + nt_local, 1] = s
    return stats


def merge_tile_stats(stats: torch.Tensor, target_z: torch.Tensor):
    """stats [rows, tiles, 2], target_z [rows] (scaled target logit) -> (logp, lse)."""
    m, s = stats[..., 0], stats[..., 1]
    M = m.max(dim=-1).values
    S = torch.zeros_like(M)
    for t in range(stats.shape[1]):     # ascending tile order
        w = torch.exp(m[:, t] - M)
        term = torch.where(torch.isinf(m[:, t]), torch.zeros_like(w), s[:, t] * w)
        S = S + term
    lse = M + torch.log(S)
    return torch.minimum(target_z - lse, torch.zeros_like(lse)), lse


def _target_z(logits, targets, vocab_start, inv_temp):
    local = targets.long() - vocab_start
    own = (local >= 0) & (local < logits.shape[1])
    z = logits.float().gather(1, local.clamp(0, logits.shape[1] - 1).unsqueeze(1)).squeeze(1)
    z = z * torch.tensor(inv_temp, dtype=torch.float32, device=z.device)
    return torch.where(own, z, torch.zeros_like(z)), own


def _restrict(lg: torch.Tensor, inv_temp: float, min_keep, keep_mask) -> torch.Tensor:
    """Logits with everything outside the sampling support set to -inf (fp32 result when restricted)."""
    if min_keep is None and keep_mask is None:
        return lg
    z = lg.float() * torch.tensor(inv_temp, dtype=torch.float32, device=lg.device)
    keep = torch.ones_like(z, dtype=torch.bool)
    if min_keep is not None:
        keep &= z >= min_keep.reshape(-1, 1).to(z.device)
    if keep_mask is not None:
        keep &= keep_mask.to(z.device)
    return lg.float().masked_fill(~keep, float("-inf"))


class NativeBatchInvariantLogpOp:
    """Selected log-prob from materialised logits with the tile contract (batch-invariant)."""
    is_fused_logp = False

    def __init__(self, temperature: float = 1.0):
        self.inv_temp = 1.0 / temperature

    def apply_fp32(self, logits, token_ids, *, min_keep=None, keep_mask=None, return_lse: bool = False):
        """``min_keep`` [rows]: scaled logits below it are outside the support; ``keep_mask`` [rows, V]
        bool: an explicit support.  Outside the support a logit counts as -inf."""
        shp = token_ids.shape
        lg = _restrict(logits.reshape(-1, logits.shape[-1]), self.inv_temp, min_keep, keep_mask)
        stats = tile_stats_reference(lg, inv_temp=self.inv_temp)
        tz, _ = _target_z(lg, token_ids.reshape(-1), 0, self.inv_temp)
        lp, lse = merge_tile_stats(stats, tz)
        return (lp.view(shp), lse.view(shp)) if return_lse else lp.view(shp)

    def __call__(self, logits, token_ids, **kw):
        return self.apply_fp32(logits, token_ids, **kw)

    forward = __call__


class NativeLinearLogpOp:
    """hidden -> selected log-prob without keeping [N, V] logits beyond the call: logits are the
    batch-invariant GEMM rounded to the compute dtype, then the tile contract."""
    is_fused_logp = True

    def __init__(self, temperature: float = 1.0):
        self.inv_temp = 1.0 / temperature

    def __call__(self, hidden, weight, targets, *, vocab_start: int = 0, n_tiles_total=None,
                 return_stats: bool = False, min_keep=None):
        logits = _restrict(det_gemm_reference(hidden, weight), self.inv_temp, min_keep, None)
        stats = tile_stats_reference(logits, vocab_start=vocab_start, inv_temp=self.inv_temp,
                                     n_tiles_total=n_tiles_total)
        tz, own = _target_z(logits, targets, vocab_start, self.inv_temp)
        if return_stats:
            return stats, tz, own
        return merge_tile_stats(stats, tz)[0]

    forward = __call__


class VocabParallelLogprobOp:
    """Vocab-parallel selected log-prob: each rank computes tile stats for its shard; stats and the
    target logit travel by all-gather only (no floating-point all-reduce); every rank merges the
    full tile list in tile order.  Works with a ``torch.distributed`` group or, with
    ``group=None``, on a list of shards in one process (simulated TP)."""

    def __init__(self, temperature: float = 1.0, group=None):
        self.linear = NativeLinearLogpOp(temperature)
        self.group = group

    def simulate(self, hidden, weight_shards: list[torch.Tensor], targets, n_tiles_total: int):
        stats = None
        tz = torch.zeros(hidden.shape[0], device=hidden.device)
        start = 0
        for w in weight_shards:
            st, z, _ = self.linear(hidden, w, targets, vocab_start=start, n_tiles_total=n_tiles_total,
                                   return_stats=True)
            nt0, nt1 = start // TILE, (start + w.shape[0] + TILE - 1) // TILE
            if stats is None:
                stats = st.clone()
            else:
                stats[:, nt0:nt1] = st[:, nt0:nt1]
            tz = tz + z
            start += w.shape[0]
        return merge_tile_stats(stats, tz)[0]

    def __call__(self, hidden, weight_shard, targets, *, vocab_start: int, n_tiles_total: int):
        import torch.distributed as dist

        st, z, _ = self.linear(hidden, weight_shard, targets, vocab_start=vocab_start,
                               n_tiles_total=n_tiles_total, return_stats=True)
        if self.group is None and not (dist.is_available() and dist.is_initialized()):
            return merge_tile_stats(st, z)[0]
        world = dist.get_world_size(self.group)
        nt_local = (weight_shard.shape[0] + TILE - 1) // TILE
        mine = st[:, vocab_start // TILE: vocab_start // TILE + nt_local].contiguous()
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine, group=self.group)
        zs = [torch.empty_like(z) for _ in range(world)]
        dist.all_gather(zs, z, group=self.group)
        stats = torch.cat(gathered, dim=1)
        if stats.shape[1] < n_tiles_total:
            pad = stats.new_zeros(stats.shape[0], n_tiles_total - stats.shape[1], 2)
            pad[..., 0] = float("-inf")
            stats = torch.cat([stats, pad], dim=1)
        tz = torch.stack(zs).sum(0)   # exactly one rank holds a non-zero entry per row
        return merge_tile_stats(stats, tz)[0]

    forward = __call__
