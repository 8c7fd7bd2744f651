"""Contract-driven vocabulary-parallel selected log-prob in PyTorch
(parity: rl_engine/reference/logprob/vocab_parallel_logp.py:44-760).

The padded vocabulary is cut into fixed tiles; every tile's fp32 (max, sum-exp) partial is computed
from a contiguous [n, tile] block by the rank that owns it; partials travel by all-gather
(transport only) and every rank merges the complete list in ascending global tile order.  The TP
degree decides who computes which tiles and nothing else, so values and gradients are bit-equal
at every TP degree (``DeterminismScope.CROSS_TP_BITWISE``) while the tile size is held fixed.

Tile size.  The contract's ``numerics.tile`` (128 ids) is the default and is what the sm_100a
kernels implement; with it this module reproduces their bits (four interleaved chains inside a
tile, tiles folded with one fma each).  ``num_vocab_tiles`` may pin another decomposition
(tile = padded vocabulary / num_vocab_tiles) for comparisons with engines that fix the tile count
instead; every shard boundary must then be aligned to that tile.

Selected log-probs are zero at inactive rows (``MaskSpec.active_mask`` is the sole authority).
The vocabulary-domain LSE is returned for every row and is differentiable everywhere.
"""
from __future__ import annotations

from typing import Any, Protocol

import torch

from rl_kernel_b200.contracts.operators.logprob import (DeterminismScope, LogprobContract, LogprobContractError,
                                                         LogprobDType)

BACKEND_ID = "pytorch-vocab-parallel-logp"
DEFAULT_NUM_VOCAB_TILES = None          # None: tiles of contract.numerics.tile ids (128)

_TORCH_TO_CONTRACT_DTYPE = {torch.bfloat16: LogprobDType.BF16, torch.float16: LogprobDType.FP16,
                            torch.float32: LogprobDType.FP32}


def _require_distributed_initialized():
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        raise LogprobContractError("tp_world_size > 1 needs an initialised torch.distributed process group")
    return dist


def _tile_size(contract: LogprobContract, num_vocab_tiles: int | None) -> int:
    padded = contract.sharding.padded_vocab_size
    if num_vocab_tiles is None:
        tile = contract.numerics.tile
    else:
        if not isinstance(num_vocab_tiles, int) or isinstance(num_vocab_tiles, bool) or num_vocab_tiles <= 0:
            raise LogprobContractError(f"num_vocab_tiles must be a positive integer; got {num_vocab_tiles!r}")
        if padded % num_vocab_tiles:
            raise LogprobContractError(f"padded_vocab_size={padded} is not divisible by num_vocab_tiles={num_vocab_tiles}")
        tile = padded // num_vocab_tiles
    for rank, (start, end) in enumerate(contract.sharding.vocab_shard_bounds):
        if start % tile or (end % tile and end != padded):
            raise LogprobContractError(f"vocab shard {rank} = [{start}, {end}) is not aligned to the tile size {tile}; "
                                       "tiles must not straddle shards")
    return tile


def _validate_invocation(local_logits, target_ids, contract, tp_group) -> None:
    if not isinstance(contract, LogprobContract):
        raise LogprobContractError("contract must be a LogprobContract")
    if local_logits.dim() != 2:
        raise LogprobContractError(f"local_logits must be 2-D [num_tokens, local_vocab]; got {local_logits.dim()}-D")
    if target_ids.dim() != 1 or target_ids.shape[0] != local_logits.shape[0]:
        raise LogprobContractError("target_ids must be 1-D with one entry per token; got shape "
                                   f"{tuple(target_ids.shape)} for {local_logits.shape[0]} tokens")
    sh = contract.sharding
    if local_logits.shape[1] != sh.local_vocab_size:
        raise LogprobContractError(f"local_logits has {local_logits.shape[1]} vocab columns but the contract declares local "
                                   f"shard [{sh.local_vocab_start}, {sh.local_vocab_end}) of size {sh.local_vocab_size}")
    if local_logits.shape[0] != contract.mask.num_tokens:
        raise LogprobContractError(f"local_logits has {local_logits.shape[0]} tokens but MaskSpec declares "
                                   f"num_tokens={contract.mask.num_tokens}")
    if _TORCH_TO_CONTRACT_DTYPE.get(local_logits.dtype) is not contract.dtype:
        raise LogprobContractError(f"local_logits dtype {local_logits.dtype} does not match the contract dtype "
                                   f"{contract.dtype.value}")
    if sh.tp_world_size > 1:
        dist = _require_distributed_initialized()
        world, rank = dist.get_world_size(group=tp_group), dist.get_rank(group=tp_group)
        if world != sh.tp_world_size:
            raise LogprobContractError(f"tp_group world size {world} does not match the contract tp_world_size="
                                       f"{sh.tp_world_size}; pass the TP subgroup, not the global group")
        if rank != sh.tp_rank:
            raise LogprobContractError(f"tp_group rank {rank} does not match the contract tp_rank={sh.tp_rank}")


def _validate_active_targets(target_1d, active_mask, real_vocab_size: int) -> None:
    bad = active_mask & ((target_1d < 0) | (target_1d >= real_vocab_size))
    if bool(bad.any().item()):
        vals = target_1d[bad]
        raise LogprobContractError(f"active target_ids must lie in the real vocabulary [0, {real_vocab_size}); got values in "
                                   f"[{int(vals.min().item())}, {int(vals.max().item())}] on active rows")


def _preflight_cross_rank_agreement(contract, tp_group, tile: int, deterministic: bool) -> None:
    """All-gather the numerical mode and stop before any mismatched collective."""
    dist = _require_distributed_initialized()
    payload = (contract.cross_rank_fingerprint(), BACKEND_ID, int(tile) if deterministic else None, bool(deterministic))
    got: list[Any] = [None] * dist.get_world_size(group=tp_group)
    dist.all_gather_object(got, payload, group=tp_group)
    for rank, other in enumerate(got):
        if other != payload:
            raise LogprobContractError(f"cross-rank preflight failed: rank {contract.sharding.tp_rank} has {payload} but rank "
                                       f"{rank} has {other}; all TP ranks must agree on the contract fingerprint, backend "
                                       "id, tile size and deterministic mode before any collective")


def _masked_scaled(local_logits, contract) -> torch.Tensor:
    """fp32 z = logit / temperature with the padding columns of this shard at -inf."""
    sh = contract.sharding
    inv_t = torch.tensor(1.0 / contract.numerics.temperature, dtype=torch.float32, device=local_logits.device)
    z = local_logits.float() * inv_t
    keep = max(0, min(sh.local_vocab_size, sh.real_vocab_size - sh.local_vocab_start))
    if keep < sh.local_vocab_size:
        z = torch.cat([z[:, :keep], z.new_full((z.shape[0], sh.local_vocab_size - keep), float("-inf"))], dim=1)
    return z


def _local_tile_stats(z_masked: torch.Tensor, tile: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-tile (max, sum-exp) of this shard, each tile reduced as a contiguous [n, tile] block in the fixed
    in-tile order: four interleaved chains (position mod 4) added sequentially, combined as (c0+c1)+(c2+c3).
    An all--inf tile yields the identity (-inf, 0) without evaluating exp(-inf - -inf)."""
    rows, n = z_masked.shape
    nt = (n + tile - 1) // tile
    if nt * tile != n:
        z_masked = torch.cat([z_masked, z_masked.new_full((rows, nt * tile - n), float("-inf"))], dim=1)
    z = z_masked.view(rows, nt, tile)
    m = z.max(dim=-1).values
    safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    e = torch.exp(z - safe.unsqueeze(-1))
    e = torch.where(torch.isinf(m).unsqueeze(-1), torch.zeros_like(e), e).view(rows, nt, tile // 4, 4)
    c = torch.zeros(rows, nt, 4, device=z.device, dtype=torch.float32)
    for j in range(tile // 4):
        c = c + e[:, :, j]
    return m, (c[..., 0] + c[..., 1]) + (c[..., 2] + c[..., 3])


class _AllGatherUneven:
    """torch.distributed.all_gather of tensors that share every dim but the last; the last dims come from the
    contract's shard table, so no size exchange is needed."""

    @staticmethod
    def apply(t, contract, tp_group, last_dims=None):
        dist = _require_distributed_initialized()
        world = contract.sharding.tp_world_size
        last_dims = last_dims or [t.shape[-1]] * world
        width = max(last_dims)
        pad = t if t.shape[-1] == width else torch.cat([t, t.new_zeros(*t.shape[:-1], width - t.shape[-1])], dim=-1)
        out = [torch.empty_like(pad) for _ in range(world)]
        dist.all_gather(out, pad.contiguous(), group=tp_group)
        return [o[..., :n] for o, n in zip(out, last_dims)]


def _gather_tile_stats(m_loc, s_loc, contract, tp_group, tile: int) -> tuple[torch.Tensor, torch.Tensor]:
    sh = contract.sharding
    if sh.tp_world_size == 1:
        return m_loc, s_loc
    counts = [(e - s + tile - 1) // tile for s, e in sh.vocab_shard_bounds]
    ms = _AllGatherUneven.apply(m_loc, contract, tp_group, counts)
    ss = _AllGatherUneven.apply(s_loc, contract, tp_group, counts)
    return torch.cat(ms, dim=1), torch.cat(ss, dim=1)


def _gather_target_logit(z_masked, target_1d, active_mask, contract, tp_group) -> tuple[torch.Tensor, torch.Tensor]:
    """Masked single-owner gather: the owner contributes the scaled target logit, every other rank exactly 0, and the
    contributions are added in rank order (one non-zero term: the sum is exact).  Returns (target_z, local index or -1)."""
    sh = contract.sharding
    local = target_1d - sh.local_vocab_start
    own = active_mask & (local >= 0) & (local < sh.local_vocab_size) & (target_1d < sh.real_vocab_size)
    idx = torch.where(own, local, torch.zeros_like(local))
    mine = torch.where(own, z_masked.gather(1, idx.unsqueeze(1)).squeeze(1), torch.zeros(1, device=z_masked.device))
    if sh.tp_world_size > 1:
        parts = _AllGatherUneven.apply(mine.unsqueeze(-1), contract, tp_group)
        total = torch.zeros_like(mine)
        for p in parts:
            total = total + p.squeeze(-1)
        mine = total
    return mine, torch.where(own, local, torch.full_like(local, -1))


def _merge_tile_partials(m_all: torch.Tensor, s_all: torch.Tensor) -> torch.Tensor:
    """Fixed-order merge over [n, tiles]: M = max m; S += s_t * exp(m_t - M) with one fma per tile in ascending t
    (empty tiles skipped); LSE = M + log S."""
    M = m_all.max(dim=1).values
    safe = torch.where(torch.isinf(M), torch.zeros_like(M), M)
    S = torch.zeros_like(M)
    for t in range(m_all.shape[1]):
        w = torch.exp(m_all[:, t] - safe)
        live = ~torch.isinf(m_all[:, t])
        S = torch.where(live, torch.addcmul(S, s_all[:, t], w), S)
    return M + torch.log(S)


def _entropy_partials(z_masked, lse) -> torch.Tensor:
    """This shard's part of -sum p log p = lse - sum p z, i.e. sum_j p_j z_j over the shard (fp32)."""
    p = torch.exp(z_masked - lse.unsqueeze(1))
    pz = torch.where(torch.isinf(z_masked), torch.zeros_like(p), p * z_masked)
    return pz.sum(dim=1)


class _VocabParallelLogprobFunction(torch.autograd.Function):
    """(selected_logp, lse[, entropy]) with the gradient coef_logp * (onehot - p) + coef_lse * p."""

    @staticmethod
    def forward(ctx, local_logits, target_1d, active_mask, contract, tp_group, tile, with_entropy, kernels):
        sh = contract.sharding
        z = _masked_scaled(local_logits, contract)
        if kernels is not None:
            m_loc, s_loc = kernels.tile_stats(local_logits, sh.local_vocab_start, sh.real_vocab_size,
                                              (sh.local_vocab_size + tile - 1) // tile)
        else:
            m_loc, s_loc = _local_tile_stats(z, tile)
        m_all, s_all = _gather_tile_stats(m_loc, s_loc, contract, tp_group, tile)
        lse = _merge_tile_partials(m_all, s_all)
        tz, local_idx = _gather_target_logit(z, target_1d, active_mask, contract, tp_group)
        logp = torch.where(active_mask, torch.minimum(tz - lse, torch.zeros_like(lse)) if contract.numerics.clamp_non_positive
                           else tz - lse, torch.zeros_like(lse))
        ctx.save_for_backward(local_logits, lse, local_idx, active_mask)
        ctx.contract, ctx.kernels, ctx.with_entropy, ctx.tp_group = contract, kernels, with_entropy, tp_group
        if with_entropy:
            part = _entropy_partials(z, lse)
            if sh.tp_world_size > 1:
                parts = _AllGatherUneven.apply(part.unsqueeze(-1), contract, tp_group)
                part = torch.zeros_like(part)
                for p in parts:                         # rank order; the same order at every TP degree only per tile
                    part = part + p.squeeze(-1)
            entropy = lse - part
            ctx.mark_non_differentiable(entropy)
            return logp, lse, entropy
        return logp, lse, torch.zeros(0, device=lse.device)

    @staticmethod
    def backward(ctx, g_logp, g_lse, _g_entropy):
        local_logits, lse, local_idx, active_mask = ctx.saved_tensors
        contract, sh = ctx.contract, ctx.contract.sharding
        inv_t = 1.0 / contract.numerics.temperature
        coef_logp = torch.where(active_mask, g_logp.float(), torch.zeros_like(lse))
        has_lse_grad = g_lse is not None and bool((g_lse != 0).any().item())
        coef_lse = g_lse.float() if has_lse_grad else torch.zeros_like(lse)
        if ctx.kernels is not None:
            grad = ctx.kernels.backward(local_logits, lse, coef_logp, coef_lse, local_idx, sh.local_vocab_start,
                                        sh.real_vocab_size, has_lse_grad)
            return grad, None, None, None, None, None, None, None
        z = _masked_scaled(local_logits, contract)
        finite = torch.isfinite(lse)
        p = torch.where(finite.unsqueeze(1), torch.exp(z - torch.where(finite, lse, torch.zeros_like(lse)).unsqueeze(1)),
                        torch.zeros_like(z))
        grad = (coef_lse - coef_logp).unsqueeze(1) * p
        own = local_idx >= 0
        rows = torch.nonzero(own, as_tuple=False).squeeze(1)
        grad[rows, local_idx[rows]] += coef_logp[rows]
        return (grad * inv_t).to(local_logits.dtype), None, None, None, None, None, None, None


class VocabParallelLogprobKernels(Protocol):
    """Device kernel pair a fused backend plugs into :func:`apply_with_kernels`.

    ``tile_stats`` returns fp32 (max, sum-exp) [tokens, local tiles] over the real-vocabulary part of each tile of the
    shard with the contract's in-tile order.  ``backward`` returns the logits gradient in the shard dtype:
    coef_logp * (onehot - p) + coef_lse * p with p = exp(z - lse), zero on padding columns."""

    def tile_stats(self, shard: torch.Tensor, vocab_start: int, real_vocab: int, num_tiles: int
                   ) -> tuple[torch.Tensor, torch.Tensor]: ...

    def backward(self, shard: torch.Tensor, lse: torch.Tensor, coef_logp: torch.Tensor, coef_lse: torch.Tensor,
                 target_local: torch.Tensor, vocab_start: int, real_vocab: int, has_lse_grad: bool) -> torch.Tensor: ...


def _run(local_logits, target_ids, *, contract, tp_group, num_vocab_tiles, validate, deterministic, with_entropy, kernels):
    if not isinstance(contract, LogprobContract):
        raise LogprobContractError("contract must be a LogprobContract")
    if not deterministic and contract.reduction.determinism_scope is DeterminismScope.CROSS_TP_BITWISE:
        raise LogprobContractError("deterministic=False cannot serve a cross_tp_bitwise contract")
    tile = _tile_size(contract, num_vocab_tiles)
    _validate_invocation(local_logits, target_ids, contract, tp_group)
    target_1d = target_ids.reshape(-1).to(device=local_logits.device, dtype=torch.long)
    active = torch.tensor(contract.mask.active_mask, dtype=torch.bool, device=local_logits.device)
    if validate:
        _validate_active_targets(target_1d, active, contract.sharding.real_vocab_size)
        if contract.sharding.tp_world_size > 1:
            _preflight_cross_rank_agreement(contract, tp_group, tile, deterministic)
    logp, lse, ent = _VocabParallelLogprobFunction.apply(local_logits, target_1d, active, contract, tp_group, tile,
                                                         with_entropy, kernels)
    if validate and bool((~torch.isfinite(lse) & active).any().item()):
        raise LogprobContractError("non-finite logsumexp on an active row: logits over the real vocabulary must be finite "
                                   "for every active token")
    return logp, lse, (ent if with_entropy else None)


def apply_with_kernels(local_logits, target_ids, *, contract: LogprobContract, tp_group: Any = None,
                       num_vocab_tiles: int | None = DEFAULT_NUM_VOCAB_TILES, validate: bool = True,
                       kernels: VocabParallelLogprobKernels) -> tuple[torch.Tensor, torch.Tensor]:
    """Contract-checked (selected_logp, lse) through a device kernel pair; transport and merge are this module's."""
    logp, lse, _ = _run(local_logits, target_ids, contract=contract, tp_group=tp_group, num_vocab_tiles=num_vocab_tiles,
                        validate=validate, deterministic=True, with_entropy=False, kernels=kernels)
    return logp, lse


class VocabParallelLogprobOp:
    """Deterministic vocabulary-parallel selected log-prob, driven by a ``LogprobContract``."""

    op_class = "logprob"
    is_batch_invariant = True
    backend_id = BACKEND_ID

    def __init__(self) -> None:
        pass

    def apply(self, local_logits, target_ids, *, contract: LogprobContract, tp_group: Any = None,
              num_vocab_tiles: int | None = DEFAULT_NUM_VOCAB_TILES, validate: bool = True, deterministic: bool = True):
        logp, lse, _ = _run(local_logits, target_ids, contract=contract, tp_group=tp_group, num_vocab_tiles=num_vocab_tiles,
                            validate=validate, deterministic=deterministic, with_entropy=False, kernels=None)
        return logp, lse

    __call__ = apply

    def apply_with_entropy(self, local_logits, target_ids, *, contract: LogprobContract, tp_group: Any = None,
                           num_vocab_tiles: int | None = DEFAULT_NUM_VOCAB_TILES, validate: bool = True,
                           with_entropy_grad: bool = False, deterministic: bool = True):
        """(selected_logp, lse, entropy of the full-vocabulary distribution).  The entropy is a diagnostic and carries
        no gradient."""
        if with_entropy_grad:
            raise LogprobContractError("the entropy is reported without a gradient; differentiate -sum p log p from logits "
                                       "instead")
        return _run(local_logits, target_ids, contract=contract, tp_group=tp_group, num_vocab_tiles=num_vocab_tiles,
                    validate=validate, deterministic=deterministic, with_entropy=True, kernels=None)


__all__ = ["BACKEND_ID", "DEFAULT_NUM_VOCAB_TILES", "VocabParallelLogprobKernels", "VocabParallelLogprobOp",
           "apply_with_kernels"]
