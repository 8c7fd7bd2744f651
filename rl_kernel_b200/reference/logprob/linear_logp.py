"""Fused linear -> selected log-prob in PyTorch, single shard and tensor parallel
(parity: rl_engine/reference/logprob/linear_logp.py:21-800).

``NativeLinearLogpOp`` never keeps more than ``chunk_size`` rows of logits: logits are the
batch-invariant GEMM of a row chunk rounded to bf16, reduced at once to tile statistics.  The tensor
parallel form computes each rank's tile statistics and target logit for its vocabulary shard,
moves them by all-gather and merges the complete tile list in ascending order; its backward
recomputes the shard's logits chunk by chunk, forms d(logits) = g * (onehot - p) / T, and
multiplies into d(hidden) (summed over ranks in the fixed tree of the deterministic collective)
and d(weight shard) (local).
"""
from __future__ import annotations

import os
from typing import Any

import torch

from rl_kernel_b200.distributed.algorithms.collectives import balanced_tree_sum
from rl_kernel_b200.reference.gemm.det_gemm import det_gemm_reference
from rl_kernel_b200.reference.logprob.tile_logp import (TILE, NativeLinearLogpOp, _target_z, merge_tile_stats,  # noqa: F401
                                                        tile_stats_reference)


def _env_flag(name: str) -> bool:
    return os.environ.get(name, "").strip().lower() in ("1", "true", "yes", "on")


def _validate_tp_targets_enabled() -> bool:
    return _env_flag("RL_KERNEL_VALIDATE_TP_TARGETS")


def _require_distributed_initialized():
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        raise RuntimeError("tensor-parallel linear log-prob needs an initialised torch.distributed process group")
    return dist


def _tensor_parallel_world_size(tp_group: Any) -> int:
    if tp_group is None:
        return 1
    if hasattr(tp_group, "world"):
        return int(tp_group.world)
    return _require_distributed_initialized().get_world_size(group=tp_group)


def _tensor_parallel_rank(tp_group: Any) -> int:
    if tp_group is None:
        return 0
    if hasattr(tp_group, "rank") and hasattr(tp_group, "world"):
        return int(tp_group.rank)
    return _require_distributed_initialized().get_rank(group=tp_group)


def should_use_tensor_parallel_linear_logp(tp_group: Any, lm_head_weight: torch.Tensor, global_vocab_size: int | None) -> bool:
    """True when the weight is a proper shard of a larger vocabulary held by a group of more than one rank."""
    if tp_group is None or _tensor_parallel_world_size(tp_group) == 1:
        return False
    return global_vocab_size is None or int(global_vocab_size) > lm_head_weight.shape[0]


def _validate_tp_vocab_partition(*, tp_group: Any, vocab_start_index: int, local_vocab_size: int,
                                 global_vocab_size: int | None) -> int:
    """Check that every rank holds the even shard its rank implies; returns the global (padded) vocabulary size."""
    world, rank = _tensor_parallel_world_size(tp_group), _tensor_parallel_rank(tp_group)
    total = int(global_vocab_size) if global_vocab_size else local_vocab_size * world
    if total != local_vocab_size * world:
        raise ValueError(f"global_vocab_size={total} is not tp_world_size={world} x local shard {local_vocab_size}")
    if int(vocab_start_index) != rank * local_vocab_size:
        raise ValueError(f"vocab_start_index={vocab_start_index} does not match rank {rank}'s shard start {rank * local_vocab_size}")
    if int(vocab_start_index) % TILE:
        raise ValueError(f"vocabulary shards must start on {TILE}-id tile boundaries; got {vocab_start_index}")
    return total


def _validate_global_targets(target_ids: torch.Tensor, global_vocab_size: int) -> None:
    if target_ids.numel() and bool(((target_ids < 0) | (target_ids >= global_vocab_size)).any()):
        bad = target_ids[(target_ids < 0) | (target_ids >= global_vocab_size)]
        raise ValueError(f"target_ids outside [0, {global_vocab_size}): {bad[:8].tolist()}")


def _gather(t: torch.Tensor, tp_group: Any) -> torch.Tensor:
    """[...] -> [world, ...] in rank order through a deterministic collective or a torch process group."""
    if hasattr(tp_group, "all_gather") and hasattr(tp_group, "world"):
        return tp_group.all_gather(t)
    dist = _require_distributed_initialized()
    out = [torch.empty_like(t) for _ in range(dist.get_world_size(group=tp_group))]
    dist.all_gather(out, t.contiguous(), group=tp_group)
    return torch.stack(out)


def _chunked_local_linear_logp_stats(hidden, weight_shard, target_ids, *, vocab_start_index: int, n_tiles_total: int,
                                     inv_temp: float, chunk_size: int):
    """(stats [rows, n_tiles_total, 2], target_z [rows]) of this shard, ``chunk_size`` rows of logits at a time."""
    rows = hidden.shape[0]
    stats = torch.zeros(rows, n_tiles_total, 2, device=hidden.device)
    stats[..., 0] = float("-inf")
    tz = torch.zeros(rows, device=hidden.device)
    for r0 in range(0, rows, chunk_size):
        r1 = min(rows, r0 + chunk_size)
        logits = det_gemm_reference(hidden[r0:r1], weight_shard)
        st = tile_stats_reference(logits, vocab_start=vocab_start_index, inv_temp=inv_temp, n_tiles_total=n_tiles_total)
        t0, nt = vocab_start_index // TILE, (weight_shard.shape[0] + TILE - 1) // TILE
        stats[r0:r1, t0:t0 + nt] = st[:, t0:t0 + nt]
        z, own = _target_z(logits, target_ids[r0:r1], vocab_start_index, inv_temp)
        tz[r0:r1] = torch.where(own, z, torch.zeros_like(z))
    return stats, tz


def _merge_tp_local_logp(local_stats: torch.Tensor, local_target: torch.Tensor, *, tp_group: Any, vocab_start_index: int,
                         local_vocab_size: int):
    """Gather every shard's tiles and target contribution in rank order and merge the complete list."""
    world = _tensor_parallel_world_size(tp_group)
    if world == 1:
        return merge_tile_stats(local_stats, local_target)
    t0, nt = vocab_start_index // TILE, (local_vocab_size + TILE - 1) // TILE
    mine = local_stats[:, t0:t0 + nt].contiguous()
    tiles = _gather(mine, tp_group)                                   # [world, rows, nt, 2]
    stats = tiles.permute(1, 0, 2, 3).reshape(local_stats.shape[0], world * nt, 2)
    target = _gather(local_target, tp_group).sum(0)                   # one non-zero term per row
    return merge_tile_stats(stats, target)


def _deterministic_tp_all_reduce_(tensor: torch.Tensor, tp_group: Any) -> torch.Tensor:
    """Sum over the TP group in the balanced binary tree (fp32 nodes rounded to the tensor's dtype)."""
    if _tensor_parallel_world_size(tp_group) == 1:
        return tensor
    if hasattr(tp_group, "all_reduce_"):
        return tp_group.all_reduce_(tensor)
    parts = _gather(tensor, tp_group)
    tensor.copy_(balanced_tree_sum(list(parts.unbind(0)), tensor.dtype))
    return tensor


def chunked_linear_logp_backward(hidden, weight, target_ids, lse, grad_logp, *, vocab_start_index: int = 0,
                                 inv_temp: float = 1.0, chunk_size: int = 4096):
    """(d hidden, d weight) of one vocabulary shard: logits recomputed per row chunk, rows summed in ascending order."""
    rows, H = hidden.shape
    dh = torch.zeros(rows, H, device=hidden.device)
    dw = torch.zeros(weight.shape, device=hidden.device)
    for r0 in range(0, rows, chunk_size):
        r1 = min(rows, r0 + chunk_size)
        logits = det_gemm_reference(hidden[r0:r1], weight).float()
        z = logits * inv_temp
        p = torch.exp(z - lse[r0:r1, None])
        local = target_ids[r0:r1] - vocab_start_index
        own = (local >= 0) & (local < weight.shape[0])
        d = -p * grad_logp[r0:r1, None]
        idx = torch.nonzero(own, as_tuple=False).squeeze(1)
        d[idx, local[idx]] += grad_logp[r0:r1][idx]
        d = (d * inv_temp).to(hidden.dtype).float()                    # the device path rounds d(logits) to bf16
        dh[r0:r1] = d @ weight.float()
        dw += d.t() @ hidden[r0:r1].float()
    return dh.to(hidden.dtype), dw.to(weight.dtype)


def tensor_parallel_linear_logp_backward(hidden, weight_shard, target_ids, lse, grad_logp, *, tp_group: Any,
                                         vocab_start_index: int, inv_temp: float = 1.0, chunk_size: int = 4096):
    dh, dw = chunked_linear_logp_backward(hidden, weight_shard, target_ids, lse, grad_logp,
                                          vocab_start_index=vocab_start_index, inv_temp=inv_temp, chunk_size=chunk_size)
    return _deterministic_tp_all_reduce_(dh, tp_group), dw


class _TensorParallelLinearLogpFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight_shard, target_ids, tp_group, vocab_start_index, global_vocab_size, inv_temp, chunk_size):
        n_tiles = (global_vocab_size + TILE - 1) // TILE
        stats, tz = _chunked_local_linear_logp_stats(hidden, weight_shard, target_ids, vocab_start_index=vocab_start_index,
                                                     n_tiles_total=n_tiles, inv_temp=inv_temp, chunk_size=chunk_size)
        logp, lse = _merge_tp_local_logp(stats, tz, tp_group=tp_group, vocab_start_index=vocab_start_index,
                                         local_vocab_size=weight_shard.shape[0])
        ctx.save_for_backward(hidden, weight_shard, target_ids, lse)
        ctx.meta = (tp_group, vocab_start_index, inv_temp, chunk_size)
        ctx.mark_non_differentiable(lse)
        return logp, lse

    @staticmethod
    def backward(ctx, g_logp, _g_lse):
        hidden, weight_shard, target_ids, lse = ctx.saved_tensors
        tp_group, start, inv_temp, chunk = ctx.meta
        dh, dw = tensor_parallel_linear_logp_backward(hidden, weight_shard, target_ids, lse, g_logp.float(), tp_group=tp_group,
                                                      vocab_start_index=start, inv_temp=inv_temp, chunk_size=chunk)
        return dh, dw, None, None, None, None, None, None


def tensor_parallel_linear_logp(hidden: torch.Tensor, lm_head_weight: torch.Tensor, target_ids: torch.Tensor,
                                bias: torch.Tensor | None = None, *, tp_group: Any, vocab_start_index: int,
                                global_vocab_size: int | None = None, temperature: float = 1.0, chunk_size: int = 4096,
                                return_lse: bool = False):
    """Vocabulary-parallel fused linear log-prob; ``lm_head_weight`` is this rank's [V / tp, H] shard."""
    if bias is not None:
        raise ValueError("the fused LM head has no bias term")
    total = _validate_tp_vocab_partition(tp_group=tp_group, vocab_start_index=vocab_start_index,
                                         local_vocab_size=lm_head_weight.shape[0], global_vocab_size=global_vocab_size)
    shp = target_ids.shape
    h = hidden.reshape(-1, hidden.shape[-1])
    tg = target_ids.reshape(-1).to(h.device).long()
    if _validate_tp_targets_enabled():
        _validate_global_targets(tg, total)
    logp, lse = _TensorParallelLinearLogpFunction.apply(h, lm_head_weight, tg, tp_group, int(vocab_start_index), total,
                                                        1.0 / temperature, chunk_size)
    return (logp.view(shp), lse.view(shp)) if return_lse else logp.view(shp)


__all__ = ["NativeLinearLogpOp", "chunked_linear_logp_backward", "should_use_tensor_parallel_linear_logp",
           "tensor_parallel_linear_logp", "tensor_parallel_linear_logp_backward"]
