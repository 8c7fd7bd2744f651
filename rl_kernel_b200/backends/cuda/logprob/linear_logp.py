"""Fused linear -> selected log-prob device operators, single shard and vocabulary-parallel
(parity: rl_engine/backends/cuda/logprob/linear_logp.py:802-1691).

The LM-head GEMM's epilogue reduces each 128-id vocabulary tile of a row to (max, sum-exp) while
the accumulator is still in tensor memory, so the [N, V] logits are never written.  Under tensor
parallelism every rank owns a slice of the tile list; the tiles travel unchanged (all-gather, or
peer stores from the epilogue) and every rank merges the full list in ascending tile order, which
makes TP = 1, 2, 4, 8 bit-equal.  ``temperature`` is applied to the bf16 logit before the tile
maximum -- one rounding point for the trainer and the rollout engine alike.  A restricted sampling
support (top-k / top-p at rollout time) is replayed either by a per-token threshold
(``min_keep``) inside the same epilogue or from a compact id list
(``sm100_deterministic_top_p_logp_from_local_logits_tp``).
"""
from __future__ import annotations

from typing import Any, Optional

import torch

from rl_kernel_b200.ops.logprob import (_IndexedLogpLseFn, linear_logp, logp_from_logits,  # noqa: F401
                                        replay_logp_from_logits)


def _scalar_temperature(temperature, rows: int) -> float:
    """The kernels take one temperature per call; a per-token tensor must hold one distinct value."""
    if temperature is None:
        return 1.0
    if isinstance(temperature, (int, float)):
        t = float(temperature)
    else:
        t32 = temperature.reshape(-1).float()
        if t32.numel() not in (1, rows):
            raise ValueError("temperature must be positive and scalar or per-token")
        t = float(t32[0].item())
        if t32.numel() > 1 and not bool((t32 == t32[0]).all()):
            raise ValueError("per-token temperatures must be equal within one call; split the batch by temperature")
    if not t > 0:
        raise ValueError("temperature must be positive")
    return t


def _collective(tp_group):
    if tp_group is None:
        return None
    if hasattr(tp_group, "all_gather") and hasattr(tp_group, "world"):
        return tp_group                                                 # already a deterministic collective
    from rl_kernel_b200.distributed.algorithms.collectives import collective_for_group

    import torch.distributed as dist

    if not dist.is_initialized() or dist.get_world_size(tp_group) == 1:
        return None
    return collective_for_group(tp_group)


def _vp_op(weight, *, vocab_start_index, global_vocab_size, real_vocab_size, temperature, tp_group):
    from rl_kernel_b200.ops.distributed import VocabParallelLinearLogpOp

    coll = _collective(tp_group)
    world = coll.world if coll is not None else 1
    padded = int(global_vocab_size) if global_vocab_size else weight.shape[0] * world
    real = padded if real_vocab_size is None or int(real_vocab_size) < 0 else int(real_vocab_size)
    op = VocabParallelLinearLogpOp(real_vocab=real, padded_vocab=padded, collective=coll, temperature=temperature)
    if op.vocab_start != int(vocab_start_index):
        raise ValueError(f"vocab_start_index={vocab_start_index} does not match the even partition "
                         f"(rank {op.rank} of {op.world} starts at {op.vocab_start})")
    return op


def sm100_deterministic_linear_logp(hidden, lm_head_weight, target_ids, bias: Optional[torch.Tensor] = None, *,
                                    temperature=None, return_logits: bool = False, real_vocab_size: int = -1,
                                    min_keep: Optional[torch.Tensor] = None):
    """(logp, lse[, logits]) for one vocabulary shard holding the whole vocabulary; the strict entry both
    the trainer and the rollout engine call with identical bytes."""
    if bias is not None:
        raise ValueError("the fused LM head has no bias term (Qwen3 has none)")
    t = _scalar_temperature(temperature, target_ids.numel())
    w = lm_head_weight if real_vocab_size is None or real_vocab_size < 0 else lm_head_weight[:real_vocab_size]
    lead = hidden.shape[:-1]
    h2 = hidden.reshape(-1, hidden.shape[-1]).contiguous()
    tg = target_ids.reshape(-1).to(device=h2.device, dtype=torch.long)
    if tg.numel() != h2.shape[0]:
        raise ValueError("target_ids must contain one id per hidden row")
    from rl_kernel_b200.backends import native as nv

    rows, V = h2.shape[0], w.shape[0]
    ntile = (V + 127) // 128
    stats = torch.empty(rows, ntile, 2, device=h2.device, dtype=torch.float32)
    tl = torch.zeros(rows, device=h2.device, dtype=torch.float32)
    logits = torch.empty(rows, V, device=h2.device, dtype=torch.bfloat16) if return_logits else None
    mk = None if min_keep is None else min_keep.reshape(-1).float().contiguous()
    with torch.no_grad():
        nv.lmhead_logp_stats(h2, w.contiguous(), tg, stats, tl, vocab_start=0, inv_temp=1.0 / t, logits_out=logits, min_keep=mk)
        logp = torch.empty(rows, device=h2.device, dtype=torch.float32)
        lse = torch.empty(rows, device=h2.device, dtype=torch.float32)
        nv.logp_merge(stats, tl, logp, lse)
    out = (logp.reshape(lead), lse.reshape(lead))
    return out + (logits.float().reshape(*lead, V),) if return_logits else out


def sm100_deterministic_linear_logp_tp(hidden, lm_head_weight, target_ids, bias: Optional[torch.Tensor] = None, *,
                                       vocab_start_index: int, global_vocab_size: int, real_vocab_size: int = -1,
                                       temperature=None, tp_group: Any = None):
    """Vocabulary-parallel (logp, lse): ``lm_head_weight`` is this rank's [V_pad / tp, H] shard.  Differentiable
    in ``hidden`` and the shard when either requires grad."""
    if bias is not None:
        raise ValueError("the fused LM head has no bias term (Qwen3 has none)")
    t = _scalar_temperature(temperature, target_ids.numel())
    op = _vp_op(lm_head_weight, vocab_start_index=vocab_start_index, global_vocab_size=global_vocab_size,
                real_vocab_size=real_vocab_size, temperature=t, tp_group=tp_group)
    logp = op(hidden, lm_head_weight, target_ids)
    return logp, op.last_lse.view(target_ids.shape) if getattr(op, "last_lse", None) is not None else None


def sm100_deterministic_logp_from_local_logits_tp(local_logits, target_ids, *, vocab_start_index: int,
                                                  global_vocab_size: int, real_vocab_size: int = -1, temperature=None,
                                                  tp_group: Any = None, min_keep: Optional[torch.Tensor] = None):
    """(logp, lse) from this rank's materialised logits shard [N, V_local] without recomputing the GEMM."""
    from rl_kernel_b200.backends import native as nv

    t = _scalar_temperature(temperature, target_ids.numel())
    coll = _collective(tp_group)
    world = coll.world if coll is not None else 1
    lg = local_logits.reshape(-1, local_logits.shape[-1]).contiguous()
    if lg.dtype != torch.bfloat16 or not lg.is_cuda:
        raise TypeError("strict TP logits log-prob requires CUDA BF16 local logits")
    rows, vl = lg.shape
    if vl * world != int(global_vocab_size) or int(vocab_start_index) % 128:
        raise ValueError("local logits must be an even, 128-aligned partition of global_vocab_size")
    real = int(global_vocab_size) if real_vocab_size is None or int(real_vocab_size) < 0 else int(real_vocab_size)
    keep_cols = max(0, min(vl, real - int(vocab_start_index)))
    tg = target_ids.reshape(-1).to(device=lg.device, dtype=torch.long).contiguous()
    ntile = int(global_vocab_size) // 128
    with torch.no_grad():
        stats = torch.empty(rows, ntile, 2, device=lg.device, dtype=torch.float32)
        stats[..., 0] = float("-inf")
        stats[..., 1] = 0
        tl = torch.zeros(rows, device=lg.device, dtype=torch.float32)
        mk = None if min_keep is None else min_keep.reshape(-1).float().contiguous()
        if keep_cols:
            nv.logits_tile_stats(lg[:, :keep_cols], tg, stats, tl, vocab_start=int(vocab_start_index), inv_temp=1.0 / t,
                                 min_keep=mk)
        if world > 1:
            per = ntile // world
            mine = stats[:, coll.rank * per:(coll.rank + 1) * per].contiguous()
            stats = coll.all_gather(mine).permute(1, 0, 2, 3).reshape(rows, ntile, 2).contiguous()
            tl = coll.all_gather(tl).sum(0)
        logp = torch.empty(rows, device=lg.device, dtype=torch.float32)
        lse = torch.empty(rows, device=lg.device, dtype=torch.float32)
        nv.logp_merge(stats, tl, logp, lse)
    return logp.reshape(target_ids.shape), lse.reshape(target_ids.shape)


def sm100_deterministic_top_p_logp_from_local_logits_tp(local_logits, target_ids, replay_ids, replay_logprobs, *,
                                                        vocab_start_index: int, global_vocab_size: int,
                                                        real_vocab_size: int = -1, temperature=None, tp_group: Any = None):
    """Score a compact top-p replay set with the dense kernels' reduction order (inference only).
    Entries of ``replay_ids`` whose ``replay_logprobs`` is not finite are not part of the support."""
    if torch.is_grad_enabled() and local_logits.requires_grad:
        raise RuntimeError("compact top-p local-logits logp is inference-only")
    if local_logits.ndim != 2 or local_logits.dtype != torch.bfloat16:
        raise TypeError("strict TP top-p logits logp requires 2-D BF16 local logits")
    if replay_ids.ndim != 2 or replay_logprobs.shape != replay_ids.shape:
        raise ValueError("top-p replay ids/logprobs must be aligned 2-D tensors")
    if replay_ids.size(0) != local_logits.size(0):
        raise ValueError("top-p replay rows must align with local logits")
    if replay_ids.size(1) > 64:
        raise ValueError("top-p replay width exceeds the compact kernel limit of 64")
    real = int(global_vocab_size) if real_vocab_size is None or int(real_vocab_size) < 0 else int(real_vocab_size)
    if not 0 < real <= int(global_vocab_size):
        raise ValueError(f"invalid real_vocab_size={real} for padded vocab={global_vocab_size}")
    t = _scalar_temperature(temperature, target_ids.numel())
    ids = replay_ids.to(device=local_logits.device, dtype=torch.long)
    ids = torch.where(torch.isfinite(replay_logprobs.to(ids.device)) & (ids < real), ids, torch.full_like(ids, -1))
    return replay_logp_from_logits(local_logits, target_ids, ids, t, vocab_start=int(vocab_start_index), return_lse=True,
                                   collective=_collective(tp_group))


class FusedLinearLogpSM100Op:
    """``op(hidden, lm_head_weight, target_ids, bias=None, *, tp_group=None, vocab_start_index=0,
    global_vocab_size=None)`` -> fp32 log-prob; differentiable."""

    is_fused_logp = True
    is_batch_invariant = True
    backward_impl = "native"
    backend_id = "b200-tcgen05"

    def __init__(self, temperature: float = 1.0) -> None:
        self.temperature = temperature

    def apply(self, hidden, lm_head_weight, target_ids, bias: Optional[torch.Tensor] = None, *, tp_group: Any = None,
              vocab_start_index: int = 0, global_vocab_size: Optional[int] = None, min_keep=None):
        if bias is not None:
            raise ValueError("the fused LM head has no bias term (Qwen3 has none)")
        coll = _collective(tp_group)
        if coll is None:
            return linear_logp(hidden, lm_head_weight, target_ids, self.temperature, min_keep=min_keep)
        if min_keep is not None:
            raise NotImplementedError("restricted support under vocabulary parallelism: use "
                                      "sm100_deterministic_logp_from_local_logits_tp(min_keep=...)")
        op = _vp_op(lm_head_weight, vocab_start_index=vocab_start_index, global_vocab_size=global_vocab_size,
                    real_vocab_size=-1, temperature=self.temperature, tp_group=coll)
        return op(hidden, lm_head_weight, target_ids)

    __call__ = apply


# the reference's Hopper spellings
FusedLinearLogpSM90Op = FusedLinearLogpSM100Op
sm90_deterministic_linear_logp = sm100_deterministic_linear_logp
sm90_deterministic_linear_logp_tp = sm100_deterministic_linear_logp_tp
sm90_deterministic_logp_from_local_logits_tp = sm100_deterministic_logp_from_local_logits_tp
sm90_deterministic_top_p_logp_from_local_logits_tp = sm100_deterministic_top_p_logp_from_local_logits_tp
