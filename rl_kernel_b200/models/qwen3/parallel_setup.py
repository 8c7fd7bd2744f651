"""Builds the ParallelContext of this process from the torch.distributed world: ranks are laid out
TP-fastest ([dp][cp][tp]), so TP peers are adjacent GPUs, CP peers are ``tp`` apart and data
parallel replicas ``tp * cp`` apart."""
from __future__ import annotations

import torch

from rl_kernel_b200.models.qwen3.engine import ParallelContext


def cp_frame_bytes_for(spec, tp: int, tokens_per_rank: int) -> int:
    """Frame size for the context-parallel collective: the largest tensor the canonical weight-gradient
    path gathers is one rank's gate/up gradient [tokens_per_rank, 2 * intermediate / tp] in bf16; a frame
    that holds it lets the gather run as one kernel (larger payloads still work, in frame-sized pieces)."""
    need = int(tokens_per_rank) * 2 * (spec.intermediate_size // max(1, tp)) * 2
    return max(256 << 20, (need + (1 << 20) - 1) >> 20 << 20)


def build_parallel_context(tp: int, cp: int, device: torch.device, dp: int = 1, *,
                           cp_frame_bytes: int | None = None) -> ParallelContext:
    import torch.distributed as dist

    if tp * cp * dp == 1 or not dist.is_initialized():
        return ParallelContext()
    world, rank = dist.get_world_size(), dist.get_rank()
    if world != tp * cp * dp:
        raise ValueError(f"world {world} != tp {tp} x cp {cp} x dp {dp}")
    from rl_kernel_b200.distributed import create_deterministic_collective

    tp_rank, cp_rank, dp_rank = rank % tp, (rank // tp) % cp, rank // (tp * cp)
    tp_group = cp_group = dp_group = None
    # every rank must create every group, in the same order
    for d in range(dp):
        for c in range(cp):
            g = dist.new_group([d * tp * cp + c * tp + t for t in range(tp)]) if tp > 1 else None
            if d == dp_rank and c == cp_rank:
                tp_group = g
    for d in range(dp):
        for t in range(tp):
            g = dist.new_group([d * tp * cp + c * tp + t for c in range(cp)]) if cp > 1 else None
            if d == dp_rank and t == tp_rank:
                cp_group = g
    for c in range(cp):
        for t in range(tp):
            g = dist.new_group([d * tp * cp + c * tp + t for d in range(dp)]) if dp > 1 else None
            if c == cp_rank and t == tp_rank:
                dp_group = g
    coll = create_deterministic_collective(tp_group, device) if tp > 1 else None
    cp_kw = {"frame_bytes": int(cp_frame_bytes)} if cp_frame_bytes else {}
    cp_coll = create_deterministic_collective(cp_group, device, **cp_kw) if cp > 1 else None
    ctx = ParallelContext(tp_rank, tp, cp_rank, cp, coll, cp_coll)
    ctx.tp_group, ctx.cp_group, ctx.dp_group = tp_group, cp_group, dp_group
    if dp > 1:
        ctx.dp_rank, ctx.dp_size = dp_rank, dp
        ctx.dp_collective = create_deterministic_collective(dp_group, device)
    return ctx
