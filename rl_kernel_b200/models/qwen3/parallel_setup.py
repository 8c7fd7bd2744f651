"""Builds the ParallelContext of this process from the torch.distributed world: ranks are laid out
TP-fastest ([cp][tp]), so TP peers are adjacent GPUs and CP peers are ``tp`` apart."""
from __future__ import annotations

import torch

from rl_kernel_b200.models.qwen3.engine import ParallelContext


def build_parallel_context(tp: int, cp: int, device: torch.device) -> ParallelContext:
    import torch.distributed as dist

    if tp * cp == 1 or not dist.is_initialized():
        return ParallelContext()
    world, rank = dist.get_world_size(), dist.get_rank()
    if world != tp * cp:
        raise ValueError(f"world {world} != tp {tp} x cp {cp}")
    from rl_kernel_b200.distributed import create_deterministic_collective

    tp_rank, cp_rank = rank % tp, rank // tp
    tp_group = cp_group = None
    for c in range(cp):
        g = dist.new_group(list(range(c * tp, (c + 1) * tp)))
        if c == cp_rank:
            tp_group = g
    for t in range(tp):
        g = dist.new_group([t + c * tp for c in range(cp)])
        if t == tp_rank:
            cp_group = g
    coll = create_deterministic_collective(tp_group, device) if tp > 1 else None
    cp_coll = create_deterministic_collective(cp_group, device) if cp > 1 else None
    ctx = ParallelContext(tp_rank, tp, cp_rank, cp, coll, cp_coll)
    ctx.tp_group, ctx.cp_group = tp_group, cp_group
    return ctx
