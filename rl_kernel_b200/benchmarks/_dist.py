"""Shared bring-up and timing for the multi-rank benchmarks (one process per GPU under
torch.distributed.run, or a single process)."""
from __future__ import annotations

import os

import torch


def init():
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    return world, rank, dev


def finish(world: int) -> None:
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


_FLUSH = {}


def timed_ms(fn, dev, world: int, iters: int = 10, warmup: int = 3, flush_l2: bool = True) -> float:
    """Median device time of ``fn`` (CUDA events on the launching stream), max over ranks.  Between
    iterations a 256 MiB buffer is rewritten so nothing survives in L2, and the ranks re-align."""
    import torch.distributed as dist

    if flush_l2 and dev not in _FLUSH:
        _FLUSH[dev] = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        if flush_l2:
            _FLUSH[dev].zero_()
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize(dev)
        ts.append(s.elapsed_time(e))
    t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
