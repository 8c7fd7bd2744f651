"""Device timing helpers: CUDA events on the launching stream, max over ranks, L2 flush."""
from __future__ import annotations

from typing import Callable

import torch

L2_BYTES = 126 * 1024 * 1024


class L2Flusher:
    """Writes a buffer larger than the 126 MB L2 so the next kernel starts cold."""

    def __init__(self, device: torch.device, nbytes: int = 2 * L2_BYTES):
        self.buf = torch.empty(nbytes // 4, dtype=torch.int32, device=device)

    def __call__(self) -> None:
        self.buf.zero_()


def time_cuda(fn: Callable[[], object], *, warmup: int = 3, iters: int = 10,
              flush: L2Flusher | None = None) -> list[float]:
    """Milliseconds per call, one CUDA-event pair per iteration, synchronised on both sides."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush is not None:
            flush()
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        out.append(s.elapsed_time(e))
    return out


def max_over_ranks(value_ms: float, group=None) -> float:
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return value_ms
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    t = torch.tensor([value_ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
