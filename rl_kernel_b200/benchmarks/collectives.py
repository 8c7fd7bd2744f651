"""Fixed-order all-reduce / all-gather on symmetric memory against NCCL, 256 KiB - 64 MiB bf16.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29551 -m rl_kernel_b200.benchmarks.collectives

One JSON line per size: device ms (median, max over ranks, L2 flushed) and bus bandwidth
(all-reduce: 2 (W-1)/W * bytes / t; all-gather: (W-1)/W * total bytes / t).
"""
from __future__ import annotations

import argparse
import json

import torch

from rl_kernel_b200.benchmarks._dist import finish, init, timed_ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes-kib", type=int, nargs="*", default=[256, 1024, 4096, 16384, 65536])
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    world, rank, dev = init()
    import torch.distributed as dist

    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

    coll = SymmetricMemoryCollective(None, dev, frame_bytes=max(a.sizes_kib) * 1024 * max(1, world))
    for kib in a.sizes_kib:
        n = kib * 1024 // 2
        x = torch.randn(n, device=dev).to(torch.bfloat16)
        y = x.clone()
        t_ar = timed_ms(lambda: coll.all_reduce_(x), dev, world, a.iters)
        t_nccl = timed_ms(lambda: dist.all_reduce(y), dev, world, a.iters)
        t_ag = timed_ms(lambda: coll.all_gather(x), dev, world, a.iters)
        out = torch.empty(world * n, device=dev, dtype=torch.bfloat16)
        t_ag_nccl = timed_ms(lambda: dist.all_gather_into_tensor(out, y), dev, world, a.iters)
        if rank == 0:
            b = kib * 1024
            print(json.dumps({"bench": "collectives", "world": world, "kib": kib,
                              "all_reduce_ms": t_ar, "nccl_all_reduce_ms": t_nccl,
                              "all_reduce_busbw_gbs": 2 * (world - 1) / world * b / t_ar / 1e6,
                              "nccl_all_reduce_busbw_gbs": 2 * (world - 1) / world * b / t_nccl / 1e6,
                              "all_gather_ms": t_ag, "nccl_all_gather_ms": t_ag_nccl,
                              "all_gather_busbw_gbs": (world - 1) * b / t_ag / 1e6}), flush=True)
    status = ext.poll_status(dev)
    if rank == 0:
        print(json.dumps({"bench": "collectives", "device_status": status}))
    finish(world)


if __name__ == "__main__":
    main()
