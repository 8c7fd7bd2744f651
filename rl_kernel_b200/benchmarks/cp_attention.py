"""Context-parallel causal attention forward + backward (GQA 32 q / 8 kv heads, head_dim 128) with
the KV / Q / dO exchange inside the kernels, over all ranks of the job (zigzag layout).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29552 -m rl_kernel_b200.benchmarks.cp_attention --seqs 8192 32768 131072

One JSON line per sequence length: device ms for forward and for backward (delta + dQ + dK/dV),
max over ranks, and the causal TFLOP/s per GPU.  A single process measures the CP = 1 kernels.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from rl_kernel_b200.benchmarks._dist import finish, init, timed_ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqs", type=int, nargs="*", default=[8192, 32768])
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    world, rank, dev = init()
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.models.qwen3.engine import train_tiles

    D, Hq, Hkv = 128, a.hq, a.hkv
    coll = None
    if world > 1:
        from rl_kernel_b200.distributed.cp_attention import CPAttention
        from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

        coll = SymmetricMemoryCollective(None, dev, frame_bytes=1 << 20)
    for S in a.seqs:
        Sl = S // world
        g = torch.Generator(device=dev).manual_seed(rank)
        q = torch.randn(Sl, Hq * D, device=dev, generator=g).to(torch.bfloat16)
        k = torch.randn(Sl, Hkv * D, device=dev, generator=g).to(torch.bfloat16)
        v = torch.randn(Sl, Hkv * D, device=dev, generator=g).to(torch.bfloat16)
        do = torch.randn(Sl, Hq * D, device=dev, generator=g).to(torch.bfloat16)
        out = torch.empty_like(q)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        if world > 1:
            cp = CPAttention(coll, dev, num_q_heads=Hq, num_kv_heads=Hkv, max_local_tokens=Sl, layout="zigzag")
            b = cp.bufs
            b.local("k").copy_(k); b.local("v").copy_(v); b.local("q").copy_(q); b.local("do").copy_(do)
            fwd = lambda: cp.forward_inplace(b.local("q"), out, b.local("lse"), 1, S)  # noqa: E731

            def bwd():
                nv.attn_bwd_delta(out, b.local("do"), b.local("delta"), Sl, Hq)
                cp.backward_inplace(dq, dk, dv, 1, S)
        else:
            tiles, kvt = train_tiles(1, S, Hq, Hkv, D, dev)
            lse, delta = torch.empty(S, Hq, device=dev), torch.empty(S, Hq, device=dev)
            sc = 1 / math.sqrt(D)
            fwd = lambda: nv.attn_fwd(q, [k], [v], out, lse, tiles, sc)  # noqa: E731

            def bwd():
                nv.attn_bwd_delta(out, do, delta, S, Hq)
                nv.attn_bwd_dq(q, do, k, v, lse, delta, dq, tiles, sc)
                nv.attn_bwd_dkv(q, do, k, v, lse, delta, dk, dv, kvt, sc)
        t_f = timed_ms(fwd, dev, world, a.iters, warmup=2)
        t_b = timed_ms(bwd, dev, world, a.iters, warmup=2)
        flops = 4.0 * Hq * D * S * S / 2
        status = ext.poll_status(dev)
        if rank == 0:
            print(json.dumps({"bench": "cp_attention", "cp": world, "seq": S, "fwd_ms": t_f, "bwd_ms": t_b,
                              "fwd_tflops_per_gpu": flops / t_f / 1e9 / world,
                              "bwd_tflops_per_gpu": 2.5 * flops / t_b / 1e9 / world, "device_status": status}), flush=True)
        if world > 1:
            del cp
    finish(world)


if __name__ == "__main__":
    main()
