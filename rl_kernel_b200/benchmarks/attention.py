"""Causal GQA attention forward/backward micro-benchmark on the sm_100a kernels.

    python -m rl_kernel_b200.benchmarks.attention --batch 2 --seq 2048 [--bwd] [--decode]

Prints one JSON line: device ms per call (CUDA events, warm-up excluded) and causal TFLOP/s.
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from rl_kernel_b200.backends import native as nv
from rl_kernel_b200.models.qwen3.engine import train_tiles


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--hq", type=int, default=32)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--decode", action="store_true", help="single-token decode at position seq-1")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    D, B, S, Hq, Hkv = 128, a.batch, a.seq, a.hq, a.hkv
    T = B * S
    scale = 1.0 / math.sqrt(D)
    k = torch.randn(T, Hkv * D, device=dev).bfloat16()
    v = torch.randn(T, Hkv * D, device=dev).bfloat16()
    if a.decode:
        G = Hq // Hkv
        q = torch.randn(B * Hq + 128, D, device=dev).bfloat16()
        o = torch.zeros_like(q)
        b = torch.arange(B).view(-1, 1)
        hk = torch.arange(Hkv).view(1, -1)
        z = torch.zeros(B, Hkv, dtype=torch.long)
        row0 = b * Hq + hk * G + z
        tiles = torch.stack([row0, z, z + G, b * S + z, hk * D + z, z + S - 1, z, z + S, row0, z + 1, z, z],
                            dim=-1).reshape(-1, 12).to(torch.int32).to(dev).contiguous()
        run = lambda: nv.attn_fwd(q, [k], [v], o, None, tiles, scale, decode=True)  # noqa: E731
        flops = 0.0
        nbytes = 2 * T * Hkv * D * 2
    else:
        q = torch.randn(T, Hq * D, device=dev).bfloat16()
        o = torch.zeros_like(q)
        lse = torch.zeros(T, Hq, device=dev)
        tiles, kvtiles = train_tiles(B, S, Hq, Hkv, D, dev)
        flops = 4.0 * B * Hq * D * S * S / 2
        nbytes = 0
        if a.bwd:
            do = torch.randn_like(q)
            delta = torch.empty(T, Hq, device=dev)
            dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
            nv.attn_fwd(q, [k], [v], o, lse, tiles, scale)
            flops *= 2.5

            def run():
                nv.attn_bwd_delta(o, do, delta, T, Hq)
                nv.attn_bwd_dq(q, do, k, v, lse, delta, dq, tiles, scale)
                nv.attn_bwd_dkv(q, do, k, v, lse, delta, dk, dv, kvtiles, scale)
        else:
            run = lambda: nv.attn_fwd(q, [k], [v], o, lse, tiles, scale)  # noqa: E731
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.iters):
        run()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / a.iters
    print(json.dumps({"mode": "decode" if a.decode else ("bwd" if a.bwd else "fwd"), "batch": B, "seq": S,
                      "ms": ms, "tflops": flops / ms / 1e9 if flops else None,
                      "kv_gbs": nbytes / ms / 1e6 if nbytes else None}))


if __name__ == "__main__":
    main()
