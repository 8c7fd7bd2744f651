"""Bandwidth-bound operators against the measured copy bandwidth: stand-alone RoPE, RMSNorm (with and without the fused
residual add), SwiGLU, the pack / unpack row mover and log-prob from logits (dense, with a support threshold, and the compact
id-list replay).  Inputs are larger than L2 (126 MB); CUDA events; median of ``--iters``.

    python -m rl_kernel_b200.benchmarks.elementwise --rows 65536
    python -m rl_kernel_b200.benchmarks.elementwise --rows 16384 --only rope        # small case for an ncu capture
"""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=65536)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", default="")
    ap.add_argument("--peak-gbs", type=float, default=6552.0, help="measured copy bandwidth of the device")
    a = ap.parse_args(argv)
    from rl_kernel_b200.ops.activation import swiglu
    from rl_kernel_b200.ops.logprob import logp_from_logits, replay_logp_from_logits
    from rl_kernel_b200.ops.norm import rms_norm
    from rl_kernel_b200.ops.packing import PackOp
    from rl_kernel_b200.ops.rope import rope

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    T = a.rows
    rows = []

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(a.iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        return sorted(ts)[len(ts) // 2]

    def add(name, nbytes, fn):
        if a.only and a.only != name:
            return
        with torch.no_grad():
            ms = timed(fn)
        rows.append({"op": name, "ms": ms, "algorithmic_gb": nbytes / 1e9, "gb_s": nbytes / ms / 1e6, "fraction_of_copy_peak": nbytes / ms / 1e6 / a.peak_gbs})

    x = torch.randn(T, 4096, device=dev, generator=g).bfloat16()              # 512 MB at 65536 rows
    w = torch.ones(4096, device=dev).bfloat16()
    qh = x.view(T, 32, 128)
    pos = (torch.arange(T, device=dev) % 4096)
    add("rope", 2 * x.numel() * 2, lambda: rope(qh.transpose(0, 1), pos, max_position=4096))
    add("rms_norm", 2 * x.numel() * 2, lambda: rms_norm(x, w))
    gate, up = x, torch.randn(T, 4096, device=dev, generator=g).bfloat16()
    add("swiglu", 3 * x.numel() * 2, lambda: swiglu(gate, up))
    mask = torch.rand(T // 128, 128, device=dev, generator=g) > 0.25
    xp = x.view(T // 128, 128, 4096)
    pk = PackOp()
    add("pack", 2 * int(mask.sum()) * 4096 * 2, lambda: pk.pack(xp, mask))
    V = 151936
    R = max(256, min(T // 16, 2048))                                         # [R, V] bf16: 311 MB at 1024 rows
    logits = (torch.randn(R, V, device=dev, generator=g) * 2).bfloat16()
    tg = torch.randint(0, V, (R,), device=dev, generator=g)
    add("logp_from_logits", logits.numel() * 2, lambda: logp_from_logits(logits, tg))
    thr = logits.float().topk(40, -1).values[:, -1].contiguous()
    add("logp_from_logits_support_threshold", logits.numel() * 2, lambda: logp_from_logits(logits, tg, min_keep=thr))
    ids = logits.float().topk(40, -1).indices
    ids[:, 0] = tg
    add("replay_logp_id_list", R * 40 * (8 + 2), lambda: replay_logp_from_logits(logits, tg, ids, 1.0))
    print(json.dumps({"bench": "elementwise", "rows": T, "peak_gb_s": a.peak_gbs, "results": rows}))


if __name__ == "__main__":
    main()
