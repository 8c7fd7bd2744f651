"""Qwen3 FFN layer by weight layout and tensor-parallel degree (parity: benchmarks/layers/benchmark_qwen_ffn_layout.py of the
reference): packed gate/up (one GEMM, SwiGLU over interleaved canonical blocks) against separate gate and up GEMMs, forward
and forward + backward, for the per-rank shapes of TP 1 / 2 / 4 / 8 (one GPU computes one rank's shard; the all-reduce of
the down projection is timed by ``benchmarks.gemm_ar``).

    python -m rl_kernel_b200.benchmarks.ffn_layout --tokens 8192
"""
from __future__ import annotations

import argparse
import json

import torch


def run(tokens: int, hidden: int, ffn: int, tp_sizes=(1, 2, 4, 8), iters: int = 5) -> list[dict]:
    from rl_kernel_b200.ops.activation import swiglu
    from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn
    from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_linear

    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(tokens, hidden, device=dev, generator=g).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    rows = []

    def timed(fn):
        for _ in range(2):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        return sorted(ts)[len(ts) // 2]

    for tp in tp_sizes:
        il = ffn // tp
        wgu = (torch.randn(2 * il, hidden, device=dev, generator=g) * 0.02).bfloat16().requires_grad_(True)
        wg, wu = (torch.randn(il, hidden, device=dev, generator=g) * 0.02).bfloat16(), (torch.randn(il, hidden, device=dev, generator=g) * 0.02).bfloat16()
        wd = (torch.randn(hidden, il, device=dev, generator=g) * 0.02).bfloat16().requires_grad_(True)
        xg = x.clone().requires_grad_(True)

        def packed():
            return qwen3_ffn(x, wgu, wd, canonical_tp=8, tp_size=tp)

        def separate():
            return det_gemm_linear(swiglu(det_gemm_linear(x, wg), det_gemm_linear(x, wu)), wd, 8 // tp)

        def packed_fb():
            y = qwen3_ffn(xg, wgu, wd, canonical_tp=8, tp_size=tp)
            y.backward(y)
            xg.grad = wgu.grad = wd.grad = None

        with torch.no_grad():
            tf_p, tf_s = timed(packed), timed(separate)
        tfb = timed(packed_fb)
        flops = 2.0 * tokens * hidden * il * 3
        rows.append({"tp": tp, "intermediate_local": il, "packed_fwd_ms": tf_p, "separate_fwd_ms": tf_s, "packed_fwd_bwd_ms": tfb,
                     "packed_fwd_tflops": flops / tf_p / 1e9, "fwd_bwd_tflops": 3 * flops / tfb / 1e9})
    return rows


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=12288)
    a = ap.parse_args(argv)
    print(json.dumps({"bench": "ffn_layout", "tokens": a.tokens, "rows": run(a.tokens, a.hidden, a.ffn)}))


if __name__ == "__main__":
    main()
