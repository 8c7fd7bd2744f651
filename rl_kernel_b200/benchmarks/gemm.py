"""det_gemm micro-benchmark against torch.matmul (cuBLAS) on the reference's table of shapes
(reports/archive/benchmarks/det_gemm_h100_tma.md) plus decode-sized M.

    python -m rl_kernel_b200.benchmarks.gemm [--shape M N K] [--nchunks C] [--iters I] [--no-cublas]

One JSON line per shape: ms, TFLOP/s, fraction of the measured cuBLAS peak (MEASURED_PEAKS.json).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from rl_kernel_b200.backends import native as nv
from rl_kernel_b200.utils.timing import L2Flusher

SHAPES = [(4096, 12288, 4096), (4096, 4096, 4096), (4096, 14336, 4096), (4096, 4096, 14336), (4096, 32000, 4096),
          (8192, 24576, 4096), (8192, 4096, 12288), (64, 6144, 4096), (64, 24576, 4096), (64, 4096, 12288)]


def bench(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", type=int, nargs=3, default=None)
    ap.add_argument("--nchunks", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--tile-n", type=int, default=0, help="force the output tile width (0 = the kernel's own choice)")
    ap.add_argument("--rotate", action="store_true",
                    help="instead of flushing L2 with writes (which leaves it full of dirty lines whose write-back "
                         "competes with a weight-streaming kernel), cycle through enough weight copies to exceed L2")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    peaks = Path("MEASURED_PEAKS.json")
    peak = json.loads(peaks.read_text())["bf16_tflops"] if peaks.exists() else 1590.0
    flush = L2Flusher(dev)
    for (M, N, K) in ([tuple(a.shape)] if a.shape else SHAPES):
        x = torch.randn(M, K, device=dev).bfloat16()
        copies = max(1, -(-400_000_000 // (N * K * 2))) if a.rotate else 1
        ws = [torch.randn(N, K, device=dev).bfloat16() for _ in range(copies)]
        w = ws[0]
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        turn = [0]

        def next_w():
            turn[0] = (turn[0] + 1) % copies
            return ws[turn[0]]

        if a.nchunks > 1 and M <= 512:
            scratch = torch.empty(a.nchunks * M * N, device=dev, dtype=torch.bfloat16)
            fn = lambda: nv.det_gemm_split(x, next_w(), out, scratch, nchunks=a.nchunks)  # noqa: E731
        else:
            fn = lambda: nv.det_gemm(x, next_w(), out, M=M, N=N, K=K, nchunks=a.nchunks, tile_n=a.tile_n)  # noqa: E731
        ms = bench(fn, a.iters, (lambda: None) if a.rotate else flush)
        rec = {"M": M, "N": N, "K": K, "nchunks": a.nchunks, "tile_n": a.tile_n, "det_gemm_ms": ms, "det_gemm_tflops": 2 * M * N * K / ms / 1e9,
               "frac_of_measured_cublas_peak": 2 * M * N * K / ms / 1e9 / peak, "weight_gbs": N * K * 2 / ms / 1e6}
        if not a.no_cublas:
            cms = bench(lambda: torch.matmul(x, next_w().t(), out=out), a.iters, (lambda: None) if a.rotate else flush)
            rec.update(cublas_ms=cms, cublas_tflops=2 * M * N * K / cms / 1e9, det_over_cublas=ms / cms)
        print(json.dumps(rec))


if __name__ == "__main__":
    main()
