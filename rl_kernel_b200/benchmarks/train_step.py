"""One training micro-batch (forward with checkpoints, LM head + log-probs, full backward) of the
Qwen3 engine, for timing and for per-kernel launch lists under ncu.

    python -m rl_kernel_b200.benchmarks.train_step --layers 2 --seqs 8 --seq-len 1536 --iters 2
"""
from __future__ import annotations

import argparse
import json

import torch

from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=1536)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--store", action="store_true", help="keep layer intermediates instead of recomputing them")
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    spec = Qwen3DenseSpec.official().with_layers(a.layers)
    params = PackedParams(spec, 0, 1, dev, with_grad=True).init_synthetic_(1)
    eng = Qwen3Engine(spec, params, max_positions=a.seq_len + 8)
    tok = torch.randint(0, spec.vocab_size, (a.seqs, a.seq_len), device=dev)
    fn = lambda: eng.train_forward_backward(tok, a.prompt_len, lambda lp: torch.full_like(lp, -1.0 / lp.numel()),  # noqa: E731
                                            store_activations=a.store)
    fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / a.iters
    T = a.seqs * a.seq_len
    print(json.dumps({"layers": a.layers, "tokens": T, "stored_activations": a.store, "ms_per_microbatch": ms, "tokens_per_s": T / ms * 1e3}))


if __name__ == "__main__":
    main()
