"""Times single-token decode steps of the Qwen3 engine (batch of sequences against a KV cache).

    python -m rl_kernel_b200.benchmarks.decode_step --layers 4 --batch 64 --pos 1000 --iters 5

Prints one JSON line with the eager per-step device time and, with --graph, the CUDA-graph time.
Used under ``ncu --metrics gpu__time_duration.sum`` to get the per-kernel launch list of a step.
"""
from __future__ import annotations

import argparse
import json

import torch

from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--pos", type=int, default=1000)
    ap.add_argument("--max-len", type=int, default=1536)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--graph", action="store_true")
    ap.add_argument("--shared-prefix", type=int, default=0, metavar="P",
                    help="the first P positions of every group of --group sequences are shared prompt pages")
    ap.add_argument("--group", type=int, default=8)
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    spec = Qwen3DenseSpec.official().with_layers(a.layers)
    params = PackedParams(spec, 0, 1, dev).init_synthetic_(1)
    eng = Qwen3Engine(spec, params, max_positions=a.max_len + 8)
    shared = None
    if a.shared_prefix:
        shared = eng.new_shared_prefix_cache(a.batch // a.group, a.group, a.shared_prefix, a.max_len - a.shared_prefix)
        kv = shared.kv
        tiles = eng.decode_tiles_shared_prefix(shared, a.group)
    else:
        kv = eng.new_kv_cache(a.batch, a.max_len)
        tiles = eng.decode_tiles(a.batch, a.max_len)
    for t in kv.k + kv.v:
        t.normal_(0, 1)
    tok = torch.randint(0, spec.vocab_size, (a.batch,), device=dev)
    pos = torch.full((a.batch,), a.pos, dtype=torch.int32, device=dev)
    keys = torch.arange(a.batch, device=dev)

    def step():
        hf = eng.decode_step(tok, pos, kv, tiles, shared=shared)
        logits = eng.logits(hf)
        return eng.sample(logits, keys, temperature=1.0, seed=1)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.iters):
        step()
    e.record()
    torch.cuda.synchronize()
    out = {"layers": a.layers, "batch": a.batch, "pos": a.pos, "shared_prefix": a.shared_prefix,
           "eager_ms_per_step": s.elapsed_time(e) / a.iters}
    if a.graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        g.replay()
        torch.cuda.synchronize()
        s.record()
        for _ in range(a.iters):
            g.replay()
        e.record()
        torch.cuda.synchronize()
        out["graph_ms_per_step"] = s.elapsed_time(e) / a.iters
    print(json.dumps(out))


if __name__ == "__main__":
    main()
