"""Kernel timeline of one decode step replayed as a CUDA graph (start / duration of every kernel
from CUPTI through torch.profiler).  Inside a graph the kernels of a step overlap through
programmatic dependent launch, so the per-kernel device times of an ncu launch list (serialised,
cold cache) do not add up to the step; this listing shows where the step's time really goes.
Times taken under the profiler are for analysis only -- report ``benchmarks.decode_step`` numbers.

    python -m rl_kernel_b200.benchmarks.decode_timeline [layers] [batch] [shared prompt length]
"""
from __future__ import annotations

import sys

import torch
from torch.profiler import profile, ProfilerActivity
from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine


def main() -> None:
    layers = int(sys.argv[1]) if len(sys.argv) > 1 else 4
    B, pos0, max_len = (int(sys.argv[2]) if len(sys.argv) > 2 else 64), 1000, 1536
    dev = torch.device("cuda:0")
    spec = Qwen3DenseSpec.official().with_layers(layers)
    params = PackedParams(spec, 0, 1, dev).init_synthetic_(1)
    eng = Qwen3Engine(spec, params, max_positions=max_len + 8)
    shared_len = int(sys.argv[3]) if len(sys.argv) > 3 else 0
    shared = None
    if shared_len:
        shared = eng.new_shared_prefix_cache(B // 8, 8, shared_len, max_len - shared_len)
        kv = shared.kv
        tiles = eng.decode_tiles_shared_prefix(shared, 8)
    else:
        kv = eng.new_kv_cache(B, max_len)
        tiles = eng.decode_tiles(B, max_len)
    for t in kv.k + kv.v:
        t.normal_(0, 1)
    tok = torch.randint(0, spec.vocab_size, (B,), device=dev)
    pos = torch.full((B,), pos0, dtype=torch.int32, device=dev)
    keys = torch.arange(B, device=dev)
    def step():
        hf = eng.decode_step(tok, pos, kv, tiles, shared=shared)
        logits = eng.logits(hf)
        return eng.sample(logits, keys, temperature=1.0, seed=1)
    for _ in range(3):
        step()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
    ev = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    ev.sort(key=lambda e: e.time_range.start)
    n = len(ev) // 3
    ev = ev[2 * n:]
    t0 = ev[0].time_range.start
    out = []
    prev_end = t0
    busy = 0.0
    for e in ev:
        st, en = e.time_range.start, e.time_range.end
        out.append("%8.1f %7.1f gap %6.1f  %s" % (st - t0, en - st, st - prev_end, e.name[:70]))
        busy += en - st
        prev_end = max(prev_end, en)
    print("\n".join(out))
    print("kernels", len(ev), "span_us", prev_end - t0, "busy_us", busy)


if __name__ == "__main__":
    main()
