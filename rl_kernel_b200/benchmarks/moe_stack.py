"""Training step (forward with checkpoints, LM-head log-probs, full backward with per-layer
recompute, gradient sync of the replicated parameters) of the Qwen3-MoE roadmap stack: 8 layers,
hidden 4096, 128 routed SwiGLU experts of width 1536 (top-8) + one shared expert, 32k tokens per
step spread over the expert-parallel ranks.

    python -m rl_kernel_b200.benchmarks.moe_stack --layers 8 --iters 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29533 -m rl_kernel_b200.benchmarks.moe_stack --layers 8 --iters 3

Timing: CUDA events around ``iters`` steps after ``warmup`` steps, max over ranks; every step
streams the expert weights (>= 4.8 GB per layer per rank), far more than L2.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=32768, help="tokens per step over all ranks")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--micro-seqs", type=int, default=4, help="sequences per micro-batch per rank")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--forward-only", action="store_true")
    a = ap.parse_args()

    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.models.qwen3_moe import MoEPackedParams, Qwen3MoeEngine, Qwen3MoeSpec

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    coll = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
        from rl_kernel_b200.distributed import create_deterministic_collective

        coll = create_deterministic_collective(None, dev)
    spec = Qwen3MoeSpec.roadmap(a.layers)
    seqs = a.tokens // a.seq_len // world
    if seqs < 1 or seqs % a.micro_seqs:
        raise SystemExit(f"{a.tokens} tokens / ({a.seq_len} x {world} ranks) must be a multiple of --micro-seqs")
    params = MoEPackedParams(spec, rank, world, dev, with_grad=not a.forward_only).init_synthetic_(1)
    eng = Qwen3MoeEngine(spec, params, ep_collective=coll, max_tokens=a.micro_seqs * a.seq_len,
                         max_positions=a.seq_len + 8, with_backward=not a.forward_only)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    tok = torch.randint(0, spec.vocab_size, (seqs, a.seq_len), device=dev, generator=g)
    prompt = a.seq_len // 4

    def step():
        if not a.forward_only:
            params.grad.zero_()
        for b0 in range(0, seqs, a.micro_seqs):
            tk = tok[b0:b0 + a.micro_seqs]
            if a.forward_only:
                eng.forward_hidden(tk)
            else:
                eng.train_forward_backward(tk, prompt, lambda lp: torch.full_like(lp, -1.0 / (a.tokens * 0.75)))
        if not a.forward_only:
            eng.sync_replicated_grads()

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    n0 = nv.LAUNCH_COUNT
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.iters):
        step()
    e.record()
    torch.cuda.synchronize()
    ms = torch.tensor([s.elapsed_time(e) / a.iters], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    from rl_kernel_b200.backends import extension as ext

    status = ext.poll_status(dev)
    if rank == 0:
        ms_v = float(ms.item())
        active = spec.active_param_count() - 2 * spec.vocab_size * spec.hidden_size
        flops = (2 if a.forward_only else 8) * active * a.tokens      # fwd + recompute + 2x bwd
        print(json.dumps({"bench": "moe_stack", "layers": a.layers, "ranks": world, "tokens_per_step": a.tokens,
                          "mode": "forward" if a.forward_only else "forward+backward (per-layer recompute)",
                          "ms_per_step": ms_v, "tokens_per_s": a.tokens / ms_v * 1e3,
                          "model_tflops_per_gpu": flops / ms_v / 1e9 / world,
                          "launches_per_step": (nv.LAUNCH_COUNT - n0) // a.iters, "device_status": status}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
