"""Vocab-parallel fused linear-LogP + GRPO/PPO ratio-KL loss, forward and backward: hidden 4096,
vocab 151936 (padded 152576) sharded over the ranks, 16k tokens.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29553 -m rl_kernel_b200.benchmarks.vocab_parallel_logp --tokens 16384

Forward: LM-head GEMM with the per-tile statistics exchanged by peer stores from its epilogue,
barrier, ordered merge, loss.  Backward: logits recomputed per chunk -> dlogits -> dH (fixed-tree
all-reduce over the shards) and dW.  CUDA events, max over ranks, L2 flushed.
"""
from __future__ import annotations

import argparse
import json

import torch

from rl_kernel_b200.benchmarks._dist import finish, init, timed_ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=5)
    a = ap.parse_args()
    world, rank, dev = init()
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
    from rl_kernel_b200.models.qwen3.engine import PackedParams, ParallelContext, Qwen3Engine

    spec = Qwen3DenseSpec.official().with_layers(0)
    ctx = ParallelContext()
    if world > 1:
        from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

        ctx = ParallelContext(rank, world, collective=SymmetricMemoryCollective(None, dev))
    params = PackedParams(spec, rank, world, dev, with_grad=True).init_synthetic_(1)
    eng = Qwen3Engine(spec, params, ctx, max_positions=64)
    N, H = a.tokens, spec.hidden_size
    g = torch.Generator(device=dev).manual_seed(5)                     # same rows / targets on every rank
    rows = torch.randn(N, H, device=dev, generator=g).to(torch.bfloat16)
    tgt = torch.randint(0, spec.vocab_size, (N,), device=dev, generator=g)
    old = torch.zeros(1, N, device=dev)
    adv = torch.randn(1, device=dev, generator=g)
    mask = torch.ones(1, N, dtype=torch.uint8, device=dev)
    state = {}

    def forward():
        logp, lse = eng.logp_from_hidden(rows, tgt, want_lse=True)
        r = nv.grpo_loss(logp.view(1, N), (logp.detach() + old).contiguous(), (logp.detach() + old).contiguous(), adv, mask,
                         clip_lo=0.2, clip_hi=0.2, beta=0.001, inv_norm=1.0 / N, want_tokens=False)
        state.update(lse=lse, dlogp=r["dlogp"].reshape(-1).contiguous())

    def backward():
        vloc = params.v_real_local
        wlm, glm = params.w["lm_head"][:vloc], params.g["lm_head"][:vloc]
        drows = eng.ws.get("lm.drows", (N, H))
        for r0 in range(0, N, 4096):
            r1 = min(N, r0 + 4096)
            n = r1 - r0
            logits = eng.ws.get("lm.logits", (4096, vloc))[:n]
            nv.det_gemm(rows[r0:r1], wlm, logits, M=n, N=vloc, K=H)
            nv.dlogits_(logits, tgt[r0:r1], state["lse"][r0:r1], state["dlogp"][r0:r1], vocab_start=params.vocab_start, inv_temp=1.0)
            nv.det_gemm(logits, wlm, drows[r0:r1], M=n, N=H, K=vloc, b_mn=True)
            nv.det_gemm(logits, rows[r0:r1], glm, M=vloc, N=H, K=n, a_mn=True, b_mn=True, accumulate=True)
        ctx.tp_all_reduce_(drows)

    forward()
    t_f = timed_ms(forward, dev, world, a.iters, warmup=2)
    t_b = timed_ms(backward, dev, world, a.iters, warmup=2)
    status = ext.poll_status(dev)
    if rank == 0:
        fl = 2.0 * N * spec.vocab_size * H
        print(json.dumps({"bench": "vocab_parallel_logp", "tp": world, "tokens": N, "vocab": spec.vocab_size,
                          "fwd_ms": t_f, "bwd_ms": t_b, "fwd_tflops_per_gpu": fl / t_f / 1e9 / world,
                          "bwd_tflops_per_gpu": 3 * fl / t_b / 1e9 / world, "device_status": status}))
    finish(world)


if __name__ == "__main__":
    main()
