"""GRPO on one GPU, end to end (parity: examples/post_training/grpo_single_gpu.py of the reference).

    python -m rl_kernel_b200.examples.grpo_single_gpu --steps 4
    python -m rl_kernel_b200.examples.grpo_single_gpu --steps 2 --top-p 0.9        # restricted sampling support, replayed in training

One process holds the rollout engine and the trainer.  Every step: sample a group of completions per prompt with the decode
kernels (CUDA graph), score them with the frozen reference, train with the same operators the sampler used, and check that
the training log-prob of every sampled token equals the log-prob the sampler recorded, bit for bit."""
from __future__ import annotations

import argparse
import json

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--prompts", type=int, default=2)
    ap.add_argument("--group", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--response-len", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--lr", type=float, default=1e-5)
    ap.add_argument("--seed", type=int, default=1234)
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("this example runs the sm_100a engines and needs a CUDA device")
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    dev = torch.device("cuda:0")
    spec = Qwen3DenseSpec.scaled(layers=2, hidden=1024, ffn=2048, q_heads=8, kv_heads=2, head_dim=128, vocab=4096)
    cfg = GRPOConfig(num_prompts=a.prompts, group_size=a.group, prompt_len=a.prompt_len, response_len=a.response_len,
                     micro_batch_seqs=min(8, a.prompts * a.group), lr=a.lr, seed=a.seed, top_k=a.top_k, top_p=a.top_p)
    trainer = GRPOTrainer(spec, cfg, dev)
    gen = torch.Generator().manual_seed(a.seed)

    def reward(tokens):                      # a toy verifiable reward: fraction of even token ids in the completion
        return (tokens[:, cfg.prompt_len:] % 2 == 0).float().mean(1)

    for step in range(a.steps):
        prompts = torch.randint(0, spec.vocab_size, (cfg.num_prompts, cfg.prompt_len), generator=gen).to(dev)
        out = trainer.step(prompts, rewards_fn=reward, step_index=step)
        torch.cuda.synchronize()
        print(json.dumps({"step": step, "reward_mean": float(out["rewards"].mean()), "loss": float(out["loss_sums"][4]),
                          "grad_norm": float(out["grad_norm"]), "train_vs_rollout_logp_mismatches": trainer.mismatch_count(out["train_logp"], out["old_logp"]),
                          "tokens": int(out["old_logp"].numel()), "phase_ms": trainer.phase_ms()}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
