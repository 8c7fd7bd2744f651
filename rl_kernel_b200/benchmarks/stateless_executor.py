"""Stateless scoring throughput (parity: benchmarks/e2e/benchmark_stateless_executor.py of the reference): reference / reward
scoring of whole sequences without a KV cache, through (a) the sm_100a engine's ``score`` path and (b) the ``nn.Module``
executor over a small CPU model (the path a Hugging Face policy takes).

    python -m rl_kernel_b200.benchmarks.stateless_executor --layers 4 --seqs 16 --seq-len 1536 --micro-batch 8
"""
from __future__ import annotations

import argparse
import json
import time

import torch


def engine_scoring(layers: int, seqs: int, seq_len: int, prompt_len: int, micro_batch: int, iters: int) -> dict:
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
    from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine

    dev = torch.device("cuda:0")
    spec = Qwen3DenseSpec.official().with_layers(layers)
    eng = Qwen3Engine(spec, PackedParams(spec, 0, 1, dev).init_synthetic_(1), max_positions=seq_len + 8)
    tok = torch.randint(0, spec.vocab_size, (seqs, seq_len), device=dev)
    H = spec.hidden_size

    def score():
        out = []
        for b0 in range(0, seqs, micro_batch):
            t = tok[b0:b0 + micro_batch]
            hf = eng.forward_hidden(t.contiguous()).view(t.shape[0], seq_len, H)
            rows = hf[:, prompt_len - 1: seq_len - 1].reshape(-1, H).contiguous()
            out.append(eng.logp_from_hidden(rows, t[:, prompt_len:].reshape(-1)))
        return torch.cat(out)

    score()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        score()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / iters
    return {"path": "engine", "layers": layers, "tokens": seqs * seq_len, "ms": ms, "tokens_per_s": seqs * seq_len / ms * 1e3}


def module_scoring(seqs: int, seq_len: int, micro_batch: int) -> dict:
    from rl_kernel_b200.runtime.executor import ModuleForwardExecutor, StatelessForwardConfig, StatelessForwardInputs
    from rl_kernel_b200.validation.fixtures.cpu_cross_config import SyntheticCpuCausalLM

    model = SyntheticCpuCausalLM(vocab_size=4096, hidden=64)
    ids = torch.randint(0, 4096, (seqs, seq_len))
    ex = ModuleForwardExecutor(model, StatelessForwardConfig(micro_batch=micro_batch))
    t0 = time.perf_counter()
    res = ex.score(StatelessForwardInputs(ids))
    return {"path": "nn.Module executor (CPU fixture model)", "tokens": seqs * seq_len, "ms": (time.perf_counter() - t0) * 1e3,
            "tokens_per_s": res.metrics["tokens_per_s"], "peak_logits_mb": res.metrics["peak_logits_mb"]}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--seqs", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=1536)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args(argv)
    rows = [module_scoring(min(a.seqs, 4), min(a.seq_len, 64), a.micro_batch)]
    if torch.cuda.is_available():
        rows.append(engine_scoring(a.layers, a.seqs, a.seq_len, a.prompt_len, a.micro_batch, a.iters))
    print(json.dumps({"bench": "stateless_executor", "rows": rows}))


if __name__ == "__main__":
    main()
