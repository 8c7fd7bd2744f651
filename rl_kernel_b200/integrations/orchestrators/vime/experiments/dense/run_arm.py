"""One arm of the experiment matrix: a group (module cases), a seed, a number of rollout steps (parity:
run_arm.py of the reference's dense experiment).  Writes ``arm.json`` (what was asked), ``rounds.jsonl`` (one record per
step), ``readback.json`` (which operator really served which module on which side) and ``DONE`` into the arm directory."""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

MATRIX = Path(__file__).with_name("experiment_matrix.json")


class ArmUnavailable(RuntimeError):
    pass


def load_matrix(path: Path | None = None) -> dict:
    return json.loads((path or MATRIX).read_text())


def resolve_arm(matrix: dict, phase: str, group: str) -> dict:
    ph = matrix["phases"][phase]
    groups = ph.get("groups") or matrix["groups"]
    if group not in groups:
        raise KeyError(f"phase {phase!r} has no group {group!r}; known: {sorted(groups)}")
    arm = dict(groups[group])
    arm.setdefault("framework_use_rollout_logprobs", ph.get("framework_use_rollout_logprobs", False))
    for module in ("attention", "ffn"):
        if arm[f"{module}_case"] != "R/R":
            raise ArmUnavailable(f"{group}: {module}_case={arm[f'{module}_case']} asks for another framework's {module}; this runtime has the "
                                 "strict operator only")
    if arm["logp_case"] not in ("R/R", "R/P"):
        raise ArmUnavailable(f"{group}: logp_case={arm['logp_case']}: the rollout samples from the fused LM head; only the training side "
                             "has a library alternative")
    return arm


def library_logp(engine, tokens, prompt_len: int, temperature: float):
    """Training-side log-prob the way a framework without the strict operator computes it: final hidden from the engine,
    logits by a library matmul in bf16, fp32 log-softmax.  Scores the response positions of the given sequences."""
    import torch

    B, S = tokens.shape
    hf = engine.forward_hidden(tokens).view(B, S, -1)[:, prompt_len - 1: S - 1]
    w = engine.p.w["lm_head"]
    logits = (hf.reshape(-1, hf.shape[-1]) @ w.t()).float()[:, : engine.spec.vocab_size] / temperature
    tg = tokens[:, prompt_len:].reshape(-1)
    return torch.log_softmax(logits, -1).gather(1, tg[:, None])[:, 0].view(B, S - prompt_len)


def run_arm(out_dir: str | Path, *, phase: str, group: str, seed: int, preset: str = "tiny", num_rollout: int | None = None,
            matrix_path: Path | None = None, device: str = "cuda:0") -> dict:
    import torch

    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    matrix = load_matrix(matrix_path)
    arm = resolve_arm(matrix, phase, group)
    ps = matrix["model_presets"][preset]
    steps = num_rollout or matrix["phases"][phase]["num_rollout"]
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    if (out / "DONE").exists():
        return json.loads((out / "summary.json").read_text())
    request = {"phase": phase, "group": group, "seed": seed, "preset": preset, "num_rollout": steps, **arm}
    (out / "arm.json").write_text(json.dumps(request, indent=1, sort_keys=True))
    if not torch.cuda.is_available():
        raise ArmUnavailable("an arm runs the sm_100a engines and needs a CUDA device")
    dev = torch.device(device)
    spec = Qwen3DenseSpec.official() if ps.get("official") else Qwen3DenseSpec.scaled(**{k: ps[k] for k in ("layers", "hidden", "ffn", "q_heads",
                                                                                                             "kv_heads", "head_dim", "vocab")})
    cfg = GRPOConfig(num_prompts=ps["prompts"], group_size=ps["group"], prompt_len=ps["prompt_len"], response_len=ps["response_len"],
                     micro_batch_seqs=min(8, ps["prompts"] * ps["group"]), seed=seed, share_rollout_weights=bool(ps.get("official")))
    trainer = GRPOTrainer(spec, cfg, dev)
    gen = torch.Generator().manual_seed(seed)
    total = {"strict_mismatches": 0, "library_mismatches": 0, "tokens": 0}
    with open(out / "rounds.jsonl", "w") as f:
        for step in range(steps):
            prompts = torch.randint(0, spec.vocab_size, (cfg.num_prompts, cfg.prompt_len), generator=gen).to(dev)
            t0 = time.perf_counter()
            res = trainer.step(prompts, step_index=step)
            torch.cuda.synchronize()
            old = res["old_logp"]
            train_lp = old if arm["framework_use_rollout_logprobs"] else res["train_logp"]
            rec = {"step": step, "tokens_compared": int(old.numel()), "mismatch_count": trainer.mismatch_count(train_lp, old),
                   "max_abs_dlogp": float((train_lp - old).abs().max()), "reward_mean": float(res["rewards"].mean()),
                   "grad_norm": float(res["grad_norm"]), "step_seconds": time.perf_counter() - t0}
            if arm["logp_case"] == "R/P":
                n = min(4, res["tokens"].shape[0])
                with torch.no_grad():
                    lib = library_logp(trainer.rollout_engine, res["tokens"][:n], cfg.prompt_len, cfg.temperature)
                ref = old.view(res["tokens"].shape[0], -1)[:n]
                rec.update(library_tokens=int(lib.numel()), library_mismatch_count=trainer.mismatch_count(lib, ref),
                           library_max_abs_dlogp=float((lib - ref).abs().max()))
                total["library_mismatches"] += rec["library_mismatch_count"]
            total["strict_mismatches"] += rec["mismatch_count"]
            total["tokens"] += rec["tokens_compared"]
            f.write(json.dumps(rec) + "\n")
    from rl_kernel_b200.runtime.registry import kernel_registry

    readback = {"rollout": {"attention": "b200-tcgen05", "ffn": "b200-tcgen05", "logp": "b200-tcgen05 (fused LM head)"},
                "train": {"attention": "b200-tcgen05", "ffn": "b200-tcgen05",
                          "logp": "b200-tcgen05 (fused LM head)" + (" + library rescoring (diagnostic)" if arm["logp_case"] == "R/P" else "")},
                "fallbacks": [], "native_ready": list(kernel_registry.native_ready())}
    (out / "readback.json").write_text(json.dumps(readback, indent=1))
    summary = {**request, **total, "model": spec.model_id}
    (out / "summary.json").write_text(json.dumps(summary, indent=1, sort_keys=True))
    (out / "DONE").write_text("ok\n")
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("out_dir")
    ap.add_argument("--phase", default="short")
    ap.add_argument("--group", default="consistency")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--preset", default="tiny")
    ap.add_argument("--num-rollout", type=int, default=None)
    a = ap.parse_args(argv)
    try:
        s = run_arm(a.out_dir, phase=a.phase, group=a.group, seed=a.seed, preset=a.preset, num_rollout=a.num_rollout)
    except ArmUnavailable as exc:
        print(json.dumps({"unavailable": str(exc)}))
        return 3
    print(json.dumps(s))
    return 0 if s["strict_mismatches"] == 0 else 2


if __name__ == "__main__":
    sys.exit(main())
