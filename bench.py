"""Headline benchmark: Qwen3-8B-shape GRPO step (rollout + reference scoring + train fwd/bwd +
optimizer) tokens/s, with the train-vs-rollout log-prob mismatch count.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...     # the unmodified reference from baseline/_ref

Weak scaling: every GPU brings 8 prompts x group 8 x (512 + 1024) tokens; tokens/s counts the
prompt and the response tokens of every sequence.  Default layout: data parallel (one whole-model
replica per GPU); ``--plan tp4xcp2`` etc. select tensor / context parallel layouts
(``parallel_plan``).  On 2, 4 or 8 GPUs the default run also measures the layout the reference's
headline runs use (tensor x context parallel: tp2, tp2xcp2, tp4xcp2) for a few steps after the
main measurement and reports it under ``named_layout`` (``--no-named-layout`` skips it).
Data is synthetic (uniform-random prompt ids, Bernoulli(0.5) rewards), weights are random-init
N(0, 0.02) of the official architecture.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

PROMPTS_PER_GPU, GROUP, PROMPT_LEN, RESPONSE_LEN = 8, 8, 512, 1024
METRIC = "qwen3_8b_grpo_step_tokens_per_s"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) < 9:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = sorted(sm)[len(sm) // 4:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def parse_plan(text: str) -> dict:
    """"tp4xcp2", "dp8", "tp2xdp4" ... -> {"tp": .., "cp": .., "dp": ..}."""
    plan = {"tp": 1, "cp": 1, "dp": 1}
    for part in text.lower().split("x"):
        for key in plan:
            if part.startswith(key):
                plan[key] = int(part[len(key):])
                break
        else:
            raise SystemExit(f"cannot parse plan component {part!r}")
    plan["name"] = "x".join(f"{k}{plan[k]}" for k in ("tp", "cp", "dp") if plan[k] > 1) or "tp1"
    return plan


def parallel_plan(n: int, override: str = "") -> dict:
    """Default: data parallel.  A B200 holds the whole 8B model with its optimizer state (about
    150 GB), so every GPU rolls out and trains its own 8 prompts x 8 samples and the only
    collective of a step is the gradient all-reduce -- the layout that keeps per-GPU work and
    per-GPU efficiency constant as N grows.  ``--plan tp4xcp2`` runs the layout the reference
    needs on 80 GB parts (tensor parallel 4 x context parallel 2, two TP4 rollout engines)."""
    plan = parse_plan(override) if override else {"tp": 1, "cp": 1, "dp": n, "name": f"dp{n}" if n > 1 else "tp1"}
    if plan["tp"] * plan["cp"] * plan["dp"] != n:
        raise SystemExit(f"plan {plan['name']} does not use {n} GPUs")
    return plan


NAMED_LAYOUT = {2: "tp2", 4: "tp2xcp2", 8: "tp4xcp2"}      # the reference's headline layout (TP4 x CP2 on 8 GPUs) and its halves


def _measure(args, plan: dict, dev, world: int, rank: int, local: int, *, warmup: int, steps: int, clocks: bool) -> dict:
    """Builds a trainer for ``plan``, runs ``warmup`` untimed and ``steps`` timed GRPO steps and
    returns the measurements (collective over all ranks; every rank gets the same numbers)."""
    import gc

    import torch
    import torch.distributed as dist

    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer
    from rl_kernel_b200.models.qwen3.parallel_setup import build_parallel_context, cp_frame_bytes_for

    spec = Qwen3DenseSpec.official()
    if args.layers:
        spec = spec.with_layers(args.layers)
    # (a training micro-batch keeps micro_batch x seq_len tokens on every rank, whatever the layout)
    ctx = build_parallel_context(plan["tp"], plan["cp"], dev, dp=plan["dp"],
                                 cp_frame_bytes=cp_frame_bytes_for(spec, plan["tp"], args.micro_batch * (PROMPT_LEN + args.response_len)))
    # one training replica spans all GPUs; a micro-batch keeps micro_batch x seq_len tokens per rank
    cfg = GRPOConfig(num_prompts=PROMPTS_PER_GPU * args.gpus, group_size=GROUP,
                     prompt_len=PROMPT_LEN, response_len=args.response_len,
                     micro_batch_seqs=args.micro_batch * plan["cp"], share_rollout_weights=False,
                     rollout_weights_in_grad_buffer=True, seed=1234,
                     store_activations=plan["cp"] == 1 and args.train_micro_batch > 0,
                     train_micro_batch_seqs=args.train_micro_batch if plan["cp"] == 1 else 0)
    trainer = GRPOTrainer(spec, cfg, dev, ctx=ctx)
    n_prompts_global = PROMPTS_PER_GPU * args.gpus
    tokens_per_step = n_prompts_global * GROUP * (PROMPT_LEN + args.response_len)

    # per-step prompts live in pinned host memory; each step copies its own batch to the device
    gen = torch.Generator().manual_seed(99)
    total = warmup + steps
    host_prompts = torch.randint(0, spec.vocab_size, (total, n_prompts_global, PROMPT_LEN), generator=gen,
                                 dtype=torch.int64).pin_memory()
    dev_prompts = torch.empty(n_prompts_global, PROMPT_LEN, dtype=torch.int64, device=dev)
    host_result = torch.empty(8, dtype=torch.float32).pin_memory()
    mismatches = 0
    mism_tokens = 0

    def one_step(i: int):
        nonlocal mismatches, mism_tokens
        dev_prompts.copy_(host_prompts[i], non_blocking=True)                      # H2D
        out = trainer.step(trainer.local_prompts(dev_prompts), step_index=i)
        # raw-bit comparison of this replica's sequences (every rank of a replica holds the same values)
        mm = (out["train_logp"].view(torch.int32) != out["old_logp"].view(torch.int32)).sum()
        res = torch.cat([out["loss_sums"][:4].float(), out["grad_norm"].float(), mm.float().reshape(1),
                         torch.zeros(2, device=dev)])
        host_result.copy_(res, non_blocking=True)                                   # D2H
        torch.cuda.current_stream().synchronize()
        mismatches += int(host_result[5].item())
        mism_tokens += out["old_logp"].numel()
        return float(host_result[0].item())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        one_step(i)
    mismatches, mism_tokens = 0, 0
    barrier()
    sampler = ClockSampler(local)
    if rank == 0 and clocks:
        sampler.start()
    n0 = nv.LAUNCH_COUNT
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    ev0.record()
    for i in range(warmup, total):
        one_step(i)
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    dev_ms = ev0.elapsed_time(ev1)
    clk = sampler.stop() if rank == 0 and clocks else {}
    launches = nv.LAUNCH_COUNT - n0
    t = torch.tensor([dev_ms, wall * 1e3], dtype=torch.float64, device=dev)
    cnt = torch.tensor([float(mismatches), float(mism_tokens)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(cnt, op=dist.ReduceOp.SUM)      # summed over replicas ...
    per_replica = plan["tp"] * plan["cp"]               # ... every rank of a replica counted the same tokens
    dev_ms, wall_ms = float(t[0]), float(t[1])
    out = {
        "plan": plan["name"], "tokens_per_step": tokens_per_step, "ms_per_step": dev_ms / steps,
        "value": tokens_per_step / (dev_ms / steps / 1e3), "e2e_value": tokens_per_step * steps / (wall_ms / 1e3),
        "mismatches": int(cnt[0]) // per_replica, "tokens_compared": int(cnt[1]) // per_replica, "clocks": clk,
        "launches": int(launches), "h2d": int(dev_prompts.numel() * 8), "d2h": int(host_result.numel() * 4),
        "cfg": cfg, "phase_ms": trainer.phase_ms(),
        "peak_mem_gb": round(torch.cuda.max_memory_allocated(dev) / 2 ** 30, 2),
        "peak_mem_reserved_gb": round(torch.cuda.max_memory_reserved(dev) / 2 ** 30, 2),
        "device_mem_free_gb": round(torch.cuda.mem_get_info(dev)[0] / 2 ** 30, 2),
    }
    # give the memory back before another layout is measured in the same process
    for c in (ctx.collective, ctx.cp_collective, ctx.dp_collective):
        if c is not None and hasattr(c, "close"):
            try:
                c.close()
            except Exception:  # noqa: BLE001 - teardown only
                pass
    del trainer, ctx
    gc.collect()
    torch.cuda.empty_cache()
    return out


def run_ours(args) -> dict:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"WORLD_SIZE={world} but --gpus {args.gpus}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    plan = parallel_plan(args.gpus, args.plan)
    m = _measure(args, plan, dev, world, rank, local, warmup=args.warmup, steps=args.steps, clocks=True)
    cfg = m["cfg"]
    result = {
        "metric": METRIC, "value": m["value"], "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform-random prompt ids, Bernoulli rewards, random-init weights)",
        "impl": "rl_kernel_b200",
        "config": {"model": "Qwen3-8B" if not args.layers else f"Qwen3-8B-shape-{args.layers}L",
                   "global_batch": PROMPTS_PER_GPU * args.gpus * GROUP, "seq_len": PROMPT_LEN + args.response_len,
                   "prompt_len": PROMPT_LEN, "response_len": args.response_len, "group_size": GROUP,
                   "parallelism": plan["name"], "micro_batch_seqs": args.micro_batch,
                   "train_micro_batch_seqs": cfg.train_micro_batch_seqs or cfg.micro_batch_seqs,
                   "activations": "stored" if cfg.store_activations else "per-layer recompute",
                   "tokens_counted": "prompt + response tokens of every sequence (global_batch x seq_len per step)",
                   "l2_policy": "inputs larger than L2 (16 GB of weights stream every pass)",
                   "includes": "weight publish (push kernel into the rollout engine's buffer), prefill, CUDA-graph "
                               "decode+sampling, reference-policy scoring, train fwd/bwd (see activations), exact "
                               "grad-norm clip, AdamW"},
        "logp_mismatch_count": m["mismatches"], "logp_tokens_compared": m["tokens_compared"],
        "clocks": m["clocks"],
        "e2e": {"value": m["e2e_value"], "unit": "tokens/s",
                "h2d_bytes_per_step": m["h2d"], "d2h_bytes_per_step": m["d2h"],
                "timing": "host wall clock around the same steps incl. H2D of prompts and D2H of loss"},
        "gpu_launches": m["launches"],
        "peak_mem_gb": m["peak_mem_gb"], "peak_mem_reserved_gb": m["peak_mem_reserved_gb"],
        "device_mem_free_gb": m["device_mem_free_gb"],
        "phase_ms_last_step": m["phase_ms"],
    }
    named = NAMED_LAYOUT.get(args.gpus)
    if named and not args.plan and args.named_layout:
        # The same job in the tensor x context parallel layout of the reference's headline runs (its
        # fused GEMM + all-reduce, context-parallel attention and vocabulary-parallel LM head are all in
        # the step).  A watchdog prints the main result if this part does not finish.
        done = threading.Event()

        def watchdog():
            if not done.wait(args.named_layout_timeout):
                if rank == 0:
                    result["named_layout"] = {"plan": named, "unavailable": f"did not finish within {args.named_layout_timeout} s"}
                    print(json.dumps(result), flush=True)
                os._exit(0)

        threading.Thread(target=watchdog, daemon=True).start()
        try:
            n = _measure(args, parse_plan(named), dev, world, rank, local, warmup=3, steps=args.named_layout_steps, clocks=False)
            result["named_layout"] = {"plan": n["plan"], "value": n["value"], "unit": "tokens/s", "ms_per_step": n["ms_per_step"],
                                      "steps": args.named_layout_steps, "warmup": 3,
                                      "logp_mismatch_count": n["mismatches"], "logp_tokens_compared": n["tokens_compared"],
                                      "gpu_launches": n["launches"], "phase_ms_last_step": n["phase_ms"],
                                      "peak_mem_gb": n["peak_mem_gb"]}
        except Exception as exc:  # noqa: BLE001 - the main measurement stands on its own
            result["named_layout"] = {"plan": named, "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
        done.set()
    if world > 1:
        dist.destroy_process_group()
    return result if rank == 0 else {}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (marks the config)")
    ap.add_argument("--response-len", type=int, default=RESPONSE_LEN, help="debug only")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--train-micro-batch", type=int, default=4,
                    help="sequences per training micro-batch with stored activations (0 = recompute, --micro-batch)")
    ap.add_argument("--plan", default="", help="debug only: e.g. tp1xcp2 instead of the default plan for --gpus")
    ap.add_argument("--named-layout", dest="named_layout", action="store_true", default=True,
                    help="after the main measurement also measure the tensor x context parallel layout (default)")
    ap.add_argument("--no-named-layout", dest="named_layout", action="store_false")
    ap.add_argument("--named-layout-steps", type=int, default=2)
    ap.add_argument("--named-layout-timeout", type=float, default=900.0)
    args = ap.parse_args()
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        out = run_reference(args)
    else:
        out = run_ours(args)
    if out:
        print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
