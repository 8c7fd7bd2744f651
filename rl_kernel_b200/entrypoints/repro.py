"""``rlk`` — reproduce / verify runs from the command line (parity: rl_engine/entrypoints/repro.py:
130-1072, with the vime/Ray job launcher replaced by the in-process sm_100a GRPO harness).

    rlk doctor                      environment, GPU, native library, peaks
    rlk prepare  --profile F        write a machine profile (.rlk-profile.json)
    rlk plan     [--case R/R]       show the integration plan and what it guarantees
    rlk run      --steps N ...      run GRPO steps (tiny model by default, --official for Qwen3-8B)
    rlk verify   RUN_DIR            re-check a run's per-step mismatch records
    rlk validate [--seal] ...       operator four-judgment matrix + cross-config drift run
    rlk report   RUN_DIR            drift report bundle (JSON + Chrome trace + table)
"""
from __future__ import annotations

import argparse
import json
import os
import platform
import shutil
import sys
import time
from pathlib import Path

PROFILE_NAME = ".rlk-profile.json"


def _gpu_busy() -> list[str]:
    """Refuse to launch on GPUs that already run compute processes (parity: repro.py:286-300)."""
    import subprocess

    try:
        out = subprocess.run(["nvidia-smi", "--query-compute-apps=pid,gpu_uuid", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=20).stdout
    except (OSError, subprocess.TimeoutExpired):
        return []
    return [line for line in out.strip().splitlines() if line.strip()]


def cmd_doctor(args) -> int:
    import torch

    from rl_kernel_b200.backends import extension
    from rl_kernel_b200.platforms import device_ctx
    from rl_kernel_b200.runtime.registry import kernel_registry

    info = {"python": sys.version.split()[0], "platform": platform.platform(), "torch": torch.__version__,
            "device": device_ctx.describe(), "native_library": str(extension.library_path()),
            "native_library_present": extension.library_path().exists(), "nvcc": shutil.which("nvcc"),
            "registry_native_ready": kernel_registry.native_ready(), "mode": os.environ.get("RL_KERNEL_MODE", "auto")}
    peaks = Path("MEASURED_PEAKS.json")
    if peaks.exists():
        info["measured_peaks"] = json.loads(peaks.read_text())
    print(json.dumps(info, indent=1, default=str))
    ok = info["native_library_present"] or not torch.cuda.is_available()
    return 0 if ok else 1


def cmd_ops(args) -> int:
    """Every operator of the registry with its candidate backends in resolution order (``--json`` for machines)."""
    from rl_kernel_b200.runtime.registry import kernel_registry

    table = kernel_registry.describe()
    if args.op:
        unknown = [o for o in args.op if o not in table]
        if unknown:
            print(f"unknown operator(s): {unknown}; known: {sorted(table)}", file=sys.stderr)
            return 2
        table = {o: table[o] for o in args.op}
    if args.json:
        print(json.dumps(table, indent=1))
        return 0
    for op, cands in table.items():
        print(op)
        for c in cands:
            mark = "*" if c is next((x for x in cands if x["usable"]), None) else " "
            print(f"  {mark} {c['id']:<12} {c['kind']:<10} {'usable' if c['usable'] else 'skipped: ' + c['reason']}")
            print(f"      {c['path']}")
    return 0


def cmd_chain_gate(args) -> int:
    """The model chain gate over the workload manifest on a scaled CPU model (seconds; no GPU needed)."""
    import torch

    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.reference import Qwen3DenseBIModel
    from rl_kernel_b200.validation.models.chain_gate import run_manifest_chain_gate

    spec = Qwen3DenseSpec.scaled(layers=args.layers, hidden=args.hidden, ffn=2 * args.hidden, q_heads=4, kv_heads=2, head_dim=args.hidden // 4,
                                 vocab=args.vocab)
    w = Qwen3DenseWeights.synthetic(spec, seed=args.seed)
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.dtype]
    rep = run_manifest_chain_gate(Qwen3DenseBIModel(spec, w, execution_dtype=dtype), gold_model=Qwen3DenseBIModel(spec, w),
                                  cells=tuple(c for c in args.cells.split(",") if c), execution_dtype=dtype)
    out = rep.to_dict()
    if args.out:
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(json.dumps(out, indent=1, default=str))
    print(json.dumps({"passed": rep.passed, "first_drift": rep.first_drift,
                      "cells": {c["cell_id"]: f"{c['mismatching_tokens']}/{c['tokens']}" for c in out["invariance"]},
                      "accuracy": None if out["accuracy"] is None else out["accuracy"]["aggregates"]}, indent=1, default=str))
    return 0 if rep.passed else 2


def cmd_prepare(args) -> int:
    prof = {"python": sys.executable, "created": time.time(), "gpus": args.gpus, "run_root": str(Path(args.run_root).resolve())}
    Path(args.profile).write_text(json.dumps(prof, indent=1))
    from rl_kernel_b200.csrc.build import build

    print(json.dumps({"profile": args.profile, "library": str(build())}))
    return 0


def cmd_plan(args) -> int:
    from rl_kernel_b200.runtime.plan import IntegrationPlan

    plan = IntegrationPlan.uniform(args.case) if args.case else IntegrationPlan.from_env()
    print(json.dumps({"plan": plan.describe(), "bitwise_guarantee": plan.bitwise_guarantee, "env": plan.to_env(),
                      "rollout": plan.side("rollout"), "train": plan.side("train")}, indent=1))
    return 0


def _parse_plan(text: str) -> dict:
    """"tp4xcp2", "dp8", "tp2xdp4" -> {"tp": .., "cp": .., "dp": ..}."""
    plan = {"tp": 1, "cp": 1, "dp": 1}
    for part in text.lower().split("x"):
        for key in plan:
            if part.startswith(key) and part[len(key):].isdigit():
                plan[key] = int(part[len(key):])
                break
        else:
            raise SystemExit(f"cannot parse plan component {part!r} (expected e.g. tp4xcp2, dp8, tp2xdp4)")
    return plan


def _validate_topology(tp: int, cp: int, gpus: int, dp: int = 1) -> None:
    if tp * cp * dp != gpus:
        raise SystemExit(f"tp ({tp}) x cp ({cp}) x dp ({dp}) must equal --gpus ({gpus})")
    for n in (tp, cp):
        if n not in (1, 2, 4, 8):
            raise SystemExit("tp and cp must be 1, 2, 4 or 8")


def _free_port() -> int:
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch_command(argv: list[str], gpus: int, port: int | None = None) -> list[str]:
    """The command that runs ``rlk <argv>`` as one rank per GPU on this node."""
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
            "--master-port", str(port or _free_port()), "-m", "rl_kernel_b200.entrypoints.repro", *argv]


def cmd_run(args) -> int:
    import torch

    plan = _parse_plan(args.plan) if args.plan else {"tp": args.tp, "cp": args.cp, "dp": max(1, args.gpus // (args.tp * args.cp))}
    _validate_topology(plan["tp"], plan["cp"], args.gpus, plan["dp"])
    if not torch.cuda.is_available():
        raise SystemExit("rlk run needs a CUDA device (use `rlk validate` for the CPU checks)")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        # one process per GPU: re-launch this command under the elastic launcher and hand its exit code back
        import subprocess

        if torch.cuda.device_count() < args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but only {torch.cuda.device_count()} CUDA devices are visible")
        busy = _gpu_busy()
        if busy and not args.allow_busy:
            raise SystemExit(f"GPUs already run compute processes: {busy}; pass --allow-busy to run anyway")
        return subprocess.call(launch_command(args.raw_argv + ["--allow-busy"], args.gpus))
    if world != args.gpus:
        raise SystemExit(f"WORLD_SIZE={world} but --gpus {args.gpus}")
    rank, local = int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1:
        busy = _gpu_busy()
        if busy and not args.allow_busy:
            raise SystemExit(f"GPUs already run compute processes: {busy}; pass --allow-busy to run anyway")
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    spec = Qwen3DenseSpec.official() if args.official else Qwen3DenseSpec.scaled(
        layers=2, hidden=1024, ffn=2048, q_heads=8, kv_heads=2, head_dim=128, vocab=4096)
    ctx = None
    if world > 1:
        import torch.distributed as dist

        from rl_kernel_b200.models.qwen3.parallel_setup import build_parallel_context, cp_frame_bytes_for

        dist.init_process_group("nccl", device_id=dev)
        tokens_per_rank = args.micro_batch * (args.prompt_len + args.response_len)
        ctx = build_parallel_context(plan["tp"], plan["cp"], dev, dp=plan["dp"],
                                     cp_frame_bytes=cp_frame_bytes_for(spec, plan["tp"], tokens_per_rank))
    cfg = GRPOConfig(num_prompts=args.prompts, group_size=args.group, prompt_len=args.prompt_len,
                     response_len=args.response_len, micro_batch_seqs=args.micro_batch * plan["cp"], lr=args.lr, seed=args.seed,
                     share_rollout_weights=args.official and world == 1)
    trainer = GRPOTrainer(spec, cfg, dev, ctx=ctx) if ctx is not None else GRPOTrainer(spec, cfg, dev)
    run_dir = Path(args.out)
    if rank == 0:
        run_dir.mkdir(parents=True, exist_ok=True)
    gen = torch.Generator().manual_seed(args.seed)
    total_mism = 0
    with open(run_dir / "rounds.jsonl" if rank == 0 else os.devnull, "w") as f:
        for step in range(args.steps):
            prompts = torch.randint(0, spec.vocab_size, (cfg.num_prompts, cfg.prompt_len), generator=gen).to(dev)
            t0 = time.perf_counter()
            out = trainer.step(prompts, step_index=step)
            torch.cuda.synchronize()
            mism = trainer.mismatch_count(out["train_logp"], out["old_logp"])
            total_mism += mism
            rec = {"step": step, "mismatch_count": mism, "tokens_compared": out["old_logp"].numel(),
                   "max_abs_dlogp": float((out["train_logp"] - out["old_logp"]).abs().max()),
                   "reward_mean": float(out["rewards"].mean()), "grad_norm": float(out["grad_norm"]),
                   "loss": float(out["loss_sums"][4]), "policy_loss": float(out["loss_sums"][5]), "kl": float(out["loss_sums"][6]), "weight_version": int(trainer.weight_version),
                   "step_seconds": time.perf_counter() - t0, "phase_ms": trainer.phase_ms()}
            f.write(json.dumps(rec) + "\n")
            if rank == 0:
                print(json.dumps(rec))
    if rank == 0:
        (run_dir / "summary.json").write_text(json.dumps({"steps": args.steps, "total_mismatches": total_mism, "model": spec.model_id,
                                                           "gpus": args.gpus, "plan": plan}))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    return 0 if total_mism == 0 else 2


def _verify_rounds(run_dir: Path) -> tuple[dict, bool]:
    """Acceptance checks of a training run: every step compared tokens and found no mismatch, every metric is finite,
    steps are consecutive and the published weight version grows by one per step."""
    import math

    recs = [json.loads(line) for line in (run_dir / "rounds.jsonl").read_text().splitlines() if line.strip()]
    bad = [r for r in recs if r["mismatch_count"] != 0]
    issues = []
    if [r["step"] for r in recs] != list(range(len(recs))):
        issues.append("steps are not consecutive from 0")
    for r in recs:
        for k in ("max_abs_dlogp", "reward_mean", "grad_norm", "loss"):
            if r.get(k) is not None and not math.isfinite(float(r[k])):
                issues.append(f"step {r['step']}: {k} is not finite")
        if r.get("tokens_compared", 0) <= 0:
            issues.append(f"step {r['step']}: no tokens compared")
    versions = [r["weight_version"] for r in recs if r.get("weight_version") is not None]
    if versions and any(b - a != 1 for a, b in zip(versions, versions[1:])):
        issues.append("weight versions do not grow by one per step")
    summary = run_dir / "summary.json"
    if summary.exists():
        want = json.loads(summary.read_text()).get("steps")
        if want is not None and want != len(recs):
            issues.append(f"summary.json names {want} steps, rounds.jsonl holds {len(recs)}")
    info = {"kind": "training_rounds", "steps": len(recs), "steps_with_mismatches": len(bad),
            "tokens_compared": sum(r["tokens_compared"] for r in recs), "total_mismatches": sum(r["mismatch_count"] for r in recs),
            "weight_versions": [versions[0], versions[-1]] if versions else None, "issues": issues}
    return info, bool(recs) and not bad and not issues


def _verify_attempts(run_dir: Path, case_id: str | None) -> tuple[dict, bool]:
    """Re-check the sealed attempts of a cross-config (``cases/``) or paired-alignment (``paired/``) run: every seal must
    verify, and every stored comparison must be reproducible from the stored tensors.  ``case_id`` restricts the check."""
    import torch

    from rl_kernel_b200.validation.cross_config._resume import comparison_matches, load_tensor_bundle, read_json_object, verify_seal
    from rl_kernel_b200.validation.cross_config.artifacts import AttemptStore

    out = {"kind": "cross_config", "cases": {}}
    ok = True
    found = False
    for sub, paired in (("cases", False), ("paired", True)):
        for root in sorted(run_dir.glob(f"**/{sub}")):
            for case_dir in sorted(p for p in root.iterdir() if p.is_dir()):
                if case_id and case_dir.name != case_id:
                    continue
                attempts = sorted((p for p in case_dir.iterdir() if p.is_dir() and p.name.isdigit()), key=lambda p: int(p.name))
                if not attempts:
                    continue
                found = True
                last = attempts[-1]
                sealed = verify_seal(last) if paired else AttemptStore.verify(last)
                row = {"attempts": len(attempts), "sealed": sealed}
                if sealed and paired:
                    res = read_json_object(last / "result.json")
                    row.update(status=res["status"], passed=res["passed"], mismatch_count=res["mismatch_count"],
                               recomputed=comparison_matches(res, load_tensor_bundle(last / "tensors.pt")))
                    ok &= row["recomputed"] and res["passed"]
                elif sealed and (last / "comparison.json").exists():
                    cmp = json.loads((last / "comparison.json").read_text())
                    row.update(mismatch_count=cmp["mismatch_count"])
                    ok &= cmp["mismatch_count"] == 0
                ok &= sealed
                out["cases"][case_dir.name] = row
    if case_id and not found:
        raise SystemExit(f"no case {case_id!r} under {run_dir}")
    return out, ok and found


def cmd_verify(args) -> int:
    run_dir = Path(args.run_dir)
    if not run_dir.exists():
        raise SystemExit(f"{run_dir} does not exist")
    if (run_dir / "rounds.jsonl").exists() and not args.case_id:
        info, ok = _verify_rounds(run_dir)
    else:
        info, ok = _verify_attempts(run_dir, args.case_id)
    print(json.dumps(info, indent=1))
    return 0 if ok else 2


def cmd_validate(args) -> int:
    import torch

    from rl_kernel_b200.validation.operators.four_judgment_matrix import four_judgment_matrix

    device = "cuda" if args.device == "auto" and torch.cuda.is_available() else ("cpu" if args.device == "auto" else args.device)
    dtype = torch.bfloat16 if device == "cuda" else torch.float32
    m = four_judgment_matrix(device=device, dtype=dtype)
    print(m.render())
    rc = 0 if m.green else 1
    if args.config:
        from rl_kernel_b200.validation.cross_config.config import ExperimentConfig
        from rl_kernel_b200.validation.cross_config.runner import run_experiment

        import dataclasses

        exp = ExperimentConfig.load(args.config)
        if args.backend:
            exp = dataclasses.replace(exp, backend=args.backend)
        summary = run_experiment(exp, args.out, resume=not args.no_resume)
        print(json.dumps(summary, indent=1))
        rc |= 0 if summary["all_bitwise_equal"] else 1
    if args.seal and args.config:
        print(json.dumps({"run_seal": summary["run_seal"]}))
    return rc


def cmd_report(args) -> int:
    from rl_kernel_b200.validation.reports.drift_report import write_drift_report

    src = Path(args.run_dir)
    if (src / "paired").exists():
        from rl_kernel_b200.validation.reports.drift_report import build_drift_report, render_drift_report, write_drift_bundle, write_drift_trace

        rep = build_drift_report(src)
        out = Path(args.out or src / "report")
        out.mkdir(parents=True, exist_ok=True)
        (out / "report.json").write_text(json.dumps(rep, indent=1, sort_keys=True, default=str))
        (out / "report.html").write_text(render_drift_report(rep))
        write_drift_trace(rep, out / "trace.json")
        write_drift_bundle(rep, out / "bundle.zip")
        print(json.dumps({"overall": rep["overall"], "cases": len(rep["cases"]), "report": str(out / "report.html"), "bundle": str(out / "bundle.zip")}))
        return 0 if rep["overall"] == "pass" else 1
    summary_file = src / "summary.json"
    if summary_file.exists() and "cases" in json.loads(summary_file.read_text()):
        summary = json.loads(summary_file.read_text())
    else:
        recs = [json.loads(line) for line in (src / "rounds.jsonl").read_text().splitlines() if line.strip()]
        summary = {"cases": {f"step{r['step']:04d}": {"mismatch_count": r["mismatch_count"], "max_abs": r["max_abs_dlogp"],
                                                      "mean_abs": 0.0, "reused": False} for r in recs}}
    paths = write_drift_report(summary, args.out or src / "report")
    print(json.dumps({k: str(v) for k, v in paths.items()}))
    return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="rlk", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("doctor").set_defaults(fn=cmd_doctor)
    p = sub.add_parser("chain-gate", help="model chain gate over the workload manifest on a scaled CPU model")
    p.add_argument("--layers", type=int, default=2)
    p.add_argument("--hidden", type=int, default=64)
    p.add_argument("--vocab", type=int, default=6600)
    p.add_argument("--dtype", choices=("float32", "bfloat16"), default="float32")
    p.add_argument("--cells", default="permuted,long_padding,singletons,chunked,decode")
    p.add_argument("--seed", type=int, default=1)
    p.add_argument("--out", default=None)
    p.set_defaults(fn=cmd_chain_gate)
    p = sub.add_parser("ops", help="list operators and the backend each would resolve to on this machine")
    p.add_argument("op", nargs="*")
    p.add_argument("--json", action="store_true")
    p.set_defaults(fn=cmd_ops)
    p = sub.add_parser("prepare")
    p.add_argument("--profile", default=PROFILE_NAME)
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--run-root", default="runs")
    p.set_defaults(fn=cmd_prepare)
    p = sub.add_parser("plan")
    p.add_argument("--case", default=None)
    p.set_defaults(fn=cmd_plan)
    p = sub.add_parser("run")
    for name, typ, dflt in (("steps", int, 2), ("gpus", int, 1), ("tp", int, 1), ("cp", int, 1), ("prompts", int, 2),
                            ("group", int, 4), ("prompt-len", int, 128), ("response-len", int, 64),
                            ("micro-batch", int, 8), ("seed", int, 1234)):
        p.add_argument(f"--{name}", type=typ, default=dflt)
    p.add_argument("--lr", type=float, default=1e-6)
    p.add_argument("--official", action="store_true", help="full Qwen3-8B shape")
    p.add_argument("--plan", default="", help="parallel layout over --gpus, e.g. tp4xcp2, dp8, tp2xdp4 (default: --tp x --cp, rest data parallel)")
    p.add_argument("--allow-busy", action="store_true")
    p.add_argument("--out", default="runs/latest")
    p.set_defaults(fn=cmd_run)
    p = sub.add_parser("verify")
    p.add_argument("run_dir")
    p.add_argument("--case-id", default=None, help="check one case of a cross-config / paired run directory")
    p.set_defaults(fn=cmd_verify)
    p = sub.add_parser("validate")
    p.add_argument("--device", default="auto")
    p.add_argument("--config", default=None)
    p.add_argument("--out", default="runs")
    p.add_argument("--no-resume", action="store_true")
    p.add_argument("--seal", action="store_true")
    p.add_argument("--backend", choices=("auto", "reference", "engine"), default=None,
                   help="scoring backend of the cross-config run: reference (CPU model) or engine (sm_100a Qwen3Engine)")
    p.set_defaults(fn=cmd_validate)
    p = sub.add_parser("report")
    p.add_argument("run_dir")
    p.add_argument("--out", default=None)
    p.set_defaults(fn=cmd_report)
    return ap


def main(argv=None) -> int:
    raw = list(sys.argv[1:] if argv is None else argv)
    args = build_parser().parse_args(raw)
    args.raw_argv = raw
    return int(args.fn(args) or 0)


if __name__ == "__main__":
    sys.exit(main())
