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


def _validate_topology(tp: int, cp: int, gpus: int) -> None:
    if tp * cp != gpus:
        raise SystemExit(f"tp ({tp}) x cp ({cp}) must equal --gpus ({gpus})")
    for n in (tp, cp):
        if n not in (1, 2, 4, 8):
            raise SystemExit("tp and cp must be 1, 2, 4 or 8")


def cmd_run(args) -> int:
    import torch

    _validate_topology(args.tp, args.cp, args.gpus)
    if not torch.cuda.is_available():
        raise SystemExit("rlk run needs a CUDA device (use `rlk validate` for the CPU checks)")
    busy = _gpu_busy()
    if busy and not args.allow_busy:
        raise SystemExit(f"GPUs already run compute processes: {busy}; pass --allow-busy to run anyway")
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    dev = torch.device("cuda:0")
    spec = Qwen3DenseSpec.official() if args.official else Qwen3DenseSpec.scaled(
        layers=2, hidden=1024, ffn=2048, q_heads=8, kv_heads=2, head_dim=128, vocab=4096)
    cfg = GRPOConfig(num_prompts=args.prompts, group_size=args.group, prompt_len=args.prompt_len,
                     response_len=args.response_len, micro_batch_seqs=args.micro_batch, lr=args.lr, seed=args.seed,
                     share_rollout_weights=args.official)
    trainer = GRPOTrainer(spec, cfg, dev)
    run_dir = Path(args.out)
    run_dir.mkdir(parents=True, exist_ok=True)
    gen = torch.Generator().manual_seed(args.seed)
    total_mism = 0
    with open(run_dir / "rounds.jsonl", "w") as f:
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
                   "step_seconds": time.perf_counter() - t0, "phase_ms": trainer.phase_ms()}
            f.write(json.dumps(rec) + "\n")
            print(json.dumps(rec))
    (run_dir / "summary.json").write_text(json.dumps({"steps": args.steps, "total_mismatches": total_mism,
                                                       "model": spec.model_id}))
    return 0 if total_mism == 0 else 2


def cmd_verify(args) -> int:
    run_dir = Path(args.run_dir)
    recs = [json.loads(line) for line in (run_dir / "rounds.jsonl").read_text().splitlines() if line.strip()]
    bad = [r for r in recs if r["mismatch_count"] != 0]
    print(json.dumps({"steps": len(recs), "steps_with_mismatches": len(bad),
                      "tokens_compared": sum(r["tokens_compared"] for r in recs),
                      "total_mismatches": sum(r["mismatch_count"] for r in recs)}))
    return 0 if recs and not bad else 2


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
    p.add_argument("--allow-busy", action="store_true")
    p.add_argument("--out", default="runs/latest")
    p.set_defaults(fn=cmd_run)
    p = sub.add_parser("verify")
    p.add_argument("run_dir")
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
    args = build_parser().parse_args(argv)
    return int(args.fn(args) or 0)


if __name__ == "__main__":
    sys.exit(main())
