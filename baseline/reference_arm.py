"""Reference arm of bench.py.

Runs the UNMODIFIED reference (installed under baseline/_ref) through its own public API in a
child process whose import path contains the reference only, never this repository (both expose
a package called ``rl_engine``).  The child is ``baseline/ref_runner.py``.

What the reference can run here: its own Qwen3-8B model class (``Qwen3DenseBIModel``) on its
Triton operator profile (the native extension is not built: the install happened on a machine
without a GPU, where the reference's build script skips it) on ONE GPU.  Its multi-GPU path needs Megatron-LM, vLLM and the
vime orchestrator, none of which ship in the reference tree, so N > 1 reports ``unavailable``.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


# History of this arm.  Its first version prefilled 64 sequences x 512 tokens in ONE forward call
# of the reference model and met "CUDA error: an illegal memory access" there (the three message
# lines are kept in profiles/reference_arm_fault.txt).  The cause, found by reading the
# reference: its Triton LM head (_det_gemm_fp32_kernel) forms output offsets as row * 151936 in
# 32-bit integers, which wrap from row 14135 on.  That call shape was the runner's own choice, not
# a workload of the reference, so ref_runner.py now keeps every forward call below that row count
# (and refuses to make a larger one).


def run_reference(args) -> dict:
    ref = HERE / "_ref"
    if not (ref / "rl_engine").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is missing: the reference was not installed on this machine"}
    if args.gpus != 1:
        return {"impl": "reference", "unavailable": "the reference's multi-GPU path needs Megatron-LM + vLLM + vime, which are not part of its tree or of this image"}
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ref)
    env.pop("TORCH_CUDA_ARCH_LIST", None)
    budget = float(os.environ.get("RLK_REF_ARM_BUDGET_S", "1200"))
    cmd = [sys.executable, str(HERE / "ref_runner.py"), "--steps", str(args.steps), "--warmup", str(args.warmup),
           "--response-len", str(args.response_len), "--time-budget", str(budget)]
    if args.layers:
        cmd += ["--layers", str(args.layers)]
    try:
        proc = subprocess.run(cmd, cwd=str(HERE), env=env, capture_output=True, text=True,
                              timeout=budget * 2 + 900)
    except subprocess.TimeoutExpired:
        return {"impl": "reference", "unavailable": "reference run exceeded the time limit of the arm"}
    for line in reversed(proc.stdout.strip().splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except json.JSONDecodeError:
                continue
    tail = (proc.stderr or proc.stdout).strip().splitlines()[-1:] or ["no output"]
    return {"impl": "reference", "unavailable": f"reference runner failed (exit {proc.returncode}): {tail[0][:300]}"}
