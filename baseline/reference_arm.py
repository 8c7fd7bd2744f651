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


# The reference's Triton operator profile faulted on the B200 of this pool ("CUDA error: an illegal
# memory access was encountered" inside the first model forward of a 2-layer, 16-token run; the
# message is kept in profiles/reference_arm_fault.txt).  Shared GPUs must not be faulted again, so
# the arm does not launch the reference's GPU code unless RLK_REF_ARM_RUN=1 is set by an operator
# who accepts that risk.
FAULT_NOTE = ("the reference's own GPU code (Triton profile of Qwen3DenseBIModel) raised 'illegal memory access' "
              "on B200 in this pool; not run again (record: profiles/reference_arm_fault.txt)")


def run_reference(args) -> dict:
    if os.environ.get("RLK_REF_ARM_RUN") != "1":
        return {"impl": "reference", "unavailable": FAULT_NOTE}
    ref = HERE / "_ref"
    if not (ref / "rl_engine").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is missing: the reference was not installed on this machine"}
    if args.gpus != 1:
        return {"impl": "reference", "unavailable": "the reference's multi-GPU path needs Megatron-LM + vLLM + vime, which are not part of its tree or of this image"}
    env = dict(os.environ)
    env["PYTHONPATH"] = str(ref)
    env.pop("TORCH_CUDA_ARCH_LIST", None)
    cmd = [sys.executable, str(HERE / "ref_runner.py"), "--steps", str(args.steps), "--warmup", str(args.warmup),
           "--response-len", str(args.response_len)]
    if args.layers:
        cmd += ["--layers", str(args.layers)]
    try:
        proc = subprocess.run(cmd, cwd=str(HERE), env=env, capture_output=True, text=True,
                              timeout=int(os.environ.get("RLK_REF_ARM_TIMEOUT_S", "5400")))
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
