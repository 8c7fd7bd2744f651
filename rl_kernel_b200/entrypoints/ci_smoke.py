"""Fail-fast check that the compiled library is the one serving the operators on a GPU runner (parity:
tools/checks/ci_smoke.py of the reference).  Two ways a GPU job can look green while running only fallbacks: the library
was never built (import falls back to the references), or it was built for another architecture (loading succeeds, the
first launch fails).  This loads the library, launches one kernel, synchronises, and compares with PyTorch.

    python -m rl_kernel_b200.entrypoints.ci_smoke
"""
from __future__ import annotations

import sys

import torch


def main() -> int:
    if not torch.cuda.is_available():
        print("[smoke] FATAL: CUDA is not available in this environment", file=sys.stderr)
        return 2
    cc = torch.cuda.get_device_capability()
    print(f"[smoke] torch {torch.__version__} (cuda {torch.version.cuda}), device {torch.cuda.get_device_name()}, sm_{cc[0]}{cc[1]}")
    from rl_kernel_b200.backends import extension as ext

    path = ext.library_path()
    if not path.exists():
        print(f"[smoke] FATAL: {path} is missing: the kernels were not built (python -m rl_kernel_b200.csrc.build)", file=sys.stderr)
        return 1
    try:
        ext.load()
    except Exception as exc:  # noqa: BLE001
        print(f"[smoke] FATAL: {path} does not load: {exc}", file=sys.stderr)
        return 1
    from rl_kernel_b200.ops.norm import rms_norm

    x = torch.randn(64, 1024, device="cuda").bfloat16()
    w = torch.ones(1024, device="cuda").bfloat16()
    try:
        y = rms_norm(x, w)
        torch.cuda.synchronize()
    except Exception as exc:  # noqa: BLE001
        print(f"[smoke] FATAL: the first kernel launch failed ({exc}); the library was probably built for another architecture "
              f"than sm_{cc[0]}{cc[1]}", file=sys.stderr)
        return 1
    ref = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    err = float((y.float() - ref).abs().max())
    if err > 0.05:
        print(f"[smoke] FATAL: kernel result is off by {err}", file=sys.stderr)
        return 1
    status = ext.poll_status(torch.device("cuda"))
    print(f"[smoke] ok: library {path.name}, max error {err:.3e}, device status {status}")
    return 0 if status == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
