"""The four judgments of an operator: forward accuracy, forward invariance, gradient accuracy,
gradient invariance (parity: rl_engine/validation/operators/four_judgment_matrix.py:21-50).
Accuracy compares with the fp32 gold inside the precision profile's tolerance; invariance is
raw-bit equality per logical token across the batch configurations of the workload manifest."""
from __future__ import annotations

import torch

from rl_kernel_b200.contracts.diagnostics.matrices import DiagnosticMatrix
from rl_kernel_b200.validation.operators.forward_invariance import run_forward_invariance
from rl_kernel_b200.validation.operators.gradient_invariance import run_gradient_invariance
from rl_kernel_b200.validation.operators.operator_specs import OP_SPECS

JUDGMENTS = ("forward_accuracy", "forward_invariance", "gradient_accuracy", "gradient_invariance")


def judge_operator(op_name: str, device="cpu", dtype=torch.float32, seed: int = 0, candidate: str = "auto") -> dict[str, tuple[str, str]]:
    spec = OP_SPECS[op_name]
    out: dict[str, tuple[str, str]] = {}
    if spec.grad_input_names:
        rep = run_gradient_invariance(op_name, candidate=candidate, device=device, dtype=dtype, seed=seed)
    else:
        rep = run_forward_invariance(op_name, candidate=candidate, device=device, dtype=dtype, seed=seed)
    out["forward_accuracy"] = ("pass" if rep.accuracy_ok else "fail", f"max_err={rep.accuracy_err:.3e}")
    bad = [k for k, c in rep.configs.items() if not c.ok]
    out["forward_invariance"] = ("pass" if not bad else "fail",
                                 ",".join(f"{k}({rep.configs[k].mismatched}/{rep.configs[k].tokens})" for k in bad))
    if spec.grad_input_names:
        out["gradient_accuracy"] = ("pass" if rep.grad_accuracy_ok else "fail", f"max_rel_err={rep.grad_accuracy_err:.3e}")
        badg = [f"{k}:d{n}" for k, per in rep.grad_configs.items() for n, c in per.items() if not c.ok]
        out["gradient_invariance"] = ("pass" if not badg else "fail", ",".join(badg))
    else:
        out["gradient_accuracy"] = out["gradient_invariance"] = ("pass", "no differentiable inputs")
    return out


def four_judgment_matrix(op_names=None, device="cpu", dtype=torch.float32, candidate: str = "auto") -> DiagnosticMatrix:
    names = list(op_names or OP_SPECS)
    m = DiagnosticMatrix("four_judgments", names, list(JUDGMENTS))
    for n in names:
        try:
            res = judge_operator(n, device, dtype, candidate=candidate)
            for j, (status, detail) in res.items():
                m.set(n, j, status, detail)
        except Exception as exc:  # noqa: BLE001 - a crashing operator is a red cell, not a crashed report
            for j in JUDGMENTS:
                m.set(n, j, "blocked", f"{type(exc).__name__}: {exc}")
    return m
