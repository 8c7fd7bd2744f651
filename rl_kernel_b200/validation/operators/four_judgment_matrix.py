"""The four judgments of an operator: forward accuracy, forward invariance, gradient accuracy,
gradient invariance (parity: rl_engine/validation/operators/four_judgment_matrix.py:21-50).
Accuracy compares with the fp32 gold inside the precision profile's tolerance; invariance is
raw-bit equality."""
from __future__ import annotations

import torch

from rl_kernel_b200.contracts.diagnostics.matrices import DiagnosticMatrix
from rl_kernel_b200.contracts.numerical import resolve_tolerance
from rl_kernel_b200.validation.operators.forward_invariance import run_forward_invariance, run_gradient_invariance
from rl_kernel_b200.validation.operators.op_specs import OpSpec, build_specs

JUDGMENTS = ("forward_accuracy", "forward_invariance", "gradient_accuracy", "gradient_invariance")


def judge_operator(spec: OpSpec, device="cpu", dtype=torch.float32, seed: int = 0) -> dict[str, tuple[str, str]]:
    out: dict[str, tuple[str, str]] = {}
    dev = torch.device(device)
    inputs = spec.make_inputs(32, dev, dtype, seed)
    cand = spec.candidate(inputs)
    gold = spec.gold(inputs)
    key = "float32" if cand.dtype == torch.float32 else str(dtype).removeprefix("torch.")
    try:
        tol = resolve_tolerance(spec.name, key)
    except KeyError:
        tol = resolve_tolerance("default", key)
    ok, err = tol.check(cand, gold)
    out["forward_accuracy"] = ("pass" if ok else "fail", f"max_abs_err={err:.3e}")
    inv = run_forward_invariance(spec, device=device, dtype=dtype, seed=seed)
    bad = [k for k, v in inv.items() if not v]
    out["forward_invariance"] = ("pass" if not bad else "fail", ",".join(bad))
    if spec.grad_inputs:
        leaf = {k: (v.detach().clone().float().requires_grad_(True) if k in spec.grad_inputs else v) for k, v in inputs.items()}
        spec.gold(leaf).sum().backward()
        leaf2 = {k: (v.detach().clone().requires_grad_(True) if k in spec.grad_inputs else v) for k, v in inputs.items()}
        spec.candidate(leaf2).float().sum().backward()
        worst = 0.0
        for k in spec.grad_inputs:
            g, c = leaf[k].grad, leaf2[k].grad.float()
            worst = max(worst, float((g - c).abs().max() / g.abs().max().clamp_min(1e-12)))
        lim = 5e-2 if dtype != torch.float32 else 1e-4
        out["gradient_accuracy"] = ("pass" if worst <= lim else "fail", f"max_rel_err={worst:.3e}")
        ginv = run_gradient_invariance(spec, device=device, dtype=dtype, seed=seed)
        badg = [k for k, v in ginv.items() if not v]
        out["gradient_invariance"] = ("pass" if not badg else "fail", ",".join(badg))
    else:
        out["gradient_accuracy"] = out["gradient_invariance"] = ("pass", "no differentiable inputs")
    return out


def four_judgment_matrix(op_names=None, device="cpu", dtype=torch.float32) -> DiagnosticMatrix:
    specs = build_specs()
    names = list(op_names or specs)
    m = DiagnosticMatrix("four_judgments", names, list(JUDGMENTS))
    for n in names:
        try:
            res = judge_operator(specs[n], device, dtype)
            for j, (status, detail) in res.items():
                m.set(n, j, status, detail)
        except Exception as exc:  # noqa: BLE001 - a crashing operator is a red cell, not a crashed report
            for j in JUDGMENTS:
                m.set(n, j, "blocked", f"{type(exc).__name__}: {exc}")
    return m
