"""Gradient invariance and accuracy of an operator (parity: rl_engine/validation/operators/
gradient_invariance.py).  The upstream gradient is a fixed value per logical token, zero on padding;
token-input gradients must be the same bits under every batch configuration; parameter gradients must
be the same bits where the token order is the same and inside a relative bound elsewhere.  Accuracy
compares with autograd through the fp32 gold formula."""
from __future__ import annotations

import torch

from rl_kernel_b200.config.workload import build_logical_batch, load_manifest
from rl_kernel_b200.validation.operators import operator_inputs as oi
from rl_kernel_b200.validation.operators.forward_invariance import (InvarianceReport, build_config_matrix,
                                                                    run_forward_invariance)
from rl_kernel_b200.validation.operators.operator_specs import GOLD, OP_SPECS, make_operator_case

PARAM_GRAD_REL_LIMIT = {"float32": 1e-5, "bfloat16": 2e-2, "float16": 5e-3}


def gold_gradients(op_name: str, *, device: str, dtype: torch.dtype, seed: int = 0, batch=None) -> dict:
    """d(sum(out * gout))/d(inputs) through the fp32 gold for the row-wise operators that have a closed form in
    ``GOLD``; keyed like the adapters' gradient dicts.  Operators without one return {} (their gradient accuracy is
    judged by their own tests against autograd)."""
    spec = OP_SPECS[op_name]
    if op_name not in GOLD or spec.adapter not in ("token_rows", "token_rows_weight"):
        return {}
    batch = batch or build_logical_batch(load_manifest())
    spec, adapter, st = make_operator_case(op_name, batch=batch, device=device, dtype=dtype, seed=seed)
    keys = list(batch.logical_keys())
    x = torch.stack([st["x"][k] for k in keys]).float().requires_grad_(True)
    w = st["weight"].float().requires_grad_(True)
    if op_name == "qk_norm":
        h = spec.params["heads"]
        y = GOLD[op_name](x.view(x.shape[0], h, -1), w).reshape(x.shape[0], -1)
    else:
        y = GOLD[op_name](x, w)
    go = oi.grad_rows(keys, y.detach().to(dtype), seed, batch).float()
    (y * go).sum().backward()
    return {"x": {k: x.grad[i] for i, k in enumerate(keys)}, "weight": w.grad}


def run_gradient_invariance(op_name: str, *, candidate: str = "auto", device: str = "cpu", dtype: torch.dtype | None = None,
                            seed: int = 0, manifest=None) -> InvarianceReport:
    m = manifest or load_manifest()
    rep = run_forward_invariance(op_name, candidate=candidate, device=device, dtype=dtype, seed=seed, manifest=m, gradients=True,
                                 configs=build_config_matrix(m))
    gold = gold_gradients(op_name, device=rep.device, dtype=getattr(torch, rep.dtype), seed=seed)
    if gold:
        base = run_forward_invariance(op_name, candidate=candidate, device=device, dtype=dtype, seed=seed, manifest=m, gradients=True,
                                      configs=build_config_matrix(m, include=("BN/full",)))
        # the baseline's own gradients are not kept on the report; recompute them once for the accuracy figure
        from rl_kernel_b200.validation.operators.forward_invariance import _run_config
        from rl_kernel_b200.validation.operators.operator_specs import make_candidate

        cand = make_candidate(op_name=op_name, candidate=candidate, device=device, dtype=dtype)
        batch = build_logical_batch(m)
        spec, adapter, st = make_operator_case(op_name, batch=batch, device=cand.device, dtype=cand.dtype, seed=seed)
        with torch.enable_grad():
            _, g = _run_config(spec, adapter, cand, st, build_config_matrix(m, include=("BN/full",))[0], batch, m, True)
        worst = 0.0
        for name, ref in gold.items():
            if name not in g:
                continue
            if isinstance(ref, dict):
                a = torch.stack([g[name][k].float() for k in sorted(ref)])
                b = torch.stack([ref[k] for k in sorted(ref)])
            else:
                a, b = g[name].float(), ref
            worst = max(worst, float((a - b).abs().max() / b.abs().max().clamp_min(1e-30)))
        rep.grad_accuracy_err = worst
        rep.grad_accuracy_ok = worst <= PARAM_GRAD_REL_LIMIT.get(rep.dtype, 2e-2) * (1.0 if rep.dtype == "float32" else 1.5)
        del base
    lim = PARAM_GRAD_REL_LIMIT.get(rep.dtype, 2e-2)
    for key, rel in rep.param_grad_rel.items():
        if rel > lim:
            cfg, name = key.split(":")
            rep.grad_configs.setdefault(cfg, {})[name + "(rel)"] = type(next(iter(rep.configs.values())))(tokens=1, mismatched=1,
                                                                                                        max_abs=rel)
    return rep


__all__ = ["PARAM_GRAD_REL_LIMIT", "gold_gradients", "run_gradient_invariance"]
