"""Forward / gradient invariance configurations (parity: rl_engine/validation/operators/
forward_invariance.py:195-294): the same logical rows are presented as the full batch, in chunks,
as singletons, permuted, and with padding rows on the left / right; every configuration must
reproduce the full-batch bits row for row."""
from __future__ import annotations

import torch

from rl_kernel_b200.utils.bits import bit_equal
from rl_kernel_b200.validation.operators.op_specs import OpSpec

CONFIGS = ("BN/full", "BN/chunked", "B1/singletons", "BN/permuted", "BN/padded_left", "BN/padded_right")


def _subset(inputs: dict, spec: OpSpec, idx: torch.Tensor) -> dict:
    return {k: (v[idx.to(v.device)] if k in spec.row_inputs else v) for k, v in inputs.items()}


def _pad(inputs: dict, spec: OpSpec, n: int, left: bool) -> dict:
    out = {}
    for k, v in inputs.items():
        if k in spec.row_inputs:
            filler = v[:n].flip(0) if v.shape[0] >= n else v[:1].expand(n, *v.shape[1:])
            out[k] = torch.cat([filler, v] if left else [v, filler]).contiguous()
        else:
            out[k] = v
    return out


def run_forward_invariance(spec: OpSpec, rows: int = 24, device="cpu", dtype=torch.float32, seed: int = 0) -> dict[str, bool]:
    inputs = spec.make_inputs(rows, torch.device(device), dtype, seed)
    full = spec.candidate(inputs).detach()
    res = {"BN/full": bit_equal(spec.candidate(inputs).detach(), full)}
    chunks = [spec.candidate(_subset(inputs, spec, torch.arange(a, min(rows, a + 7)))).detach() for a in range(0, rows, 7)]
    res["BN/chunked"] = bit_equal(torch.cat(chunks), full)
    singles = [spec.candidate(_subset(inputs, spec, torch.tensor([i]))).detach() for i in range(rows)]
    res["B1/singletons"] = bit_equal(torch.cat(singles), full)
    perm = torch.randperm(rows, generator=torch.Generator().manual_seed(seed + 1))
    res["BN/permuted"] = bit_equal(spec.candidate(_subset(inputs, spec, perm)).detach(), full[perm.to(full.device)])
    res["BN/padded_left"] = bit_equal(spec.candidate(_pad(inputs, spec, 5, True)).detach()[5:], full)
    res["BN/padded_right"] = bit_equal(spec.candidate(_pad(inputs, spec, 5, False)).detach()[:rows], full)
    return res


def run_gradient_invariance(spec: OpSpec, rows: int = 16, device="cpu", dtype=torch.float32, seed: int = 0) -> dict[str, bool]:
    """Row-local input gradients must not depend on the batch composition."""
    row_grad = [k for k in spec.grad_inputs if k in spec.row_inputs]
    if not row_grad:
        return {}
    inputs = spec.make_inputs(rows, torch.device(device), dtype, seed)
    gout = None

    def grads(sub):
        nonlocal gout
        leaf = {k: (v.detach().clone().requires_grad_(True) if k in row_grad else v) for k, v in sub.items()}
        out = spec.candidate(leaf)
        g = torch.ones_like(out) if gout is None else gout[: out.shape[0]]
        out.backward(g)
        return {k: leaf[k].grad.detach() for k in row_grad}

    full = grads(inputs)
    singles = [grads(_subset(inputs, spec, torch.tensor([i]))) for i in range(rows)]
    return {f"grad[{k}] B1 == BN": bit_equal(torch.cat([s[k] for s in singles]), full[k]) for k in row_grad}
