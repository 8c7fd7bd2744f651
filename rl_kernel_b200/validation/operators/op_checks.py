"""Generic operator suite: candidates against a gold implementation over explicit cases (parity:
rl_engine/validation/operators/op_checks.py:23-611).

A case is a named set of inputs; a candidate is any callable taking them.  ``run_operator_suite`` runs every
candidate on every case, compares each output tensor with the gold's inside the precision profile's tolerance for the
candidate's output dtype, optionally compares input gradients (one backward with fixed upstream gradients on both
sides), and records determinism (two runs of the candidate give the same bits)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Sequence

import torch

from rl_kernel_b200.contracts.numerical import resolve_tolerance


@dataclass(frozen=True)
class OperatorCase:
    name: str
    op_class: str
    dtype: torch.dtype
    inputs: Mapping[str, Any]
    grad_inputs: tuple[str, ...] = ()
    seed: int = 0


@dataclass(frozen=True)
class CandidateSpec:
    name: str
    fn: Callable[..., Any]
    backend_id: str = ""
    device: str = "cpu"
    is_gold: bool = False


@dataclass(frozen=True)
class OutputCheck:
    index: int
    passed: bool
    max_abs_err: float
    atol: float
    rtol: float
    bitwise_equal: bool
    dtype: str
    shape: tuple[int, ...]


@dataclass(frozen=True)
class CaseCheck:
    case: str
    outputs: tuple[OutputCheck, ...]
    gradients: Mapping[str, OutputCheck] = field(default_factory=dict)
    deterministic: bool = True
    error: str | None = None

    @property
    def passed(self) -> bool:
        return self.error is None and self.deterministic and all(o.passed for o in self.outputs) and all(
            g.passed for g in self.gradients.values())


@dataclass(frozen=True)
class CandidateReport:
    candidate: str
    backend_id: str
    cases: tuple[CaseCheck, ...]

    @property
    def passed(self) -> bool:
        return all(c.passed for c in self.cases)


@dataclass(frozen=True)
class OperatorCheckReport:
    op_name: str
    gold: str
    candidates: tuple[CandidateReport, ...]

    @property
    def passed(self) -> bool:
        return all(c.passed for c in self.candidates)

    def failures(self) -> list[str]:
        return [f"{c.candidate}/{k.case}: {k.error or 'mismatch'}" for c in self.candidates for k in c.cases if not k.passed]


def _tensors(v: Any) -> list[torch.Tensor]:
    if isinstance(v, torch.Tensor):
        return [v]
    if isinstance(v, (tuple, list)):
        return [t for x in v for t in _tensors(x)]
    if isinstance(v, Mapping):
        return [t for k in sorted(v) for t in _tensors(v[k])]
    return []


def _call(fn, inputs: Mapping[str, Any]) -> Any:
    return fn(**inputs)


def _tolerance(op_name: str, dtype: torch.dtype):
    key = str(dtype).removeprefix("torch.")
    try:
        return resolve_tolerance(op_name, key)
    except KeyError:
        return resolve_tolerance("default", key)


def _compare(op_name: str, i: int, cand: torch.Tensor, gold: torch.Tensor) -> OutputCheck:
    if cand.shape != gold.shape:
        return OutputCheck(i, False, float("inf"), 0.0, 0.0, False, str(cand.dtype), tuple(cand.shape))
    if not cand.dtype.is_floating_point:
        same = bool(torch.equal(cand.cpu(), gold.cpu().to(cand.dtype)))
        return OutputCheck(i, same, 0.0 if same else float("inf"), 0.0, 0.0, same, str(cand.dtype), tuple(cand.shape))
    tol = _tolerance(op_name, cand.dtype)
    ok, err = tol.check(cand.float().cpu(), gold.float().cpu())
    bits = cand.dtype == gold.dtype and bool(torch.equal(cand.cpu().contiguous().view(torch.uint8), gold.cpu().contiguous().view(torch.uint8)))
    return OutputCheck(i, bool(ok), float(err), tol.atol, tol.rtol, bits, str(cand.dtype).removeprefix("torch."), tuple(cand.shape))


def _grad_outputs(outs: list[torch.Tensor], seed: int) -> list[torch.Tensor]:
    g = torch.Generator().manual_seed(seed + 4242)
    return [torch.randn(o.shape, generator=g).to(o.dtype).to(o.device) for o in outs]


def _with_grads(fn, case: OperatorCase, device: str):
    leaves = {}
    inputs = {}
    for k, v in case.inputs.items():
        if isinstance(v, torch.Tensor):
            v = v.to(device)
            if k in case.grad_inputs:
                v = v.detach().clone().requires_grad_(True)
                leaves[k] = v
        inputs[k] = v
    outs = [o for o in _tensors(_call(fn, inputs)) if o.dtype.is_floating_point]
    if leaves:
        torch.autograd.backward([o for o in outs if o.requires_grad],
                                [g for o, g in zip(outs, _grad_outputs(outs, case.seed)) if o.requires_grad])
    return outs, {k: (t.grad if t.grad is not None else torch.zeros_like(t)) for k, t in leaves.items()}


def _run_case(op_name: str, cand: CandidateSpec, gold: CandidateSpec, case: OperatorCase) -> CaseCheck:
    try:
        with torch.enable_grad():
            g_out, g_grad = _with_grads(gold.fn, case, gold.device)
            c_out, c_grad = _with_grads(cand.fn, case, cand.device)
            c_out2, _ = _with_grads(cand.fn, case, cand.device)
    except Exception as exc:  # noqa: BLE001 - a crashing candidate is a failed case with its reason
        return CaseCheck(case.name, (), error=f"{type(exc).__name__}: {exc}")
    if len(c_out) != len(g_out):
        return CaseCheck(case.name, (), error=f"candidate returned {len(c_out)} tensors, gold {len(g_out)}")
    outs = tuple(_compare(op_name, i, c.detach(), g.detach()) for i, (c, g) in enumerate(zip(c_out, g_out)))
    grads = {k: _compare(op_name, i, c_grad[k], g_grad[k]) for i, k in enumerate(sorted(c_grad))}
    det = all(torch.equal(a.detach().cpu().contiguous().view(torch.uint8), b.detach().cpu().contiguous().view(torch.uint8))
              for a, b in zip(c_out, c_out2))
    return CaseCheck(case.name, outs, grads, det)


def run_operator_suite(op_name: str, candidates: Sequence[CandidateSpec], cases: Sequence[OperatorCase]) -> OperatorCheckReport:
    golds = [c for c in candidates if c.is_gold]
    if len(golds) != 1:
        raise ValueError("exactly one candidate is the gold")
    gold = golds[0]
    reports = tuple(CandidateReport(c.name, c.backend_id, tuple(_run_case(op_name, c, gold, k) for k in cases))
                    for c in candidates if not c.is_gold)
    return OperatorCheckReport(op_name, gold.name, reports)


__all__ = ["CandidateReport", "CandidateSpec", "CaseCheck", "OperatorCase", "OperatorCheckReport", "OutputCheck", "run_operator_suite"]
