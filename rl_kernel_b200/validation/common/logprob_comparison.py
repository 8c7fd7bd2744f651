"""Single-GPU selected-log-prob comparison: a candidate backend against the fp32 reference (parity:
rl_engine/validation/common/logprob_comparison.py:28-353, also a CLI).

Candidates: ``pytorch`` (the tile-stat reference operator) and ``b200`` (the sm_100a kernels; aliases
``cuda-sm100``, ``sm100``, and -- for command lines written for the reference -- ``cuda-sm90`` / ``sm90``).
Each exposes the direct diagnostic ``(logp, lse)`` so that a drift can be attributed to the
normaliser or to the target logit.
"""
from __future__ import annotations

import argparse
import json
import logging
import sys
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Sequence

import torch

from rl_kernel_b200.validation.common.logprob_drift import LogprobDriftStats, summarize_logprob_drift


class LogprobBackendUnavailable(RuntimeError):
    pass


@dataclass(frozen=True)
class LogprobComparisonInputs:
    logits: torch.Tensor                         # [N, V]
    target_ids: torch.Tensor                     # [N]; ``ignore_index`` marks rows that are skipped
    active_token_mask: torch.Tensor | None = None
    ignore_index: int = -100


@dataclass(frozen=True)
class LogprobCandidate:
    name: str
    requested_backend: str
    actual_backend: str
    fn: Callable[[torch.Tensor, torch.Tensor, int], tuple[torch.Tensor, torch.Tensor]]
    provenance: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LogprobPathDrift:
    candidate_name: str
    lse: LogprobDriftStats
    dlogp: LogprobDriftStats
    bitwise_logp: bool
    provenance: dict[str, Any]


@dataclass(frozen=True)
class LogprobComparisonReport:
    reference_name: str
    drifts: tuple[LogprobPathDrift, ...]
    input_provenance: dict[str, Any]

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


_ALIASES = {"pytorch": "pytorch", "native": "pytorch", "b200": "b200", "cuda-sm100": "b200", "sm100": "b200", "cuda-sm90": "b200",
            "sm90": "b200"}


def _with_ignored(fn, logits, targets, ignore_index):
    """Run ``fn(logits, safe_targets) -> (logp, lse)`` and zero the rows whose target is ``ignore_index``."""
    skip = targets == ignore_index
    lp, lse = fn(logits, targets.masked_fill(skip, 0))
    return lp.masked_fill(skip, 0.0), lse.masked_fill(skip, 0.0)


def make_logprob_candidate(backend: str) -> LogprobCandidate:
    name = _ALIASES.get(backend.strip().lower().replace("_", "-"))
    if name is None:
        raise ValueError(f"unsupported logprob comparison backend {backend!r}; expected one of {sorted(_ALIASES)}")
    if name == "pytorch":
        from rl_kernel_b200.reference.logprob.tile_logp import NativeBatchInvariantLogpOp

        op = NativeBatchInvariantLogpOp()

        def direct(logits, targets):
            return op.apply_fp32(logits, targets, return_lse=True)
    else:
        if not torch.cuda.is_available():
            raise LogprobBackendUnavailable("the b200 backend needs a CUDA device")
        from rl_kernel_b200.ops.logprob import logp_from_logits

        op = logp_from_logits

        def direct(logits, targets):
            if not logits.is_cuda:
                raise LogprobBackendUnavailable("the b200 backend takes CUDA tensors")
            return logp_from_logits(logits, targets, return_lse=True)

    def run(logits, targets, ignore_index):
        try:
            return _with_ignored(direct, logits, targets, ignore_index)
        except (NotImplementedError, OSError) as exc:
            raise LogprobBackendUnavailable(f"backend {name!r} cannot execute this input: {exc}") from exc

    impl = getattr(op, "__qualname__", type(op).__qualname__)
    return LogprobCandidate(f"{name}-batch-invariant-logp", name, name, run,
                            {"requested_alias": backend, "implementation": f"{getattr(op, '__module__', type(op).__module__)}.{impl}"})


def _reference(logits, targets, ignore_index):
    def gold(lg, tg):
        lse = torch.logsumexp(lg.double(), -1)
        return (lg.double().gather(1, tg[:, None])[:, 0] - lse).float(), lse.float()

    return _with_ignored(gold, logits, targets, ignore_index)


def _validate(inputs: LogprobComparisonInputs) -> torch.Tensor:
    lg, tg = inputs.logits, inputs.target_ids
    if lg.dim() != 2 or tg.dim() != 1 or tg.shape[0] != lg.shape[0]:
        raise ValueError(f"logits must be [N, V] and target_ids [N]; got {tuple(lg.shape)} and {tuple(tg.shape)}")
    if tg.dtype != torch.long:
        raise ValueError("target_ids must be int64")
    live = tg != inputs.ignore_index
    if bool(((tg < 0) | (tg >= lg.shape[1]))[live].any()):
        raise ValueError("target ids outside [0, vocab) other than ignore_index")
    mask = live
    if inputs.active_token_mask is not None:
        if inputs.active_token_mask.dtype != torch.bool or inputs.active_token_mask.shape != tg.shape:
            raise ValueError("active_token_mask must be bool with the shape of target_ids")
        mask = mask & inputs.active_token_mask.to(tg.device)
    return mask


def compare_single_gpu_logprob(inputs: LogprobComparisonInputs, candidates: Sequence[LogprobCandidate | str] = ("pytorch",)
                               ) -> LogprobComparisonReport:
    mask = _validate(inputs)
    ref_lp, ref_lse = _reference(inputs.logits, inputs.target_ids, inputs.ignore_index)
    drifts = []
    for c in candidates:
        cand = make_logprob_candidate(c) if isinstance(c, str) else c
        lp, lse = cand.fn(inputs.logits, inputs.target_ids, inputs.ignore_index)
        drifts.append(LogprobPathDrift(cand.name, summarize_logprob_drift(lse.float(), ref_lse, mask=mask),
                                       summarize_logprob_drift(lp.float(), ref_lp, mask=mask),
                                       bool(torch.equal(lp.float()[mask], ref_lp[mask])),
                                       {"requested_backend": cand.requested_backend, "actual_backend": cand.actual_backend,
                                        **cand.provenance}))
    prov = {"rows": int(inputs.logits.shape[0]), "vocab": int(inputs.logits.shape[1]), "active": int(mask.sum()),
            "dtype": str(inputs.logits.dtype).removeprefix("torch."), "device": str(inputs.logits.device),
            "ignore_index": inputs.ignore_index}
    return LogprobComparisonReport("fp64-log-softmax", tuple(drifts), prov)


def route_rl_kernel_logs_to_stderr() -> None:
    """Keep stdout for the JSON report: the package's loggers write to stderr."""
    for name in ("rl_kernel_b200", "rl_engine"):
        log = logging.getLogger(name)
        for h in list(log.handlers):
            log.removeHandler(h)
        log.addHandler(logging.StreamHandler(sys.stderr))
        log.propagate = False


def main(argv: Sequence[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description="selected-log-prob drift of a backend against the fp64 reference")
    ap.add_argument("--backend", action="append", default=None)
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--vocab", type=int, default=4096)
    ap.add_argument("--dtype", choices=("float32", "bfloat16"), default="float32")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output", default=None)
    a = ap.parse_args(argv)
    route_rl_kernel_logs_to_stderr()
    g = torch.Generator().manual_seed(a.seed)
    logits = (torch.randn(a.rows, a.vocab, generator=g) * 3).to(getattr(torch, a.dtype)).to(a.device)
    targets = torch.randint(0, a.vocab, (a.rows,), generator=g).to(a.device)
    rep = compare_single_gpu_logprob(LogprobComparisonInputs(logits, targets), tuple(a.backend or ("pytorch",)))
    text = json.dumps(rep.to_dict(), indent=2, sort_keys=True)
    if a.output:
        open(a.output, "w").write(text + "\n")
    print(text)


__all__ = ["LogprobBackendUnavailable", "LogprobCandidate", "LogprobComparisonInputs", "LogprobComparisonReport", "LogprobPathDrift",
           "compare_single_gpu_logprob", "make_logprob_candidate", "route_rl_kernel_logs_to_stderr"]

if __name__ == "__main__":
    main()
