"""Rollout-vs-training score comparison under the tolerance contract (parity: rl_engine/validation/cross_config/
comparison.py:25-318).

Order of judgment: artifacts well-formed (same case and attempt, matching shapes, finite active
scores, known dtypes) -> semantic identities equal (same tokens, same selected ids, same active
mask, same checkpoint and tokenizer policy) -> the fixed |dlogp| threshold of the two compute
dtypes -> per-token mismatch mask.  Inactive positions are set to zero before anything is stored,
so that an ignored NaN cannot poison a resumable artifact.
"""
from __future__ import annotations

from typing import Any, Optional

import torch

from rl_kernel_b200.contracts.numerical import cross_config_threshold, tolerance_contract_fingerprint
from rl_kernel_b200.validation.cross_config.schema import (AlignmentResult, AlignmentStatus, ScoreArtifact, ScoreSide,
                                                           SemanticIdentitySpec, TokenComparisonArtifact)

_IDENTITY_FIELDS = ("checkpoint_id", "model_version", "tokenizer_policy", "tokenizer_id", "token_ids", "selected_token_ids",
                    "active_mask", "attention_mask", "position_ids", "pre_update_state")


def semantic_identity_errors(rollout: SemanticIdentitySpec, training: SemanticIdentitySpec) -> tuple[str, ...]:
    errs = [f"identity.{f} differs between rollout and training" for f in _IDENTITY_FIELDS if getattr(rollout, f) != getattr(training, f)]
    for f in ("cache_metadata", "packing_metadata"):
        a, b = dict(getattr(rollout, f)), dict(getattr(training, f))
        shared = set(a) & set(b)
        if any(a[k] != b[k] for k in shared):
            errs.append(f"identity.{f} disagrees on a shared key")
    return tuple(errs)


def recompute_mismatch_mask(rollout_logprobs: torch.Tensor, training_logprobs: torch.Tensor, active_mask: torch.Tensor,
                            fixed_threshold: float) -> torch.Tensor:
    """Active tokens whose |training - rollout| exceeds the threshold.  A threshold of zero asks for equal bits (so that
    +0 / -0 or two NaN payloads never pass as equal by accident of float comparison)."""
    a, b = rollout_logprobs.float(), training_logprobs.float()
    if fixed_threshold == 0.0:
        off = a.contiguous().view(torch.int32) != b.contiguous().view(torch.int32)
    else:
        off = (b - a).abs() > fixed_threshold
    return off & active_mask.bool()


def _dtype_name(s: str) -> Optional[str]:
    n = str(s).removeprefix("torch.").lower()
    return {"bf16": "bfloat16", "bfloat16": "bfloat16", "fp16": "float16", "float16": "float16", "half": "float16", "fp32": "float32",
            "float32": "float32", "float": "float32"}.get(n)


def _artifact_errors(r: ScoreArtifact, t: ScoreArtifact) -> tuple[str, ...]:
    errs = []
    if r.side is not ScoreSide.ROLLOUT or t.side is not ScoreSide.TRAINING:
        errs.append("expected a rollout artifact and a training artifact, in that order")
    if r.case_id != t.case_id:
        errs.append("artifacts belong to different cases")
    if r.attempt_id != t.attempt_id:
        errs.append("artifacts belong to different attempts")
    if r.selected_logprobs.shape != t.selected_logprobs.shape:
        errs.append("selected_logprobs shapes differ")
    if not torch.equal(r.active_mask, t.active_mask):
        errs.append("active masks of the artifacts differ")
    for a in (r, t):
        if not a.selected_logprobs.dtype.is_floating_point:
            errs.append(f"{a.side.value} selected_logprobs must be floating point")
        if _dtype_name(a.scorer.dtype) is None:
            errs.append(f"{a.side.value} scorer dtype {a.scorer.dtype!r} is not a known compute dtype")
    return tuple(errs)


def _artifact_identity_errors(r: ScoreArtifact, t: ScoreArtifact) -> list[str]:
    errs = []
    for a in (r, t):
        want = torch.tensor(a.identity.active_mask, dtype=torch.bool)
        if want.shape != a.active_mask.shape or not torch.equal(want, a.active_mask):
            errs.append(f"{a.side.value} artifact active_mask does not match its identity")
    return errs


def _diagnostics(a, b, mask, diff, mismatches: int) -> dict[str, Any]:
    d = diff[mask]
    i = int(torch.where(mask.reshape(-1), diff.reshape(-1), torch.full_like(diff.reshape(-1), -1.0)).argmax())
    row, col = divmod(i, diff.shape[-1]) if diff.dim() == 2 else (0, i)
    bitwise = int((a.contiguous().view(torch.int32) != b.contiguous().view(torch.int32))[mask].sum())
    return {"max_abs_diff": float(d.max()), "mean_abs_diff": float(d.mean()), "worst_token": [int(row), int(col)],
            "worst_rollout": float(a.reshape(-1)[i]), "worst_training": float(b.reshape(-1)[i]), "mismatch_fraction": mismatches / int(d.numel()),
            "bitwise_mismatch_count": bitwise, "signed_mean_diff": float((b - a)[mask].mean())}


class FixedThresholdComparator:
    """The only judgment the contract allows between the two sides: a fixed absolute bound per compute-dtype pair."""

    def __init__(self, *, bitwise: bool = False):
        self.bitwise = bitwise       # judge at threshold 0 (equal bits): what this framework's own two sides must meet

    def _result(self, r, status, **kw) -> AlignmentResult:
        base = dict(case_id=r.case_id, attempt_id=r.attempt_id, status=status, comparable=False, passed=False, active_token_count=0,
                    mismatch_count=0, contract_fingerprint=tolerance_contract_fingerprint())
        base.update(kw)
        return AlignmentResult(**base)

    def compare(self, rollout: ScoreArtifact, training: ScoreArtifact) -> AlignmentResult:
        errs = _artifact_errors(rollout, training)
        if errs:
            return self._result(rollout, AlignmentStatus.INVALID_ARTIFACT, artifact_errors=errs)
        ident = list(semantic_identity_errors(rollout.identity, training.identity)) + _artifact_identity_errors(rollout, training)
        if ident:
            return self._result(rollout, AlignmentStatus.INVALID_IDENTITY, identity_errors=tuple(dict.fromkeys(ident)))
        thr = 0.0 if self.bitwise else cross_config_threshold(_dtype_name(rollout.scorer.dtype), _dtype_name(training.scorer.dtype))
        a, b = rollout.selected_logprobs.float(), training.selected_logprobs.float()
        mask = rollout.active_mask.bool()
        n = int(mask.sum())
        if n and not (bool(torch.isfinite(a[mask]).all()) and bool(torch.isfinite(b[mask]).all())):
            return self._result(rollout, AlignmentStatus.INVALID_ARTIFACT, active_token_count=n, fixed_threshold=thr,
                                artifact_errors=("active selected logprobs must be finite",))
        a, b = a.masked_fill(~mask, 0.0), b.masked_fill(~mask, 0.0)
        diff = (b - a).abs()
        mism = recompute_mismatch_mask(a, b, mask, thr)
        tokens = TokenComparisonArtifact(a, b, mask, diff, mism, thr)
        if n == 0:
            return self._result(rollout, AlignmentStatus.ZERO_ACTIVE_TOKENS, fixed_threshold=thr, token_artifact=tokens)
        count = int(mism.sum())
        return self._result(rollout, AlignmentStatus.PASS if count == 0 else AlignmentStatus.FAIL, comparable=True, passed=count == 0,
                            active_token_count=n, mismatch_count=count, fixed_threshold=thr,
                            diagnostics=_diagnostics(a, b, mask, diff, count), token_artifact=tokens)


def compare_score_artifacts(rollout: ScoreArtifact, training: ScoreArtifact, *, bitwise: bool = False) -> AlignmentResult:
    return FixedThresholdComparator(bitwise=bitwise).compare(rollout, training)


__all__ = ["FixedThresholdComparator", "compare_score_artifacts", "recompute_mismatch_mask", "semantic_identity_errors"]
