"""Resuming a paired run (parity: rl_engine/validation/cross_config/_resume.py:63-394): a stored attempt is reused only
if it is sealed, its seal verifies, it was produced for the same execution fingerprint, and its stored comparison can be
recomputed from its stored tensors with the same outcome."""
from __future__ import annotations

import hashlib
from pathlib import Path
from typing import Any, Mapping, Optional

import torch

from rl_kernel_b200.validation.cross_config._json import strict_json_loads
from rl_kernel_b200.validation.cross_config.comparison import recompute_mismatch_mask

ATTEMPT_FILES = ("request.json", "rollout.json", "training.json", "result.json", "tensors.pt")


def read_json_object(path: Path) -> dict[str, Any]:
    v = strict_json_loads(path.read_text())
    if not isinstance(v, dict):
        raise ValueError(f"{path} does not hold a JSON object")
    return v


def file_sha256(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


def seal_attempt(attempt: Path) -> str:
    seal = {p.name: file_sha256(p) for p in sorted(attempt.iterdir()) if p.is_file() and p.name != "COMPLETE"}
    import json

    text = json.dumps(seal, sort_keys=True)
    (attempt / "COMPLETE").write_text(text)
    return hashlib.sha256(text.encode()).hexdigest()


def verify_seal(attempt: Path) -> bool:
    f = attempt / "COMPLETE"
    if not f.exists():
        return False
    try:
        seal = read_json_object(f)
    except ValueError:
        return False
    files = {p.name for p in attempt.iterdir() if p.is_file() and p.name != "COMPLETE"}
    return files == set(seal) and all(file_sha256(attempt / n) == h for n, h in seal.items())


def load_tensor_bundle(path: Path) -> Mapping[str, torch.Tensor]:
    b = torch.load(path, weights_only=True)
    need = {"rollout_logprobs", "training_logprobs", "active_mask"}
    if not isinstance(b, dict) or not need <= set(b):
        raise ValueError(f"{path} lacks {sorted(need - set(b) if isinstance(b, dict) else need)}")
    return b


def comparison_matches(result: Mapping[str, Any], tensors: Mapping[str, torch.Tensor]) -> bool:
    """Recompute the mismatch count from the stored tensors under the stored threshold."""
    if not result.get("comparable"):
        return True                                     # nothing numerical to recheck: the stored status stands
    thr = result.get("fixed_threshold")
    if thr is None:
        return False
    mask = tensors["active_mask"].bool()
    mism = recompute_mismatch_mask(tensors["rollout_logprobs"], tensors["training_logprobs"], mask, float(thr))
    return int(mism.sum()) == int(result.get("mismatch_count", -1)) and int(mask.sum()) == int(result.get("active_token_count", -1))


def completed_attempt_matches(attempt: Path, *, execution_fingerprint: str, case_id: str) -> Optional[dict[str, Any]]:
    """The stored result if ``attempt`` can stand in for a fresh execution of this request, else None."""
    if not attempt.is_dir() or not verify_seal(attempt):
        return None
    try:
        request = read_json_object(attempt / "request.json")
        result = read_json_object(attempt / "result.json")
        tensors = load_tensor_bundle(attempt / "tensors.pt")
    except (OSError, ValueError, RuntimeError):
        return None
    if request.get("execution_fingerprint") != execution_fingerprint or request.get("case_id") != case_id:
        return None
    if result.get("case_id") != case_id or not comparison_matches(result, tensors):
        return None
    return result


__all__ = ["ATTEMPT_FILES", "comparison_matches", "completed_attempt_matches", "file_sha256", "load_tensor_bundle", "read_json_object",
           "seal_attempt", "verify_seal"]
