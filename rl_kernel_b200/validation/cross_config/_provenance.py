"""Provenance of a scoring run (parity: rl_engine/validation/cross_config/_provenance.py:38-327): the environment a
case executed in, a fingerprint of the code that produced the numbers, and the requested -> actual chain per side."""
from __future__ import annotations

import hashlib
import json
import os
import platform
import subprocess
import sys
from pathlib import Path
from typing import Any, Mapping, Optional

import torch

from rl_kernel_b200.validation.cross_config.runtime import AdapterMaterialization, RuntimeMaterialization, aggregate_status
from rl_kernel_b200.validation.cross_config.schema import (MaterializationStatus, RuntimeProvenance, ScoreArtifact, ScorerSpec,
                                                           ScoreSide)

_PACKAGE_ROOT = Path(__file__).resolve().parents[2]
_ENV_KEYS = ("CUDA_VISIBLE_DEVICES", "NCCL_ALGO", "NCCL_PROTO", "NCCL_NVLS_ENABLE", "CUBLAS_WORKSPACE_CONFIG", "RL_KERNEL_STRICT",
             "RL_KERNEL_DISABLE_NATIVE", "VLLM_BATCH_INVARIANT", "WORLD_SIZE", "RANK")


def canonical_fingerprint(value: Any) -> str:
    return hashlib.sha256(json.dumps(json_safe(value), sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def json_safe(v: Any) -> Any:
    if isinstance(v, Mapping):
        return {str(k): json_safe(x) for k, x in v.items()}
    if isinstance(v, (list, tuple, set, frozenset)):
        return [json_safe(x) for x in (sorted(v, key=str) if isinstance(v, (set, frozenset)) else v)]
    if isinstance(v, torch.Tensor):
        return {"dtype": str(v.dtype), "shape": list(v.shape)}
    if isinstance(v, (str, int, bool)) or v is None:
        return v
    if isinstance(v, float):
        return v if v == v and abs(v) != float("inf") else str(v)
    return getattr(v, "value", str(v))


def source_tree_fingerprint(root: Path = _PACKAGE_ROOT, suffixes: tuple[str, ...] = (".py", ".cu", ".cuh", ".h", ".json")) -> str:
    """sha256 over the package's sources (path and content, sorted): two runs compare only if this agrees."""
    h = hashlib.sha256()
    for p in sorted(root.rglob("*")):
        if p.is_file() and p.suffix in suffixes and "__pycache__" not in p.parts:
            h.update(str(p.relative_to(root)).encode())
            h.update(hashlib.sha256(p.read_bytes()).digest())
    return h.hexdigest()


def native_library_fingerprint() -> Optional[str]:
    lib = _PACKAGE_ROOT / "librlk_b200.so"
    return hashlib.sha256(lib.read_bytes()).hexdigest() if lib.exists() else None


def git_revision(root: Path = _PACKAGE_ROOT.parent) -> Optional[str]:
    try:
        out = subprocess.run(["git", "-C", str(root), "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5)
    except (OSError, subprocess.SubprocessError):
        return None
    return out.stdout.strip() or None if out.returncode == 0 else None


def execution_environment_provenance(*, include_source: bool = True) -> dict[str, Any]:
    env = {"python": sys.version.split()[0], "platform": platform.platform(), "torch": torch.__version__,
           "cuda_runtime": torch.version.cuda, "cuda_available": torch.cuda.is_available(),
           "device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else None,
           "env": {k: os.environ.get(k) for k in _ENV_KEYS}, "git_revision": git_revision(),
           "native_library_sha256": native_library_fingerprint()}
    if include_source:
        env["source_tree_sha256"] = source_tree_fingerprint()
    return env


def effective_runtime_status(m: AdapterMaterialization, *, observed: Optional[Mapping[str, Any]] = None) -> MaterializationStatus:
    """Status of one side after the run: a knob the adapter applied but whose value the runtime read back differently
    becomes a FALLBACK; one that cannot be read back stays UNOBSERVABLE."""
    statuses = []
    for a in m.applications:
        s = a.status
        if observed is not None and a.path in observed and s is MaterializationStatus.APPLIED and observed[a.path] != a.materialized:
            s = MaterializationStatus.FALLBACK
        statuses.append(s)
    return aggregate_status(statuses)


def side_provenance(side: ScoreSide, materialization: RuntimeMaterialization, *, actual: Optional[Mapping[str, Any]] = None,
                    implementation_fingerprint: str = "", rank: int = 0, world_size: int = 1) -> RuntimeProvenance:
    m = materialization.adapters.get(side.value)
    apps = m.applications if m is not None else ()
    return RuntimeProvenance(requested={a.path: a.requested for a in apps}, normalized={a.path: a.requested for a in apps},
                             materialized={a.path: a.materialized for a in apps},
                             actual=dict(actual) if actual is not None else {a.path: a.actual for a in apps},
                             status=effective_runtime_status(m, observed=actual) if m is not None else MaterializationStatus.UNSUPPORTED,
                             construction_fingerprint=materialization.case.construction_fingerprint,
                             distributed_context_fingerprint=materialization.case.distributed_context_fingerprint,
                             process_fingerprint=materialization.case.process_fingerprint,
                             implementation_fingerprint=implementation_fingerprint,
                             evidence={a.path: dict(a.evidence) for a in apps if a.evidence}, rank=rank, world_size=world_size)


def concrete_scorer_spec(spec: ScorerSpec, *, device: str, world_size: int) -> ScorerSpec:
    return ScorerSpec(spec.side, spec.backend_id, spec.dtype, device, world_size, spec.topology, spec.construction_options,
                      spec.operator_overrides)


def score_metadata(artifact: ScoreArtifact) -> dict[str, Any]:
    t = artifact.selected_logprobs
    return {"case_id": artifact.case_id, "attempt_id": artifact.attempt_id, "side": artifact.side.value, "shape": list(t.shape),
            "dtype": str(t.dtype).removeprefix("torch."), "active_tokens": int(artifact.active_mask.sum()),
            "sha256": hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest(),
            "scorer": artifact.scorer.to_dict(), "status": artifact.provenance.status.value}


def execution_fingerprint(materialization: RuntimeMaterialization, *, scorer_fingerprints: Mapping[str, str],
                          environment: Optional[Mapping[str, Any]] = None) -> str:
    """What a stored attempt must share with a new request to be reused: the case, what was materialised, the scorers'
    code and the environment's code identity."""
    env = environment or {}
    return canonical_fingerprint({"case_id": materialization.case.case.case_id, "materialized": materialization.case.materialized,
                                  "status": materialization.case.status.value, "scorers": dict(scorer_fingerprints),
                                  "source": env.get("source_tree_sha256"), "native": env.get("native_library_sha256"),
                                  "torch": env.get("torch")})


__all__ = ["canonical_fingerprint", "concrete_scorer_spec", "effective_runtime_status", "execution_environment_provenance",
           "execution_fingerprint", "git_revision", "json_safe", "native_library_fingerprint", "score_metadata", "side_provenance",
           "source_tree_fingerprint"]
