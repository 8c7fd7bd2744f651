"""Append-only, sealed run artifacts with resume (parity: rl_engine/validation/cross_config/
{artifacts,_resume}.py; docs/contracts/cross_config_logprob_drift_contract.md:239-265).

runs/<exp>/cases/<case>/<attempt>/{requested,actual,comparison}.json, score.pt, COMPLETE
``COMPLETE`` holds the SHA-256 of every file of the attempt; an attempt is reusable only when it is
complete, its seal verifies and its ``requested.json`` equals the request."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch


def _sha(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


class AttemptStore:
    def __init__(self, root: str | Path, experiment_id: str):
        self.root = Path(root) / experiment_id / "cases"

    def _case_dir(self, case: str) -> Path:
        return self.root / case

    def attempts(self, case: str) -> list[Path]:
        d = self._case_dir(case)
        return sorted((p for p in d.iterdir() if p.is_dir()), key=lambda p: int(p.name)) if d.exists() else []

    def new_attempt(self, case: str) -> Path:
        n = len(self.attempts(case))
        p = self._case_dir(case) / str(n)
        p.mkdir(parents=True, exist_ok=False)
        return p

    @staticmethod
    def write(attempt: Path, requested: dict, actual: dict, score: torch.Tensor, comparison: dict | None = None) -> None:
        (attempt / "requested.json").write_text(json.dumps(requested, sort_keys=True))
        (attempt / "actual.json").write_text(json.dumps(actual, sort_keys=True))
        torch.save(score, attempt / "score.pt")
        if comparison is not None:
            (attempt / "comparison.json").write_text(json.dumps(comparison, sort_keys=True))
        seal = {p.name: _sha(p) for p in sorted(attempt.iterdir()) if p.name != "COMPLETE"}
        (attempt / "COMPLETE").write_text(json.dumps(seal, sort_keys=True))

    @staticmethod
    def verify(attempt: Path) -> bool:
        seal_file = attempt / "COMPLETE"
        if not seal_file.exists():
            return False
        seal = json.loads(seal_file.read_text())
        files = {p.name for p in attempt.iterdir() if p.name != "COMPLETE"}
        return files == set(seal) and all(_sha(attempt / n) == h for n, h in seal.items())

    def reusable(self, case: str, requested: dict) -> Path | None:
        for a in reversed(self.attempts(case)):
            if self.verify(a) and json.loads((a / "requested.json").read_text()) == json.loads(json.dumps(requested, sort_keys=True)):
                return a
        return None

    def seal_run(self) -> str:
        """Seal of the whole run directory (``rlk validate --seal``)."""
        h = hashlib.sha256()
        for p in sorted(self.root.rglob("COMPLETE")):
            h.update(str(p.relative_to(self.root)).encode())
            h.update(p.read_bytes())
        out = self.root.parent / "RUN_SEAL"
        out.write_text(h.hexdigest())
        return h.hexdigest()


# ------------------------------------------------------------------------------------------------ append-only store
# The store the alignment layer's attempts live in, with the guarantees a reader may rely on: a file never changes once
# written (re-writing identical content is a no-op, different content is an error), every file appears whole (written
# beside its target, flushed, renamed), names that could leave the experiment directory are refused, and an attempt is
# complete only when its COMPLETE summary lists the hash of every artifact (parity: ArtifactStore,
# rl_engine/validation/cross_config/artifacts.py:60-500).
import os
import re
from collections.abc import Mapping
from typing import Any


class ArtifactError(RuntimeError):
    """An artifact is missing, was altered, or would have been overwritten."""


_SAFE = re.compile(r"^[A-Za-z0-9][A-Za-z0-9._-]{0,127}$")


def _safe_component(value: str, label: str) -> str:
    if not isinstance(value, str) or not _SAFE.match(value) or ".." in value:
        raise ArtifactError(f"{label} {value!r} is not a safe path component (letters, digits, '.', '_', '-')")
    return value


def _canonical_json(value: Mapping[str, Any]) -> str:
    return json.dumps(value, sort_keys=True, separators=(",", ":"), allow_nan=False) + "\n"


def _fsync_dir(d: Path) -> None:
    try:
        fd = os.open(d, os.O_RDONLY)
    except OSError:
        return
    try:
        os.fsync(fd)
    except OSError:
        pass
    finally:
        os.close(fd)


class ArtifactStore:
    COMPLETE = "COMPLETE"

    def __init__(self, root: str | Path):
        self.root = Path(root)

    # ---- layout
    def experiment_dir(self, experiment_id: str) -> Path:
        return self.root / _safe_component(experiment_id, "experiment_id")

    def initialize_experiment(self, experiment_id: str, config: Mapping[str, Any], *, plan: Mapping[str, Any] | None = None) -> Path:
        """Create (or re-open) an experiment: its config -- and plan, if given -- are written once; opening it again with
        other content is an error, which is what makes ``resume`` safe."""
        d = self.experiment_dir(experiment_id)
        d.mkdir(parents=True, exist_ok=True)
        self._write_or_verify(d / "experiment_config.json", _canonical_json(config))
        if plan is not None:
            self._write_or_verify(d / "plan.json", _canonical_json(plan))
        return d

    def create_attempt(self, experiment_id: str, case_id: str, request: Mapping[str, Any]) -> Path:
        """A new numbered attempt directory of a case with its ``request.json``; attempts are never reused or renumbered."""
        case_dir = self.experiment_dir(experiment_id) / "cases" / _safe_component(case_id, "case_id")
        case_dir.mkdir(parents=True, exist_ok=True)
        for _ in range(1000):
            nums = [int(p.name) for p in case_dir.iterdir() if p.is_dir() and p.name.isdigit()]
            attempt = case_dir / str(max(nums, default=-1) + 1)
            try:
                attempt.mkdir(exist_ok=False)
            except FileExistsError:                   # another process took the number: take the next one
                continue
            self._write_new(attempt / "request.json", _canonical_json(request))
            return attempt
        raise ArtifactError(f"could not allocate an attempt under {case_dir}")

    # ---- writing
    def write_json(self, attempt_dir: str | Path, name: str, value: Mapping[str, Any]) -> Path:
        path = self._artifact_path(attempt_dir, name, ".json")
        self._write_or_verify(path, _canonical_json(value))
        return path

    def write_tensor_bundle(self, attempt_dir: str | Path, name: str, tensors: Mapping[str, torch.Tensor], *,
                            metadata: Mapping[str, Any] | None = None) -> Path:
        path = self._artifact_path(attempt_dir, name, ".pt")
        if path.exists():
            raise ArtifactError(f"{path} already exists; artifacts are append-only")
        payload = {"schema": "cross_config.tensor_bundle.v1", "tensors": {k: v.detach().cpu().contiguous() for k, v in tensors.items()},
                   "metadata": dict(metadata or {})}
        tmp = path.with_name(path.name + f".tmp{os.getpid()}")
        with open(tmp, "wb") as f:
            torch.save(payload, f)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
        _fsync_dir(path.parent)
        return path

    def load_tensor_bundle(self, path: str | Path) -> dict[str, Any]:
        d = torch.load(Path(path), map_location="cpu", weights_only=False)
        if not isinstance(d, Mapping) or d.get("schema") != "cross_config.tensor_bundle.v1" or not isinstance(d.get("tensors"), Mapping):
            raise ArtifactError(f"{path} is not a tensor bundle of this store")
        return dict(d)

    def complete_attempt(self, attempt_dir: str | Path, summary: Mapping[str, Any] | None = None) -> Path:
        """Seal an attempt: COMPLETE lists the SHA-256 of every artifact present plus the caller's summary."""
        a = Path(attempt_dir)
        if (a / self.COMPLETE).exists():
            raise ArtifactError(f"{a} is already complete")
        if not (a / "request.json").exists():
            raise ArtifactError(f"{a} has no request.json")
        files = {p.name: _sha(p) for p in sorted(a.iterdir()) if p.is_file() and ".tmp" not in p.name}
        self._write_new(a / self.COMPLETE, _canonical_json({"schema": "cross_config.complete.v1", "artifacts": files, "summary": dict(summary or {})}))
        return a / self.COMPLETE

    # ---- reading
    def validate_completed_attempt(self, attempt_dir: str | Path) -> dict[str, Any]:
        """The COMPLETE record of an attempt after checking that every listed artifact is there with its hash and that
        nothing else was added."""
        a = Path(attempt_dir)
        seal = a / self.COMPLETE
        if not seal.exists():
            raise ArtifactError(f"{a} is not complete")
        rec = json.loads(seal.read_text())
        if rec.get("schema") != "cross_config.complete.v1" or not isinstance(rec.get("artifacts"), dict):
            raise ArtifactError(f"{seal} is not a COMPLETE record of this store")
        present = {p.name for p in a.iterdir() if p.is_file() and p.name != self.COMPLETE and ".tmp" not in p.name}
        if present != set(rec["artifacts"]):
            raise ArtifactError(f"{a}: artifacts changed after completion (added {sorted(present - set(rec['artifacts']))}, "
                                f"missing {sorted(set(rec['artifacts']) - present)})")
        for name, digest in rec["artifacts"].items():
            if _sha(a / name) != digest:
                raise ArtifactError(f"{a / name} was modified after completion")
        return rec

    def completed_attempt(self, experiment_id: str, case_id: str, request: Mapping[str, Any] | None = None) -> Path | None:
        """The newest attempt of a case that is complete, intact and (if given) was made for exactly ``request``."""
        case_dir = self.experiment_dir(experiment_id) / "cases" / _safe_component(case_id, "case_id")
        if not case_dir.exists():
            return None
        for a in sorted((p for p in case_dir.iterdir() if p.is_dir() and p.name.isdigit()), key=lambda p: int(p.name), reverse=True):
            try:
                self.validate_completed_attempt(a)
            except ArtifactError:
                continue
            if request is None or (a / "request.json").read_text() == _canonical_json(request):
                return a
        return None

    # ---- internals
    def _artifact_path(self, attempt_dir: str | Path, name: str, suffix: str) -> Path:
        a = Path(attempt_dir)
        if (a / self.COMPLETE).exists():
            raise ArtifactError(f"{a} is complete; nothing can be added")
        stem = name[:-len(suffix)] if name.endswith(suffix) else name
        return a / (_safe_component(stem, "artifact name") + suffix)

    def _write_or_verify(self, path: Path, text: str) -> None:
        if path.exists():
            if path.read_text() != text:
                raise ArtifactError(f"{path} already exists with different content; artifacts are append-only")
            return
        self._write_new(path, text)

    def _write_new(self, path: Path, text: str) -> None:
        if path.exists():
            raise ArtifactError(f"{path} already exists; artifacts are append-only")
        tmp = path.with_name(path.name + f".tmp{os.getpid()}")
        with open(tmp, "w") as f:
            f.write(text)
            f.flush()
            os.fsync(f.fileno())
        try:
            os.link(tmp, path)                        # fails if another writer published first: never overwrites
        except FileExistsError:
            raise ArtifactError(f"{path} was published by another writer") from None
        finally:
            os.unlink(tmp)
        _fsync_dir(path.parent)
