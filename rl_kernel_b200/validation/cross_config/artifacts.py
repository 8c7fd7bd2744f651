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
