"""Strict experiment configuration for cross-configuration drift runs: unknown fields are errors,
knobs come from an allow-list (parity: rl_engine/validation/cross_config/config.py and
docs/contracts/cross_config_logprob_drift_contract.md:112-131)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from pathlib import Path

KNOB_ALLOWLIST = {
    "tp_size": (1, 2, 4, 8), "cp_size": (1, 2, 4, 8), "batch_size": None, "chunk_size": None,
    "padding": ("none", "left", "right"), "decode_from": None, "operator_override": None, "dtype": ("float32", "bfloat16"),
}


@dataclass(frozen=True)
class CaseConfig:
    name: str
    knobs: dict = field(default_factory=dict)

    def __post_init__(self):
        for k, v in self.knobs.items():
            if k not in KNOB_ALLOWLIST:
                raise ValueError(f"case {self.name!r}: knob {k!r} is not in the allow-list {sorted(KNOB_ALLOWLIST)}")
            allowed = KNOB_ALLOWLIST[k]
            if allowed is not None and v not in allowed:
                raise ValueError(f"case {self.name!r}: knob {k}={v!r} not in {allowed}")


@dataclass(frozen=True)
class ExperimentConfig:
    experiment_id: str
    reference_case: str
    cases: tuple[CaseConfig, ...]
    seed: int = 20260812
    num_sequences: int = 4
    seq_len: int = 24
    model: dict = field(default_factory=dict)
    backend: str = "reference"            # reference (CPU batch-invariant model) | engine (sm_100a Qwen3Engine) | auto

    def __post_init__(self):
        if self.backend not in ("reference", "engine", "auto"):
            raise ValueError(f"backend {self.backend!r} is not one of reference / engine / auto")
        names = [c.name for c in self.cases]
        if len(set(names)) != len(names):
            raise ValueError("case names must be unique")
        if self.reference_case not in names:
            raise ValueError(f"reference_case {self.reference_case!r} is not one of the cases")

    @classmethod
    def from_dict(cls, d: dict) -> "ExperimentConfig":
        known = {f.name for f in fields(cls)}
        unknown = set(d) - known
        if unknown:
            raise ValueError(f"unknown experiment fields: {sorted(unknown)}")
        cases = []
        for c in d.get("cases", []):
            extra = set(c) - {"name", "knobs"}
            if extra:
                raise ValueError(f"unknown case fields: {sorted(extra)}")
            cases.append(CaseConfig(c["name"], dict(c.get("knobs", {}))))
        return cls(**{**d, "cases": tuple(cases)})

    @classmethod
    def load(cls, path: str | Path) -> "ExperimentConfig":
        return cls.from_dict(json.loads(Path(path).read_text()))
