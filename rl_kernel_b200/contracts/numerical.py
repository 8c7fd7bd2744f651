"""Tolerance resolution (parity: rl_engine/contracts/numerical.py:191-660, profile ws1.json).

Two kinds of judgment exist and must not be mixed: ACCURACY (candidate vs fp32 gold, within a
per-operator tolerance) and INVARIANCE (candidate vs itself under another batch / chunk / padding /
parallel layout: raw-bit equality, never a tolerance)."""
from __future__ import annotations

import json
from dataclasses import dataclass
from functools import lru_cache
from pathlib import Path

import torch

_PROFILE_DIR = Path(__file__).resolve().parent / "profiles" / "precision"


@dataclass(frozen=True)
class ToleranceSpec:
    atol: float
    rtol: float
    scale: str = "elementwise"   # or "row_abs_max": rtol applies to the largest |gold| of the row

    def check(self, candidate: torch.Tensor, gold: torch.Tensor) -> tuple[bool, float]:
        c, g = candidate.float(), gold.float()
        err = (c - g).abs()
        if self.scale == "row_abs_max":
            bound = self.atol + self.rtol * g.abs().amax(dim=-1, keepdim=True).expand_as(g)
        else:
            bound = self.atol + self.rtol * g.abs()
        worst = float((err - bound).max()) if err.numel() else 0.0
        return worst <= 0.0, float(err.max()) if err.numel() else 0.0


@lru_cache(maxsize=8)
def load_precision_profile(name: str = "ws1") -> dict:
    path = _PROFILE_DIR / f"{name}.json"
    data = json.loads(path.read_text())
    for key in ("profile_id", "defaults", "operators", "chain"):
        if key not in data:
            raise ValueError(f"precision profile {path} lacks {key!r}")
    return data


def resolve_tolerance(op_name: str, dtype: torch.dtype | str, profile: str = "ws1") -> ToleranceSpec:
    data = load_precision_profile(profile)
    key = str(dtype).removeprefix("torch.")
    entry = data["operators"].get(op_name, {}).get(key) or data["defaults"].get(key)
    if entry is None:
        raise KeyError(f"no tolerance for operator {op_name!r} dtype {key!r} in profile {profile!r}")
    return ToleranceSpec(float(entry["atol"]), float(entry["rtol"]), entry.get("scale", "elementwise"))


def load_contract(profile: str = "ws1") -> dict:
    """The whole precision profile (the tolerance contract) as a plain dict."""
    return load_precision_profile(profile)


def tolerance_contract_fingerprint(profile: str = "ws1") -> str:
    """sha256 of the canonical JSON of the profile: artifacts judged under different contracts never compare."""
    import hashlib

    return hashlib.sha256(json.dumps(load_precision_profile(profile), sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def cross_config_threshold(dtype_a: str, dtype_b: str | None = None, profile: str = "ws1") -> float:
    """Fixed |dlogp| bound between a rollout and a training score computed in the given dtypes."""
    table = load_precision_profile(profile)["cross_config"]["fixed_threshold"]
    names = {"bf16": "bfloat16", "fp16": "float16", "fp32": "float32", "half": "float16", "float": "float32"}
    keys = [names.get(str(d).removeprefix("torch."), str(d).removeprefix("torch.")) for d in (dtype_a, dtype_b or dtype_a)]
    for k in keys:
        if k not in table:
            raise KeyError(f"no cross-config threshold for dtype {k!r}")
    return max(float(table[k]) for k in keys)


def chain_thresholds(profile: str = "ws1") -> dict:
    return dict(load_precision_profile(profile)["chain"])
