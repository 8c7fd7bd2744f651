"""Strict JSON reading for run artifacts (parity: rl_engine/validation/cross_config/_json.py:13-44): duplicate keys,
NaN / Infinity constants and floats that overflow to infinity are errors, so that an artifact has one meaning."""
from __future__ import annotations

import json
import math
from typing import Any


def _unique(pairs: list[tuple[str, Any]]) -> dict[str, Any]:
    out: dict[str, Any] = {}
    for k, v in pairs:
        if k in out:
            raise ValueError(f"duplicate JSON object key {k!r}")
        out[k] = v
    return out


def _no_constant(name: str) -> Any:
    raise ValueError(f"non-finite JSON constant {name!r} is not allowed")


def _finite_float(text: str) -> float:
    v = float(text)
    if not math.isfinite(v):
        raise ValueError(f"JSON number {text!r} is not a finite float")
    return v


def strict_json_loads(value: str) -> Any:
    return json.loads(value, object_pairs_hook=_unique, parse_constant=_no_constant, parse_float=_finite_float)


def strict_json_dumps(value: Any, *, indent: int | None = None) -> str:
    return json.dumps(value, indent=indent, sort_keys=True, allow_nan=False)


__all__ = ["strict_json_dumps", "strict_json_loads"]
