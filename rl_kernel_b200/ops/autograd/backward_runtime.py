"""Records which backward implementation ran for an operator (parity: record_backward,
rl_engine/ops/autograd/backward_runtime.py:15-45)."""
from __future__ import annotations

import threading

_LOCK = threading.Lock()
_RECORDS: dict[str, dict] = {}


def record_backward(op_name: str, impl: str, **extra) -> None:
    with _LOCK:
        r = _RECORDS.setdefault(op_name, {"impl": impl, "count": 0})
        r["impl"] = impl
        r["count"] += 1
        r.update(extra)


def backward_records() -> dict[str, dict]:
    with _LOCK:
        return {k: dict(v) for k, v in _RECORDS.items()}


def reset() -> None:
    with _LOCK:
        _RECORDS.clear()
