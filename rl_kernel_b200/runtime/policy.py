"""Run modes (parity: RLKernelMode, rl_engine/runtime/policy.py:13-80).

strict : every contract-bearing operator must be the deterministic kernel; any fallback raises.
audit  : deterministic kernels where available; fallbacks are allowed but reported.
auto   : like audit without route reports.
off    : reference operators only (the library changes nothing)."""
from __future__ import annotations

import enum
import os


class RLKernelMode(str, enum.Enum):
    STRICT = "strict"
    AUDIT = "audit"
    AUTO = "auto"
    OFF = "off"

    @classmethod
    def parse(cls, value: str | None) -> "RLKernelMode":
        if value is None or value == "":
            return cls.AUTO
        try:
            return cls(value.strip().lower())
        except ValueError as exc:
            raise ValueError(f"RL_KERNEL_MODE must be one of {[m.value for m in cls]}, got {value!r}") from exc


def current_mode() -> RLKernelMode:
    return RLKernelMode.parse(os.environ.get("RL_KERNEL_MODE"))


def strict_contract_enabled() -> bool:
    return current_mode() is RLKernelMode.STRICT


def route_report_enabled() -> bool:
    flag = os.environ.get("RL_KERNEL_ROUTE_REPORT")
    if flag is not None:
        return flag.strip() not in ("", "0", "false", "False")
    return current_mode() in (RLKernelMode.STRICT, RLKernelMode.AUDIT)


def route_report(module: str, requested: str, actual: str, fallback: bool) -> str:
    line = f"[RL-Kernel][route] mode={current_mode().value} module={module} requested={requested} actual={actual} fallback={int(fallback)}"
    if route_report_enabled():
        from rl_kernel_b200.utils.logger import info_once, init_logger

        info_once(init_logger(), line)
    return line
