"""Process-local integration state (parity: rl_engine/integrations/common/state.py:14-57).  Ray actors and serving workers
are separate processes: each owns one integration object per framework, and the orchestrator-side providers find it
here so that their calls are counted in the same read-back."""
from __future__ import annotations

from threading import Lock
from typing import Literal

from rl_kernel_b200.integrations.common.runtime import FrameworkOperatorIntegration

FrameworkName = Literal["megatron", "vllm", "deepspeed"]
_ACTIVE: dict[str, FrameworkOperatorIntegration] = {}
_LOCK = Lock()


def set_active_integration(framework: str, integration: FrameworkOperatorIntegration) -> None:
    if integration.framework != framework:
        raise ValueError(f"integration framework {integration.framework!r} does not match {framework!r}")
    with _LOCK:
        existing = _ACTIVE.get(framework)
        if existing is not None and existing is not integration:
            raise RuntimeError(f"a {framework} integration is already installed in this process")
        _ACTIVE[framework] = integration


def get_active_integration(framework: str) -> FrameworkOperatorIntegration | None:
    with _LOCK:
        return _ACTIVE.get(framework)


def clear_active_integration(framework: str) -> None:
    with _LOCK:
        _ACTIVE.pop(framework, None)


__all__ = ["FrameworkName", "clear_active_integration", "get_active_integration", "set_active_integration"]
