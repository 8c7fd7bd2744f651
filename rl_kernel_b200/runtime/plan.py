"""Integration plan: which side (rollout / train) uses the deterministic operators for which
module.  "R" = RL-Kernel strict operator, "P" = the framework's own operator; the four cases
P/P, R/R, P/R, R/P are read from RL_KERNEL_{ATTENTION,FFN,LOGP}_CASE
(parity: IntegrationPlan, rl_engine/runtime/plan.py:50-164)."""
from __future__ import annotations

import os
from dataclasses import dataclass

_CASES = ("P/P", "R/R", "P/R", "R/P")
_MODULES = ("attention", "ffn", "logp")


@dataclass(frozen=True)
class ModuleCase:
    rollout: str
    train: str

    @classmethod
    def parse(cls, text: str) -> "ModuleCase":
        t = text.strip().upper()
        if t not in _CASES:
            raise ValueError(f"case must be one of {_CASES}, got {text!r}")
        return cls(*t.split("/"))

    @property
    def strict_both(self) -> bool:
        return self.rollout == "R" and self.train == "R"

    def __str__(self) -> str:
        return f"{self.rollout}/{self.train}"


@dataclass(frozen=True)
class IntegrationPlan:
    attention: ModuleCase
    ffn: ModuleCase
    logp: ModuleCase

    @classmethod
    def from_env(cls, env: dict | None = None, default: str = "R/R") -> "IntegrationPlan":
        env = os.environ if env is None else env
        return cls(*(ModuleCase.parse(env.get(f"RL_KERNEL_{m.upper()}_CASE", default)) for m in _MODULES))

    @classmethod
    def uniform(cls, case: str) -> "IntegrationPlan":
        c = ModuleCase.parse(case)
        return cls(c, c, c)

    def side(self, side: str) -> dict[str, bool]:
        """{module: uses RL-Kernel operator} for 'rollout' or 'train'."""
        if side not in ("rollout", "train"):
            raise ValueError(side)
        return {m: getattr(getattr(self, m), side) == "R" for m in _MODULES}

    @property
    def bitwise_guarantee(self) -> bool:
        """Train-rollout bit equality is only promised when every module is R on both sides."""
        return all(getattr(self, m).strict_both for m in _MODULES)

    def to_env(self) -> dict[str, str]:
        return {f"RL_KERNEL_{m.upper()}_CASE": str(getattr(self, m)) for m in _MODULES}

    def describe(self) -> str:
        return " ".join(f"{m}={getattr(self, m)}" for m in _MODULES)
