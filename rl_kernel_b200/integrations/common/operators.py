"""Handles that bind a semantic operator to a framework call site and keep its contract
(parity: SemanticOperatorHandle, rl_engine/integrations/common/operators.py:98)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class SemanticOperatorHandle:
    semantic_op: str
    operator: object
    contract: object | None = None
    module: str = ""
    calls: int = field(default=0)

    def __call__(self, *a, **k):
        self.calls += 1
        return self.operator(*a, **k)

    def fingerprint(self) -> str | None:
        return self.contract.cross_rank_fingerprint() if self.contract is not None else None
