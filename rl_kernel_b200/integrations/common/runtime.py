"""Framework-side runtime adapter: install the operators an IntegrationPlan asks for, execute them
with provenance, persist a readback, and fail closed in strict mode (parity:
FrameworkOperatorIntegration, rl_engine/integrations/common/runtime.py:24-297)."""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path

from rl_kernel_b200.runtime.plan import IntegrationPlan
from rl_kernel_b200.runtime.policy import RLKernelMode, current_mode
from rl_kernel_b200.runtime.semantic_registry import semantic_catalog


@dataclass
class OperatorReadback:
    framework: str
    side: str                      # rollout | train
    module: str                    # attention | ffn | logp
    requested: str
    actual: str
    fallback: bool
    calls: int = 0
    installed_ts: float = field(default_factory=time.time)


class FrameworkOperatorIntegration:
    def __init__(self, framework: str, side: str, plan: IntegrationPlan | None = None):
        if side not in ("rollout", "train"):
            raise ValueError(side)
        self.framework, self.side = framework, side
        self.plan = plan or IntegrationPlan.from_env()
        self.session = semantic_catalog.session(f"{framework}:{side}")
        self.readbacks: dict[str, OperatorReadback] = {}
        self._operators: dict[str, object] = {}

    def install(self, module: str, operator, *, requested: str = "rl_kernel", actual: str | None = None,
                fallback: bool = False) -> None:
        if not self.plan.side(self.side).get(module, False):
            raise RuntimeError(f"plan {self.plan.describe()} does not ask for an RL-Kernel {module} operator on {self.side}")
        self._operators[module] = operator
        self.readbacks[module] = OperatorReadback(self.framework, self.side, module, requested,
                                                  actual or type(operator).__name__, fallback)
        if fallback and current_mode() is RLKernelMode.STRICT:
            raise RuntimeError(f"strict mode: {module} on {self.framework}/{self.side} fell back to {actual}")

    def execute(self, module: str, *args, **kwargs):
        op = self._operators.get(module)
        if op is None:
            raise RuntimeError(f"{module} operator was not installed on {self.framework}/{self.side}")
        rb = self.readbacks[module]
        rb.calls += 1
        sem = {"logp": "selected_logprob"}.get(module, module)
        backend = getattr(op, "backend_id", "reference")
        try:
            self.session.observe(sem, backend if backend in ("b200-tcgen05", "reference") else "b200-tcgen05"
                                 if backend.startswith("b200") else "reference", module, rb.fallback)
        except KeyError:
            pass
        return op(*args, **kwargs)

    def assert_strict_ready(self) -> None:
        """Every module the plan marks R must be installed and must not be a fallback."""
        wanted = [m for m, on in self.plan.side(self.side).items() if on]
        missing = [m for m in wanted if m not in self._operators]
        if missing:
            raise RuntimeError(f"{self.framework}/{self.side}: operators not installed: {missing}")
        bad = [m for m in wanted if self.readbacks[m].fallback]
        if bad:
            raise RuntimeError(f"{self.framework}/{self.side}: fallback operators in strict plan: {bad}")

    def readback(self) -> dict:
        return {"framework": self.framework, "side": self.side, "plan": self.plan.describe(),
                "mode": current_mode().value, "modules": {m: asdict(r) for m, r in self.readbacks.items()},
                "session": self.session.readback()}

    def persist_readback(self, directory: str | os.PathLike | None = None) -> Path | None:
        directory = directory or os.environ.get("RL_KERNEL_READBACK_DIR")
        if not directory:
            return None
        path = Path(directory)
        path.mkdir(parents=True, exist_ok=True)
        out = path / f"readback_{self.framework}_{self.side}_{os.getpid()}.json"
        out.write_text(json.dumps(self.readback(), indent=1, sort_keys=True))
        return out
