"""Framework-side runtime adapter: install the operators an IntegrationPlan asks for, route every call to the framework's
own operator or to this package's by the plan, keep evidence of what actually ran (hooks installed, calls, backend ids,
fallbacks, profiling-only calls, eager or captured execution), persist it as a read-back JSON per process and fail closed in
strict mode (parity: FrameworkOperatorIntegration, rl_engine/integrations/common/runtime.py:24-297).

Two ways to drive it.  A binding that owns the call site installs an operator and calls ``execute(module, *args)``.  A
binding that wraps a framework method keeps the framework's callable and calls ``route(module, native, *args)``: the plan
decides which of the two runs.  Both leave the same evidence; ``assert_strict_evidence`` is the check after a run and the
read-back files are what ``experiments/dense/validate_artifacts.py`` reads."""
from __future__ import annotations

import atexit
import json
import os
import threading
import time
from collections import Counter
from collections.abc import Callable, Mapping
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

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


MODULES = ("attention", "ffn", "logp")
EXECUTION_MODES = ("eager", "compiled_cuda_graph")
OWN_BACKEND_PREFIXES = ("rl_kernel_b200.", "b200", "rlkernel.", "pytorch-", "reference")
_FOREIGN_COMPILER_MARKERS = ("triton", "inductor")


@dataclass(frozen=True)
class ExecutionEvidence:
    """What one module last ran as, with its running call count (the ``operators`` section of a read-back)."""
    framework: str
    target: str
    module: str
    case_id: str
    implementation: str                 # "rl_kernel" or "production" (the framework's own operator)
    backend_id: str
    call_count: int
    execution_mode: str = "eager"
    provenance: Mapping[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        d = dict(self.__dict__)
        d["provenance"] = dict(self.provenance)
        return d


def _walk(value: Any, depth: int = 0):
    if depth > 6:
        return
    if isinstance(value, Mapping):
        for k, v in value.items():
            yield k, v
            yield from _walk(v, depth + 1)
    elif isinstance(value, (list, tuple)):
        for v in value:
            yield from _walk(v, depth + 1)


def _mentions_foreign_compiler(value: Any) -> bool:
    text = json.dumps(value, default=str).lower()
    return any(m in text for m in _FOREIGN_COMPILER_MARKERS)


def _reports_fallback(provenance: Any) -> bool:
    return any(k in ("fallback", "fell_back") and v is True for k, v in _walk(provenance))


def _is_profile_only(provenance: Any) -> bool:
    return any(k == "profile_only" and v is True for k, v in _walk(provenance))


def _actual_backend(provenance: Any) -> str | None:
    for k, v in _walk(provenance):
        if k == "actual_backend" and isinstance(v, str) and v:
            return v
    return None


def _runtime_platform(provenance: Any) -> str | None:
    for k, v in _walk(provenance):
        if k == "runtime_platform" and isinstance(v, str):
            return v
    return None


class FrameworkOperatorIntegration:
    def __init__(self, framework: str, side: str, plan: IntegrationPlan | None = None,
                 rl_kernel_operators: Mapping[str, Callable[..., Any]] | None = None):
        side = {"training": "train"}.get(side, side)
        if side not in ("rollout", "train"):
            raise ValueError(side)
        self.framework, self.side = framework, side
        self.target = "training" if side == "train" else "rollout"
        self.plan = plan or IntegrationPlan.from_env()
        self.session = semantic_catalog.session(f"{framework}:{side}")
        self.readbacks: dict[str, OperatorReadback] = {}
        self._operators: dict[str, object] = dict(rl_kernel_operators or {})
        self._lock = threading.Lock()
        self._counts: Counter[str] = Counter()
        self._profile_counts: Counter[str] = Counter()
        self._evidence: dict[str, ExecutionEvidence] = {}
        self._installed_hooks: dict[str, str] = {}
        self._fallbacks: list[dict[str, str]] = []
        self._reported_routes: set[str] = set()
        self._persisted_routes: dict[str, tuple] = {}
        if os.environ.get("RL_KERNEL_READBACK_DIR", "").strip():
            atexit.register(self.persist_readback)

    # ---- evidence-keeping API (what a wrapping binding calls)
    def _module(self, module: str) -> str:
        m = module.strip().lower()
        if m not in MODULES:
            raise ValueError(f"unknown integration module {module!r}")
        return m

    def uses_rl_kernel(self, module: str) -> bool:
        return bool(self.plan.side(self.side).get(self._module(module), False))

    def install_operator(self, module: str, operator: Callable[..., Any]) -> None:
        m = self._module(module)
        if not callable(operator):
            raise TypeError("operator must be callable")
        with self._lock:
            self._operators[m] = operator

    def record_installed_hook(self, module: str, hook_id: str) -> None:
        """The framework method ``hook_id`` now goes through this integration (evidence that the patch took)."""
        m = self._module(module)
        if not isinstance(hook_id, str) or not hook_id.strip():
            raise ValueError("hook_id must be a non-empty string")
        with self._lock:
            self._installed_hooks[m] = hook_id.strip()
        self.persist_readback()

    def record_fallback(self, module: str, reason: str) -> None:
        m = self._module(module)
        with self._lock:
            self._fallbacks.append({"module": m, "reason": str(reason)})
        self.persist_readback()

    def record_profile_call(self, module: str) -> None:
        """A shape / memory profiling pass of the framework went through the hook: counted, not taken for execution."""
        m = self._module(module)
        with self._lock:
            self._profile_counts[m] += 1
            first = self._profile_counts[m] == 1
        if first:
            self.persist_readback()

    def record_execution(self, module: str, selected: Callable[..., Any], *, execution_mode: str = "eager",
                         execution_provenance: Mapping[str, Any] | None = None) -> None:
        """One eager call, or one call inside a captured graph, of ``selected`` for ``module``."""
        m = self._module(module)
        own = self.uses_rl_kernel(m)
        if own and selected is not self._operators.get(m):
            raise RuntimeError(f"{self.framework} {m} execution evidence did not use the installed RL-Kernel operator")
        if execution_mode not in EXECUTION_MODES:
            raise ValueError(f"unknown execution mode {execution_mode!r}")
        backend_id = getattr(selected, "backend_id", None)
        if not isinstance(backend_id, str) or not backend_id.strip():
            backend_id = f"rl_kernel_b200.{m}.unidentified" if own else f"{self.framework}.production.{m}"
        if execution_provenance is None:
            raw = getattr(selected, "provenance", {})
            provenance = dict(raw) if isinstance(raw, Mapping) else {}
        else:
            provenance = dict(execution_provenance)
        actual = _actual_backend(provenance) or backend_id
        fallback = _reports_fallback(provenance)
        route = ("rl_kernel" if own else "production", backend_id, actual, fallback, _runtime_platform(provenance))
        with self._lock:
            self._counts[m] += 1
            self._evidence[m] = ExecutionEvidence(self.framework, self.target, m, str(getattr(self.plan, m)), route[0], backend_id,
                                                  self._counts[m], execution_mode, provenance)
            report = m not in self._reported_routes
            self._reported_routes.add(m)
            changed = self._persisted_routes.get(m) != route
            self._persisted_routes[m] = route
        if changed:
            self.persist_readback()
        if report:
            from rl_kernel_b200.runtime.policy import route_report

            route_report(f"{self.framework}/{self.target}/{m}", route[0], actual, fallback)
        if own and fallback:
            self.record_fallback(m, f"operator provenance selected {actual}")
            raise RuntimeError(f"{self.framework} {m} strict RL-Kernel route reported fallback")

    def route(self, module: str, native: Callable[..., Any], *args: Any, **kwargs: Any) -> Any:
        """Run ``native`` (the framework's own callable) or the installed operator, whichever the plan selects for this
        side, and keep the evidence."""
        m = self._module(module)
        if not callable(native):
            raise TypeError("native operator must be callable")
        if self.uses_rl_kernel(m):
            selected = self._operators.get(m)
            if selected is None:
                raise RuntimeError(f"{self.framework} {m} selected RL-Kernel but no operator was installed")
        else:
            selected = native
        result = selected(*args, **kwargs)
        if _is_profile_only(getattr(selected, "provenance", {})):
            self.record_profile_call(m)
        else:
            self.record_execution(m, selected)
        return result

    def assert_strict_evidence(self, *, require_cuda: bool = True) -> None:
        """After a run: every module the plan gives to RL-Kernel was hooked, was called, ran one of this package's
        backends on the GPU without a tracing compiler, and nothing fell back."""
        rb = self.readback()
        problems: list[str] = []
        wanted = [m for m in MODULES if self.uses_rl_kernel(m)]
        hooks = [m for m in wanted if m not in rb["installed_hooks"]]
        calls = [m for m in wanted if int(rb["operators"].get(m, {}).get("call_count", 0)) <= 0]
        wrong = []
        for m in wanted:
            op = rb["operators"].get(m)
            if op is None:
                continue
            if not str(op["backend_id"]).startswith(OWN_BACKEND_PREFIXES):
                wrong.append(f"{m}={op['backend_id']}")
            elif _mentions_foreign_compiler(op):
                wrong.append(f"{m}=tracing-compiler")
            elif require_cuda and _runtime_platform(op.get("provenance")) not in ("cuda",):
                wrong.append(f"{m}=non-cuda")
        if hooks:
            problems.append("missing hooks: " + ", ".join(hooks))
        if calls:
            problems.append("zero calls: " + ", ".join(calls))
        if wrong:
            problems.append("unexpected backends: " + ", ".join(wrong))
        if rb["fallbacks"]:
            problems.append(f"fallbacks: {rb['fallbacks']}")
        if problems:
            raise RuntimeError(f"{self.framework} {self.target} integration is not strict-ready: " + "; ".join(problems))

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
        with self._lock:
            operators = {m: e.to_dict() for m, e in self._evidence.items()}
            # modules driven through install()/execute() count as evidence too
            for m, r in self.readbacks.items():
                if m not in operators and r.calls:
                    op = self._operators.get(m)
                    operators[m] = ExecutionEvidence(self.framework, self.target, m, str(getattr(self.plan, m)), "rl_kernel",
                                                     str(getattr(op, "backend_id", r.actual)), r.calls, "eager",
                                                     dict(getattr(op, "provenance", {}) or {})).to_dict()
            return {"framework": self.framework, "side": self.side, "target": self.target, "plan": self.plan.describe(),
                    "plan_cases": self.plan.to_env(), "mode": current_mode().value,
                    "modules": {m: asdict(r) for m, r in self.readbacks.items()}, "installed_hooks": dict(self._installed_hooks),
                    "fallbacks": list(self._fallbacks) + [{"module": m, "reason": f"installed as a fallback ({r.actual})"}
                                                          for m, r in self.readbacks.items() if r.fallback],
                    "profile_calls": dict(self._profile_counts), "operators": operators, "session": self.session.readback()}

    def persist_readback(self, directory: str | os.PathLike | None = None) -> Path | None:
        directory = directory or os.environ.get("RL_KERNEL_READBACK_DIR")
        if not directory:
            return None
        path = Path(directory)
        path.mkdir(parents=True, exist_ok=True)
        out = path / f"{self.framework}-{self.target}-{os.getpid()}.json"
        tmp = out.with_suffix(".tmp")                      # written beside the target and renamed: readers never see half a file
        tmp.write_text(json.dumps(self.readback(), indent=1, sort_keys=True, default=str))
        tmp.replace(out)
        return out
