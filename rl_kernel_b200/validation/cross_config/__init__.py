"""Plan and run cross-configuration alignment experiments.  The package root stays small: the planning types load
eagerly, the runner and the runtime materialisers on first use (parity: rl_engine/validation/cross_config/__init__.py)."""
from importlib import import_module

_LAZY = {
    "compare_score_artifacts": "comparison", "ExperimentConfig": "config", "load_config": "config",
    "ExecutionPlan": "execution_plan", "build_execution_plan": "execution_plan", "ExperimentPlan": "planner", "Planner": "planner",
    "PairedRunResult": "runner", "PairedRunner": "runner", "run_alignment": "runner", "run_experiment": "runner",
    "RuntimeMaterializer": "runtime", "RuntimeTools": "runtime", "ArtifactStore": "artifacts", "ArtifactError": "artifacts",
}


def __getattr__(name: str):
    if name in _LAZY:
        return getattr(import_module(f"{__name__}.{_LAZY[name]}"), name)
    raise AttributeError(name)


__all__ = sorted(_LAZY)
