"""Ray actor manager for rollout / training workers; Ray is imported lazily so that a stand-in
module can be injected (parity: RayActorManager, rl_engine/integrations/common/ray_actor_manager.py:75-223)."""
from __future__ import annotations

from collections.abc import Mapping, Sequence
from dataclasses import dataclass, field
from typing import Any


class RayUnavailableError(RuntimeError):
    """The optional Ray runtime cannot be imported here."""


def load_ray():
    try:
        import ray  # noqa: PLC0415 - optional dependency
    except ImportError as exc:
        raise RayUnavailableError("Ray is not installed; pass ray_module= (or install ray) to host workers in actors") from exc
    return ray


@dataclass(frozen=True)
class RayRuntimeConfig:
    """How the manager treats the Ray runtime: start it on first use (``ray.init`` with ``ignore_reinit_error`` so that an
    already running cluster is reused) and whether to stop it when the manager closes."""
    auto_init: bool = True
    init_kwargs: Mapping[str, Any] = field(default_factory=dict)
    shutdown_ray_on_close: bool = False

    def resolved_init_kwargs(self) -> dict[str, Any]:
        return {"ignore_reinit_error": True, **dict(self.init_kwargs)}


@dataclass(frozen=True)
class RayActorOptions:
    """Resources and lifecycle of one actor; unset fields are left to Ray's defaults."""
    num_cpus: float | None = None
    num_gpus: float | None = None
    resources: Mapping[str, float] = field(default_factory=dict)
    name: str | None = None
    namespace: str | None = None
    max_restarts: int | None = None
    max_task_retries: int | None = None
    scheduling_strategy: Any = None
    lifetime: str | None = None

    def to_ray_options(self) -> dict[str, Any]:
        out = {k: getattr(self, k) for k in ("num_cpus", "num_gpus", "name", "namespace", "max_restarts", "max_task_retries",
                                             "scheduling_strategy", "lifetime") if getattr(self, k) is not None}
        if self.resources:
            out["resources"] = dict(self.resources)
        return out


@dataclass(frozen=True)
class RayWorkerSpec:
    """Factory and constructor arguments of a worker that lives in an actor."""
    worker_factory: Any
    args: Sequence[Any] = field(default_factory=tuple)
    kwargs: Mapping[str, Any] = field(default_factory=dict)
    actor_options: RayActorOptions = field(default_factory=RayActorOptions)


@dataclass
class WorkerHandle:
    name: str
    actor: object
    kind: str


class _RayWorkerActor:
    """Body of the remote actor: owns one worker object and forwards calls to it."""

    def __init__(self, factory, *args, **kwargs):
        self.worker = factory(*args, **kwargs)

    def call(self, method: str, *args, **kwargs):
        return getattr(self.worker, method)(*args, **kwargs)

    def health(self) -> bool:
        return True

    def health_check(self) -> dict:
        """Identity of the hosted worker plus whatever its own ``health_check`` says."""
        import os

        info = {"ok": True, "worker_type": type(self.worker).__name__, "pid": os.getpid()}
        own = getattr(self.worker, "health_check", None)
        if callable(own):
            info["worker"] = own()
        return info


class _TypedHandle:
    """Calls on a hosted worker by method name, resolved through ``ray.get``."""

    def __init__(self, actor: Any, ray_module: Any):
        self.actor, self._ray = actor, ray_module

    def _call(self, method: str, *args, **kwargs):
        return self._ray.get(self.actor.call.remote(method, *args, **kwargs))

    def health_check(self):
        return self._ray.get(self.actor.health.remote())


class RayRolloutWorkerHandle(_TypedHandle):
    def rollout(self, spec):
        return self._call("rollout", spec)

    def update_weights(self, manifest):
        return self._call("update_weights", manifest)

    def release_weights(self):
        return self._call("release_weights")


class RayTrainingWorkerHandle(_TypedHandle):
    def train(self, rollout):
        return self._call("train", rollout)

    def publish_weights(self, weight_version: int, **kwargs):
        return self._call("publish_weights", weight_version, **kwargs)

    def release_weights(self, update_id: str):
        return self._call("release_weights", update_id)


class RayActorManager:
    def __init__(self, ray_module=None, num_gpus_per_worker: float = 1.0, runtime: RayRuntimeConfig | None = None):
        self.ray = ray_module if ray_module is not None else load_ray()
        self.num_gpus = num_gpus_per_worker
        self.runtime = runtime or RayRuntimeConfig()
        self.workers: dict[str, WorkerHandle] = {}
        self._started = False

    def __enter__(self) -> "RayActorManager":
        self.ensure_runtime()
        return self

    def __exit__(self, *exc) -> None:
        self.shutdown()

    def ensure_runtime(self):
        """Start Ray once if the config asks for it and it is not running yet."""
        if not self._started and self.runtime.auto_init and hasattr(self.ray, "init"):
            running = getattr(self.ray, "is_initialized", lambda: False)()
            if not running:
                self.ray.init(**self.runtime.resolved_init_kwargs())
            self._started = True
        return self.ray

    def create_worker_actor(self, spec: RayWorkerSpec, *, name: str | None = None, kind: str = "worker") -> WorkerHandle:
        """An actor from a spec; its options (resources, restarts, placement) come from ``spec.actor_options``."""
        self.ensure_runtime()
        opts = spec.actor_options.to_ray_options()
        opts.setdefault("num_gpus", self.num_gpus)
        name = name or opts.get("name") or f"{kind}-{len(self.workers)}"
        if name in self.workers:
            raise ValueError(f"worker {name!r} already exists")
        actor = self.ray.remote(**opts)(_RayWorkerActor).remote(spec.worker_factory, *spec.args, **dict(spec.kwargs))
        self.workers[name] = WorkerHandle(name, actor, kind)
        return self.workers[name]

    def create_rollout_worker(self, spec: RayWorkerSpec, *, name: str | None = None) -> RayRolloutWorkerHandle:
        return RayRolloutWorkerHandle(self.create_worker_actor(spec, name=name, kind="rollout").actor, self.ray)

    def create_training_worker(self, spec: RayWorkerSpec, *, name: str | None = None) -> RayTrainingWorkerHandle:
        return RayTrainingWorkerHandle(self.create_worker_actor(spec, name=name, kind="training").actor, self.ray)

    def spawn(self, name: str, kind: str, factory, *args, **kwargs) -> WorkerHandle:
        if name in self.workers:
            raise ValueError(f"worker {name!r} already exists")
        remote_cls = self.ray.remote(num_gpus=self.num_gpus)(_RayWorkerActor)
        handle = WorkerHandle(name, remote_cls.remote(factory, *args, **kwargs), kind)
        self.workers[name] = handle
        return handle

    def call(self, name: str, method: str, *args, **kwargs):
        return self.ray.get(self.workers[name].actor.call.remote(method, *args, **kwargs))

    def broadcast(self, kind: str, method: str, *args, **kwargs) -> dict:
        refs = {n: h.actor.call.remote(method, *args, **kwargs) for n, h in self.workers.items() if h.kind == kind}
        return {n: self.ray.get(r) for n, r in refs.items()}

    def publish_weights(self, trainer: str, rollout_kind: str = "rollout", weight_version: int = 0) -> dict:
        manifest = self.call(trainer, "publish_weights", weight_version)
        return self.broadcast(rollout_kind, "update_weights", manifest)

    def health_check(self) -> dict[str, bool]:
        out = {}
        for n, h in self.workers.items():
            try:
                out[n] = bool(self.ray.get(h.actor.health.remote()))
            except Exception:  # noqa: BLE001 - a dead actor is reported, not raised
                out[n] = False
        return out

    def shutdown(self) -> None:
        for h in self.workers.values():
            try:
                self.ray.kill(h.actor)
            except Exception:  # noqa: BLE001
                pass
        self.workers.clear()
        if self._started and self.runtime.shutdown_ray_on_close and hasattr(self.ray, "shutdown"):
            self.ray.shutdown()
        self._started = False
