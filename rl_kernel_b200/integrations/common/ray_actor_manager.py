"""Ray actor manager for rollout / training workers; Ray is imported lazily so that a stand-in
module can be injected (parity: RayActorManager, rl_engine/integrations/common/ray_actor_manager.py:75-223)."""
from __future__ import annotations

from dataclasses import dataclass


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


class RayActorManager:
    def __init__(self, ray_module=None, num_gpus_per_worker: float = 1.0):
        if ray_module is None:
            import ray as ray_module  # noqa: PLC0415 - optional dependency
        self.ray, self.num_gpus = ray_module, num_gpus_per_worker
        self.workers: dict[str, WorkerHandle] = {}

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
