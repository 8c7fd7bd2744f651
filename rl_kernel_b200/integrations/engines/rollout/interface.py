"""Rollout-engine side of the weight-sync protocol (parity: RolloutExecutor,
rl_engine/integrations/engines/rollout/interface.py:25-93): import -> install -> acknowledge, and on
any failure reject and keep serving the previous version."""
from __future__ import annotations

from rl_kernel_b200.integrations.common.weights import WeightInstallAdapter, WeightSyncError, WeightUpdateManifest


class RolloutExecutor:
    def __init__(self, bridge, installer: WeightInstallAdapter, generate_fn=None):
        self.bridge, self.installer, self.generate_fn = bridge, installer, generate_fn
        self.weight_version = -1
        self.active_update: str | None = None
        self.last_error: str | None = None

    def update_weights(self, manifest: WeightUpdateManifest) -> dict:
        if manifest.weight_version <= self.weight_version:
            reason = f"stale weight_version {manifest.weight_version} <= {self.weight_version}"
            self.bridge.reject(manifest.update_id, reason)
            self.last_error = reason
            return {"status": "rejected", "reason": reason, "weight_version": self.weight_version}
        try:
            tensors = self.bridge.import_update(manifest)
            self.installer.install(tensors, manifest)
        except Exception as exc:  # noqa: BLE001 - any failure keeps the previous version
            reason = f"{type(exc).__name__}: {exc}"
            self.bridge.reject(manifest.update_id, reason)
            self.last_error = reason
            return {"status": "rejected", "reason": reason, "weight_version": self.weight_version}
        self.bridge.acknowledge(manifest.update_id)
        self.weight_version, self.active_update = manifest.weight_version, manifest.update_id
        return {"status": "acknowledged", "weight_version": self.weight_version}

    def generate(self, *args, **kwargs):
        if self.generate_fn is None:
            raise WeightSyncError("no generate function bound")
        return self.generate_fn(*args, **kwargs)
