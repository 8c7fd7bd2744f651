"""Rollout-engine side of the weight-sync protocol and the rollout entry points
(parity: RolloutExecutor, rl_engine/integrations/engines/rollout/interface.py:25-194).

``update_weights(manifest)``: import -> install -> acknowledge; on any failure the update is
rejected, the previous version stays active and the error is raised.  After a successful switch the
superseded update is released.  ``try_update_weights`` is the same without the raise: it returns a
status record, which is what an orchestrator loop usually wants.
"""
from __future__ import annotations

from typing import Any, Mapping, Optional, Sequence

import torch

from rl_kernel_b200.integrations.common.weights import (WeightBridgeUnavailableError, WeightConsumer,
                                                         WeightInstallAdapter, WeightUpdateManifest,
                                                         WeightUpdateRejectedError, make_weight_bridge)
from rl_kernel_b200.utils.logger import logger


class RolloutExecutor:
    def __init__(self, model_config: Optional[dict] = None, *, weight_bridge: Optional[WeightConsumer] = None,
                 weight_transport: Optional[str] = None, weight_install_adapter: Optional[WeightInstallAdapter] = None,
                 generate_fn=None, sampler=None):
        self.config = dict(model_config or {})
        default_transport = "cuda-vmm" if torch.cuda.is_available() else "local-clone"
        transport = weight_transport or str(self.config.get("weight_transport", default_transport))
        self.bridge = weight_bridge or make_weight_bridge(transport)
        self.weight_install_adapter = weight_install_adapter
        self.shared_weights: dict[str, torch.Tensor] = {}
        self.active_weight_version: Optional[int] = None
        self.active_weight_update_id: Optional[str] = None
        self.last_error: Optional[str] = None
        self.generate_fn, self.sampler = generate_fn, sampler
        self.logp_op = self.attn_op = None
        from rl_kernel_b200.runtime.registry import resolve_logp_op_type

        self.logp_op_type = resolve_logp_op_type(self.config.get("logp_backend") or "auto",
                                                 require_batch_invariant=bool(self.config.get("require_batch_invariant_logp", False)))

    # the earlier attribute name of the active version
    @property
    def weight_version(self) -> int:
        return -1 if self.active_weight_version is None else self.active_weight_version

    @weight_version.setter
    def weight_version(self, v: int) -> None:
        self.active_weight_version = None if v is None or v < 0 else int(v)

    # ---------------------------------------------------------------- weights
    def update_weights(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]:
        logger.info("Importing weight update %s version=%s transport=%s", manifest.update_id, manifest.weight_version,
                    manifest.transport)
        previous = self.active_weight_update_id
        try:
            if self.active_weight_version is not None and manifest.weight_version <= self.active_weight_version:
                raise WeightUpdateRejectedError(
                    f"stale weight_version {manifest.weight_version} <= active {self.active_weight_version}")
            imported = dict(self.bridge.import_update(manifest))
            if self.weight_install_adapter is not None:
                self.weight_install_adapter.install(manifest, imported)
            self.bridge.acknowledge(manifest.update_id)
        except Exception as exc:
            self.last_error = f"{type(exc).__name__}: {exc}"
            try:
                self.bridge.reject(manifest.update_id, f"rollout weight install failed: {exc}")
            except Exception:  # noqa: BLE001 - the original error is the one to report
                logger.exception("Failed to reject weight update %s", manifest.update_id)
            raise
        self.shared_weights = imported
        self.active_weight_version, self.active_weight_update_id = manifest.weight_version, manifest.update_id
        if previous is not None and previous != manifest.update_id:
            self.release_weight_update(previous)
        return self.shared_weights

    def try_update_weights(self, manifest: WeightUpdateManifest) -> dict:
        try:
            self.update_weights(manifest)
        except Exception as exc:  # noqa: BLE001 - reported in the record
            return {"status": "rejected", "reason": f"{type(exc).__name__}: {exc}", "weight_version": self.weight_version}
        return {"status": "acknowledged", "weight_version": self.weight_version}

    def release_weights(self) -> None:
        if self.active_weight_update_id is not None:
            self.release_weight_update(self.active_weight_update_id)

    def release_weight_update(self, update_id: str) -> None:
        if self.weight_install_adapter is not None:
            self.weight_install_adapter.release(update_id)
        self.bridge.release(update_id)
        if self.active_weight_update_id == update_id:
            self.shared_weights = {}
            self.active_weight_update_id = None

    def update_weights_via_ipc(self, ipc_handles: Mapping[str, Any]):
        """Raw handle imports are refused: a manifest carries the version, the descriptors and the
        acknowledgement / release lifecycle that a bare handle table lacks."""
        del ipc_handles
        raise WeightBridgeUnavailableError("publish a WeightUpdateManifest and call update_weights(manifest)")

    # ---------------------------------------------------------------- rollout
    def _prepare_kernels(self) -> None:
        if self.logp_op is None:
            from rl_kernel_b200.runtime.registry import kernel_registry

            self.logp_op = kernel_registry.get_op(self.logp_op_type)
            self.attn_op = kernel_registry.get_op("attn")

    def generate_candidates(self, prompts, *, num_generations: Optional[int] = None,
                            sampling_params: Optional[Mapping[str, Any]] = None) -> dict[str, Any]:
        """GRPO candidates through the bound shared-prefix sampler (the prompt is prefilled once per group)."""
        if self.sampler is None:
            raise WeightBridgeUnavailableError("no sampler bound: pass sampler=SharedPrefixSampler(...)")
        return self.sampler.generate(prompts, num_generations=num_generations, sampling_params=sampling_params)

    def generate(self, *args, **kwargs):
        if self.generate_fn is None:
            raise WeightBridgeUnavailableError("no generate function bound")
        return self.generate_fn(*args, **kwargs)

    def execute_rollout(self, input_ids: torch.Tensor) -> dict[str, Any]:
        self._prepare_kernels()
        return {"status": "success", "device": str(input_ids.device), "logp_op": type(self.logp_op).__name__,
                "attn_op": type(self.attn_op).__name__}
