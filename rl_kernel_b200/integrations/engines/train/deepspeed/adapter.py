"""DeepSpeed-style training worker: wraps an engine object exposing ``backward`` / ``step`` and a
module, trains on a rollout with the strict log-prob + GRPO operators, and publishes a full
(ZeRO-gathered) state through the weight bridge (parity: DeepSpeedTrainingWorker,
rl_engine/integrations/engines/train/deepspeed/adapter.py:74-316)."""
from __future__ import annotations

import torch

from rl_kernel_b200.integrations.common.weights import WeightPublisher
from rl_kernel_b200.integrations.engines.train.contract import (RolloutBatchMixin, RolloutStageResult,
                                                                 TrainingStageResult)
from rl_kernel_b200.ops.loss import grpo_loss
from rl_kernel_b200.ops.logprob import linear_logp


def gather_zero3_parameter(param, group=None) -> torch.Tensor:
    """Assemble a ZeRO-3 partitioned parameter: every rank of ``group`` holds ``param.ds_tensor`` (a flat slice, the last
    one zero-padded); the whole is their concatenation in rank order cut to ``ds_numel`` and shaped ``ds_shape``.
    Without an initialised process group the local partition must already be the whole parameter."""
    import torch.distributed as dist

    part = param.ds_tensor.detach().reshape(-1)
    numel = int(getattr(param, "ds_numel", part.numel()))
    shape = tuple(getattr(param, "ds_shape", param.shape))
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        parts = [torch.empty_like(part) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, part.contiguous(), group=group)
        flat = torch.cat(parts)
    else:
        flat = part
    if flat.numel() < numel:
        raise ValueError(f"partitions hold {flat.numel()} elements, the parameter has {numel}")
    return flat[:numel].reshape(shape).clone()


class DeepSpeedTrainingWorker(RolloutBatchMixin):
    def __init__(self, engine, publisher: WeightPublisher, *, hidden_fn=None, lm_head_name: str = "lm_head.weight",
                 clip_eps: float = 0.2, kl_coef: float = 0.0, temperature: float = 1.0, ref_scorer=None,
                 gather_context=None):
        self.engine, self.publisher = engine, publisher
        self.hidden_fn = hidden_fn or (lambda module, ids: module(ids))
        self.lm_head_name, self.clip_eps, self.kl_coef, self.temperature = lm_head_name, clip_eps, kl_coef, temperature
        self.ref_scorer, self.gather_context = ref_scorer, gather_context
        self.weight_version = 0

    def _lm_head(self):
        return dict(self.engine.module.named_parameters())[self.lm_head_name]

    def train(self, rollout: RolloutStageResult) -> TrainingStageResult:
        rollout.validate()
        P, R = rollout.prompt_len, rollout.rollout_logp.shape[1]
        hidden = self.hidden_fn(self.engine.module, rollout.tokens)            # [B, S, H]
        rows = hidden[:, P - 1:P - 1 + R]
        logp = linear_logp(rows, self._lm_head(), rollout.tokens[:, P:], self.temperature)
        ref = self.ref_scorer.score(rollout) if self.ref_scorer is not None and self.kl_coef > 0 else None
        adv = self.advantages(rollout)
        loss, pol, kl = grpo_loss(logp, rollout.rollout_logp, ref, adv, rollout.response_mask, clip_eps=self.clip_eps,
                                  beta=self.kl_coef)
        self.engine.backward(loss)
        self.engine.step()
        gn = getattr(self.engine, "get_global_grad_norm", lambda: 0.0)() or 0.0
        return TrainingStageResult(float(loss.detach()), float(pol.detach()), float(kl.detach()), float(gn), logp.detach(),
                                   self.mismatches(logp.detach(), rollout), int(rollout.response_mask.sum()),
                                   self.weight_version)

    def _full_state(self) -> dict[str, torch.Tensor]:
        """The whole model on every rank.  ZeRO-3 keeps only a 1 / dp flat partition of every parameter on a rank
        (``param.ds_tensor``; ``ds_shape`` / ``ds_numel`` describe the whole).  Order of preference: an injected
        ``gather_context`` (``deepspeed.zero.GatheredParameters``), else this worker's own rank-ordered all-gather of the
        partitions, else the state dict as it is (ZeRO stage 0-2: parameters are whole)."""
        module = self.engine.module
        params = dict(module.named_parameters())
        partitioned = {k: p for k, p in params.items() if hasattr(p, "ds_tensor")}
        if self.gather_context is not None:
            with self.gather_context(module.parameters()):
                return {k: v.detach().clone() for k, v in module.state_dict().items()}
        state = {k: v.detach().clone() for k, v in module.state_dict().items() if k not in partitioned}
        for name, p in partitioned.items():
            state[name] = gather_zero3_parameter(p, getattr(self.engine, "dp_process_group", None) or getattr(p, "ds_process_group", None))
        return state

    def publish_weights(self, weight_version: int):
        if weight_version <= self.weight_version and self.weight_version != 0:
            raise ValueError("weight_version must increase")
        self.weight_version = weight_version
        return self.publisher.publish(self._full_state(), weight_version, {"layout": {"kind": "full-state"}, "source": "deepspeed"})
