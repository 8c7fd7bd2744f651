"""GRPO / PPO clipped surrogate with group-normalised advantages and the k3 KL penalty
(parity: NativeGRPOLossOp, rl_engine/reference/loss/grpo_loss.py:12-129)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from rl_kernel_b200.reference.loss.ratio_kl import NativeRatioKLOp, ratio_kl_from_logps


def _masked_mean(x, mask):
    m = mask.to(x.dtype)
    return (x * m).sum() / m.sum().clamp_min(1.0)


def grpo_loss_from_logps(logp, old_logp, ref_logp, sample_adv, mask, *, clip_eps: float = 0.2,
                         beta: float = 0.0, clip_eps_high: float | None = None, denominator: float | None = None):
    """(loss, policy_loss, kl) from per-token log-probs; gradients flow into ``logp``.  ``denominator`` replaces the
    call's own active-token count (a micro-batch passes the step's global count)."""
    hi = clip_eps if clip_eps_high is None else clip_eps_high
    ratio, kl = ratio_kl_from_logps(logp, old_logp, ref_logp, mask)
    m = mask.bool()
    adv = sample_adv.reshape(-1, 1).expand_as(m).float().masked_fill(~m, 0.0)
    pol = -torch.minimum(ratio * adv, torch.clamp(ratio, 1.0 - clip_eps, 1.0 + hi) * adv)
    if denominator is None:
        policy_loss, klm = _masked_mean(pol, m), _masked_mean(kl, m)
    else:
        inv = 1.0 / float(denominator)
        policy_loss, klm = (pol * m).sum() * inv, (kl * m).sum() * inv
    return policy_loss + beta * klm, policy_loss, klm


class NativeGRPOLossOp:
    def __init__(self):
        self._ratio_kl = NativeRatioKLOp()

    def group_advantages(self, rewards, *, samples_per_prompt: Optional[int] = None,
                         group_boundaries: Optional[Sequence[int] | torch.Tensor] = None, eps: float = 1e-6):
        r = rewards.reshape(-1).float()
        gid = self._group_ids(r.numel(), r.device, samples_per_prompt, group_boundaries)
        ng = int(gid.max().item()) + 1 if r.numel() else 0
        cnt = r.new_zeros(ng).index_add_(0, gid, torch.ones_like(r))
        mean = r.new_zeros(ng).index_add_(0, gid, r) / cnt
        d = r - mean[gid]
        var = r.new_zeros(ng).index_add_(0, gid, d * d) / cnt     # two-pass variance
        return d / var.clamp_min(eps ** 2).sqrt()[gid]

    @staticmethod
    def _group_ids(n, device, samples_per_prompt, group_boundaries):
        if (samples_per_prompt is None) == (group_boundaries is None):
            raise ValueError("give exactly one of samples_per_prompt / group_boundaries")
        if samples_per_prompt is not None:
            if samples_per_prompt <= 0 or n % samples_per_prompt:
                raise ValueError("batch must be a multiple of samples_per_prompt")
            return torch.arange(n, device=device) // samples_per_prompt
        b = torch.as_tensor(group_boundaries, device=device, dtype=torch.long)
        if b.numel() < 2 or b[0] != 0 or b[-1] != n or (b[1:] <= b[:-1]).any():
            raise ValueError("group_boundaries must increase from 0 to the batch size")
        return torch.repeat_interleave(torch.arange(b.numel() - 1, device=device), b[1:] - b[:-1])

    @staticmethod
    def expand_advantages(sample_advantages, completion_mask):
        m = completion_mask.bool()
        return sample_advantages.reshape(-1, 1).expand_as(m).clone().masked_fill(~m, 0.0)

    def apply(self, policy_logits, ref_logits, action_ids, old_logps, sample_advantages, completion_mask, *,
              clip_eps: float = 0.2, beta: float = 0.0):
        ratio, kl = self._ratio_kl(policy_logits, ref_logits, action_ids, completion_mask, old_logps)
        m = completion_mask.bool()
        adv = self.expand_advantages(sample_advantages, completion_mask).float()
        pol = -torch.minimum(ratio * adv, torch.clamp(ratio, 1.0 - clip_eps, 1.0 + clip_eps) * adv)
        policy_loss, klm = _masked_mean(pol, m), _masked_mean(kl, m)
        return policy_loss + beta * klm, policy_loss, klm

    def forward(self, policy_logits, ref_logits, action_ids, old_logps, rewards, completion_mask, *,
                clip_eps: float = 0.2, beta: float = 0.0, samples_per_prompt=None, group_boundaries=None,
                eps: float = 1e-6):
        adv = self.group_advantages(rewards, samples_per_prompt=samples_per_prompt,
                                    group_boundaries=group_boundaries, eps=eps)
        return self.apply(policy_logits, ref_logits, action_ids, old_logps, adv, completion_mask,
                          clip_eps=clip_eps, beta=beta)

    __call__ = forward
