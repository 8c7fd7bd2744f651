"""GRPO / PPO ratio-KL loss operators on per-token log-probs (native forward + analytic backward)."""
from __future__ import annotations

import torch

from rl_kernel_b200.ops._dispatch import use_native
from rl_kernel_b200.reference.loss.grpo_loss import NativeGRPOLossOp, grpo_loss_from_logps
from rl_kernel_b200.reference.loss.ratio_kl import ratio_kl_from_logps


class _GRPOLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logp, old_logp, ref_logp, adv, mask, clip_lo, clip_hi, beta, denominator=None):
        from rl_kernel_b200.backends import native as nv

        m8 = mask.to(torch.uint8).contiguous()
        cnt = float(mask.sum().clamp_min(1).item()) if denominator is None else float(denominator)
        r = nv.grpo_loss(logp.float().contiguous(), old_logp.float().contiguous(),
                         None if ref_logp is None else ref_logp.float().contiguous(), adv.float().contiguous(), m8,
                         clip_lo=clip_lo, clip_hi=clip_hi, beta=beta, inv_norm=1.0 / cnt)
        ctx.save_for_backward(r["dlogp"])
        t = r["totals"]
        return t[4], t[5], t[6]

    @staticmethod
    def backward(ctx, g_loss, g_pol, g_kl):
        (dlogp,) = ctx.saved_tensors
        return dlogp * g_loss, None, None, None, None, None, None, None, None


def grpo_loss(logp, old_logp, ref_logp, sample_advantages, mask, *, clip_eps: float = 0.2, beta: float = 0.0,
              clip_eps_high: float | None = None, denominator: float | None = None):
    """(loss, policy_loss, kl) for logp/old/ref [B, L], per-sequence advantages [B], mask [B, L].
    Gradients flow into ``logp`` through the total loss.  ``denominator``: the token count the sums are divided by
    (default: this call's own active tokens); a micro-batch of a larger step passes the step's global count, so that
    its per-token gradients are the bits the whole batch would give."""
    hi = clip_eps if clip_eps_high is None else clip_eps_high
    if not use_native(logp):
        return grpo_loss_from_logps(logp, old_logp, ref_logp, sample_advantages, mask, clip_eps=clip_eps, beta=beta,
                                    clip_eps_high=hi, denominator=denominator)
    return _GRPOLossFn.apply(logp, old_logp, ref_logp, sample_advantages, mask, clip_eps, hi, beta, denominator)


def ratio_kl(logp, old_logp, ref_logp, mask):
    """Per-token (ratio, k3 KL); elementwise math identical on every device."""
    return ratio_kl_from_logps(logp, old_logp, ref_logp, mask)


def group_advantages(rewards: torch.Tensor, samples_per_prompt: int, eps: float = 1e-6) -> torch.Tensor:
    if not use_native(rewards):
        return NativeGRPOLossOp().group_advantages(rewards, samples_per_prompt=samples_per_prompt, eps=eps)
    from rl_kernel_b200.backends import native as nv

    r = rewards.reshape(-1).float().contiguous()
    return nv.group_advantages(r, r.numel() // samples_per_prompt, samples_per_prompt, eps)


class GRPOLossOp:
    backend_id = "b200"
    backward_impl = "native"

    def __init__(self, clip_eps: float = 0.2, beta: float = 0.0):
        self.clip_eps, self.beta = clip_eps, beta

    def __call__(self, logp, old_logp, ref_logp, sample_advantages, mask, *, denominator: float | None = None):
        return grpo_loss(logp, old_logp, ref_logp, sample_advantages, mask, clip_eps=self.clip_eps, beta=self.beta,
                         denominator=denominator)

    forward = __call__
    group_advantages = staticmethod(group_advantages)
