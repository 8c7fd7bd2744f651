"""Per-token ratio / KL and the data-parallel GRPO loss on the sm_100a loss kernel.

``RatioKLNativeOp``: policy ratio exp(logp - old) and k3 reference KL per token from
logits, without a [tokens, V] softmax: the selected log-probs come from the batch-invariant tile
kernel, the per-token terms from the loss kernel (parity: the Triton ratio_kl operator,
rl_engine/backends/shared/triton/loss/ratio_kl.py:22-87).

``DistributedGRPOLossNativeOp``: every data-parallel rank owns whole sequences; the loss kernel
produces per-sequence totals in ascending token order, the totals and the integer token counts are
gathered in rank order through the group's collective and summed in ascending global sequence
order, advantages are normalised on the gathered rewards -- the result is identical on every rank
and identical to one rank holding the whole batch (parity: DistributedGRPOLossOp,
rl_engine/reference/loss/distributed_grpo_loss.py:177-299, 319-449).
"""
from __future__ import annotations

import torch


class RatioKLNativeOp:
    backend_id = "b200"

    def __init__(self, temperature: float = 1.0):
        self.temperature = temperature

    def __call__(self, policy_logits, ref_logits, action_ids, attention_mask, old_logps):
        from rl_kernel_b200.backends import native as nv
        from rl_kernel_b200.ops.logprob import logp_from_logits

        mask = attention_mask.bool()
        vocab = policy_logits.size(-1)
        if (mask & ((action_ids < 0) | (action_ids >= vocab))).any():
            raise ValueError(f"action_ids at active positions must be in [0, {vocab})")
        ids = action_ids.masked_fill(~mask, 0)
        lp = logp_from_logits(policy_logits, ids, self.temperature)
        with torch.no_grad():
            lr = logp_from_logits(ref_logits, ids, self.temperature)
        B, L = lp.reshape(-1, lp.shape[-1]).shape
        r = nv.grpo_loss(lp.detach().reshape(B, L).float().contiguous(), old_logps.reshape(B, L).float().contiguous(),
                         lr.reshape(B, L).float().contiguous(), torch.zeros(B, device=lp.device),
                         mask.reshape(B, L).to(torch.uint8).contiguous(), clip_lo=0.2, clip_hi=0.2, beta=0.0, inv_norm=1.0,
                         want_tokens=True)
        # the kernel's per-token values carry no graph; re-attach the (elementwise) dependence on lp:
        # d ratio / d lp = ratio, d kl / d lp = 1 - exp(ref - lp) = -(kl + ref - lp)
        rt, kt = r["ratio_tok"].view_as(lp), r["kl_tok"].view_as(lp)
        dlp = lp - lp.detach()
        ratio = rt + dlp * rt
        kl = kt - dlp * (kt + (lr - lp.detach()))
        return ratio.masked_fill(~mask, 1.0), kl.masked_fill(~mask, 0.0)

    forward = __call__


class _DistGRPOFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logp, old_logp, ref_logp, adv_local, mask_u8, op, total_tokens):
        from rl_kernel_b200.backends import native as nv

        r = nv.grpo_loss(logp.float().contiguous(), old_logp.float().contiguous(),
                         None if ref_logp is None else ref_logp.float().contiguous(), adv_local.float().contiguous(),
                         mask_u8, clip_lo=op.clip_eps, clip_hi=op.clip_eps_high, beta=op.beta,
                         inv_norm=1.0 / total_tokens, want_tokens=False)
        ctx.save_for_backward(r["dlogp"])
        return r["seq_sums"]

    @staticmethod
    def backward(ctx, g_seq):
        (dlogp,) = ctx.saved_tensors
        # the loss is a fixed linear combination of the sequence sums: d loss / d logp is what the
        # kernel already produced for inv_norm = 1 / total tokens
        return dlogp, None, None, None, None, None, None


class DistributedGRPOLossNativeOp:
    backend_id = "b200"
    backward_impl = "native"

    def __init__(self, collective=None, clip_eps: float = 0.2, beta: float = 0.0, clip_eps_high: float | None = None):
        self.collective, self.clip_eps, self.beta = collective, clip_eps, beta
        self.clip_eps_high = clip_eps if clip_eps_high is None else clip_eps_high
        self.world = getattr(collective, "world", 1) if collective is not None else 1
        self.rank = getattr(collective, "rank", 0) if collective is not None else 0

    def _gather(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        return self.collective.all_gather(t.contiguous()).flatten(0, 1)

    def __call__(self, logp, old_logp, ref_logp, rewards_local, mask, *, samples_per_prompt: int):
        from rl_kernel_b200.backends import native as nv

        rewards = self._gather(rewards_local.float().reshape(-1))
        n = rewards_local.numel()
        adv_all = nv.group_advantages(rewards.contiguous(), rewards.numel() // samples_per_prompt, samples_per_prompt, 1e-6)
        adv_local = adv_all[self.rank * n:(self.rank + 1) * n]
        m8 = mask.to(torch.uint8).contiguous()
        cnt_all = self._gather(mask.sum(1).to(torch.float32))          # exact: integer counts below 2^24
        total = float(cnt_all.sum().clamp_min(1).item())
        seq = _DistGRPOFn.apply(logp, old_logp, ref_logp, adv_local, m8, self, total)   # [B, 4]: policy, kl sums ...
        pol_all, kl_all = self._gather(seq[:, 0].contiguous()), self._gather(seq[:, 1].contiguous())
        pol_sum, kl_sum = pol_all.new_zeros(()), kl_all.new_zeros(())
        for i in range(pol_all.numel()):                               # ascending global sequence order
            pol_sum = pol_sum + pol_all[i]
            kl_sum = kl_sum + kl_all[i]
        policy_loss, kl = pol_sum / total, kl_sum / total
        # gradients flow through this rank's own sequence sums (the gathered copies carry no graph)
        own = (seq[:, 0].sum() + self.beta * seq[:, 1].sum()) / total
        loss = (policy_loss + self.beta * kl).detach() + own - own.detach()
        return loss, policy_loss.detach(), kl.detach()

    forward = __call__
