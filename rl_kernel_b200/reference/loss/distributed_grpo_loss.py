"""Data-parallel GRPO loss with rank-count-independent bits: every DP rank owns whole sequences,
per-sequence (policy, kl) totals and integer token counts are all-gathered in DP-rank order and
summed in ascending global sequence order; advantages are normalised from the gathered rewards on
every rank (parity: DistributedGRPOLossOp, rl_engine/reference/loss/distributed_grpo_loss.py:177-449)."""
from __future__ import annotations

import torch

from rl_kernel_b200.reference.loss.grpo_loss import NativeGRPOLossOp
from rl_kernel_b200.reference.loss.ratio_kl import ratio_kl_from_logps


class DistributedGRPOLossOp:
    def __init__(self, group=None, clip_eps: float = 0.2, beta: float = 0.0):
        self.group, self.clip_eps, self.beta = group, clip_eps, beta
        self._local = NativeGRPOLossOp()

    def _gather(self, t: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(self.group) == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(dist.get_world_size(self.group))]
        dist.all_gather(parts, t.contiguous(), group=self.group)
        return torch.cat(parts)

    def sequence_totals(self, logp, old_logp, ref_logp, adv_local, mask):
        ratio, kl = ratio_kl_from_logps(logp, old_logp, ref_logp, mask)
        m = mask.bool()
        adv = adv_local.reshape(-1, 1).expand_as(m).float().masked_fill(~m, 0.0)
        pol = -torch.minimum(ratio * adv, torch.clamp(ratio, 1 - self.clip_eps, 1 + self.clip_eps) * adv)
        # fixed ascending token order inside a sequence
        pol_seq = torch.stack([self._seq_sum(pol[i], m[i]) for i in range(pol.shape[0])])
        kl_seq = torch.stack([self._seq_sum(kl[i], m[i]) for i in range(kl.shape[0])])
        return pol_seq, kl_seq, m.sum(1).to(torch.int64)

    @staticmethod
    def _seq_sum(x, m):
        s = x.new_zeros(())
        for v in x[m]:
            s = s + v
        return s

    def __call__(self, logp, old_logp, ref_logp, rewards_local, mask, *, samples_per_prompt: int):
        """All inputs are this rank's sequences. Returns (loss, policy_loss, kl) identical on all ranks
        and identical to the single-rank result on the concatenated batch."""
        rewards = self._gather(rewards_local.float())
        adv_all = self._local.group_advantages(rewards, samples_per_prompt=samples_per_prompt)
        import torch.distributed as dist

        rank = dist.get_rank(self.group) if dist.is_available() and dist.is_initialized() else 0
        n = rewards_local.numel()
        adv_local = adv_all[rank * n:(rank + 1) * n]
        pol_seq, kl_seq, cnt = self.sequence_totals(logp, old_logp, ref_logp, adv_local, mask)
        pol_all, kl_all, cnt_all = self._gather(pol_seq), self._gather(kl_seq), self._gather(cnt)
        pol_sum, kl_sum = pol_all.new_zeros(()), kl_all.new_zeros(())
        for i in range(pol_all.numel()):       # ascending global sequence order
            pol_sum = pol_sum + pol_all[i]
            kl_sum = kl_sum + kl_all[i]
        total = cnt_all.sum().clamp_min(1).to(pol_sum.dtype)
        policy_loss, kl = pol_sum / total, kl_sum / total
        return policy_loss + self.beta * kl, policy_loss, kl

    forward = __call__
