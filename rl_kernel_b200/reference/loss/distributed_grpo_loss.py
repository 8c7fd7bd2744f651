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


# ------------------------------------------------------------------------------------------------ contract driven
# The same reduction, driven by a ``GRPOLossContract`` over vocabulary-parallel LOGITS (not log-probs): tensor
# parallelism is delegated to the contract-driven vocabulary-parallel log-prob, this operator owns the sums over tokens
# and sequences (parity: DistributedGRPOLossOp.apply, rl_engine/reference/loss/distributed_grpo_loss.py:301-449).
from dataclasses import dataclass, field  # noqa: E402
from typing import Any, Iterator  # noqa: E402

from rl_kernel_b200.contracts.operators.loss import (AdvantageNormalizer, GRPOLossContract, KLEstimator,  # noqa: E402
                                                      LossContractError, TokenNormalizer)

BACKEND_ID = "rl_kernel_b200.reference.distributed_grpo_loss"


@dataclass(frozen=True)
class GRPOLossResult:
    """Unpacks as ``loss, policy_loss, kl``.  The per-sequence vectors are the last intermediate that does not depend on
    the parallel layout; they are what two configurations should be compared on (the scalar averages them into 24
    mantissa bits and can round a real reordering away) and they say which sequence a drift comes from."""
    loss: torch.Tensor
    policy_loss: torch.Tensor
    kl: torch.Tensor
    advantages: torch.Tensor
    per_sequence_policy: torch.Tensor
    per_sequence_kl: torch.Tensor
    per_sequence_active_tokens: torch.Tensor
    provenance: dict[str, Any] = field(default_factory=dict)

    def __iter__(self) -> Iterator[torch.Tensor]:
        yield from (self.loss, self.policy_loss, self.kl)


def _dist_for(world: int):
    import torch.distributed as dist

    if world > 1 and not (dist.is_available() and dist.is_initialized()):
        raise LossContractError("the contract declares dp_world_size > 1: an initialized process group is required")
    return dist


def _gather_rows(local: torch.Tensor, contract: GRPOLossContract, dp_group) -> torch.Tensor:
    """[local sequences, ...] -> [num_sequences, ...] in global sequence order.  Shards may be uneven: every rank pads to
    the widest shard, the gathered pieces are cut back by the contract's bounds.  Nothing is added in transit."""
    sh = contract.sharding
    if sh.dp_world_size == 1:
        return local
    dist = _dist_for(sh.dp_world_size)
    widest = max(e - s for s, e in sh.sequence_shard_bounds)
    pad = local if local.shape[0] == widest else torch.cat([local, local.new_zeros(widest - local.shape[0], *local.shape[1:])])
    parts = [torch.empty_like(pad) for _ in range(sh.dp_world_size)]
    dist.all_gather(parts, pad.contiguous(), group=dp_group)
    mine = sh.dp_rank
    # the local piece keeps its autograd history; the others are constants of this rank's graph
    return torch.cat([(local if r == mine else parts[r][:e - s]) for r, (s, e) in enumerate(sh.sequence_shard_bounds)])


def _ordered_sum(x: torch.Tensor, dim_len: int) -> torch.Tensor:
    """Sum over the last axis of fixed extent ``dim_len`` in ascending index order (one add per element)."""
    acc = x.new_zeros(x.shape[:-1])
    for j in range(dim_len):
        acc = acc + x[..., j]
    return acc


def group_advantages_from_contract(global_rewards: torch.Tensor, contract: GRPOLossContract) -> torch.Tensor:
    """Advantage of every sequence of the global batch from the gathered rewards (two-pass variance, population std)."""
    adv = contract.objective.advantage
    out = torch.empty_like(global_rewards, dtype=torch.float32)
    b = contract.sharding.group_boundaries
    for g in range(contract.sharding.num_groups):
        r = global_rewards[b[g]:b[g + 1]].float()
        n = r.numel()
        mean = _ordered_sum(r.reshape(1, n), n)[0] / n
        c = r - mean
        if adv.normalizer is AdvantageNormalizer.MEAN_ONLY:
            out[b[g]:b[g + 1]] = c
        else:
            var = _ordered_sum((c * c).reshape(1, n), n)[0] / n
            out[b[g]:b[g + 1]] = c / (var.sqrt() + adv.std_eps)
    return out


class ContractGRPOLossOp:
    """``apply(policy_local_logits [n, V_local], action_ids [n], old_logps [n], rewards [local sequences], contract=...)``
    with n = this DP rank's token slots (whole padded sequences) and V_local this TP rank's vocabulary shard."""

    op_class = "grpo_loss"
    is_batch_invariant = True
    backend_id = BACKEND_ID

    def __init__(self) -> None:
        from rl_kernel_b200.reference.logprob.vocab_parallel_logp import VocabParallelLogprobOp

        self._logprob = VocabParallelLogprobOp()

    def __call__(self, *args: Any, **kwargs: Any) -> GRPOLossResult:
        return self.apply(*args, **kwargs)

    @staticmethod
    def _validate(policy, ref, action_ids, old_logps, rewards, contract: GRPOLossContract, dp_group) -> None:
        sh = contract.sharding
        n = sh.local_num_token_slots
        if policy.dim() != 2 or policy.shape[0] != n:
            raise LossContractError(f"policy_local_logits must be [{n}, local_vocab] (this rank's token slots); got {tuple(policy.shape)}")
        if ref is not None and ref.shape != policy.shape:
            raise LossContractError(f"ref_local_logits shape {tuple(ref.shape)} must match policy_local_logits {tuple(policy.shape)}")
        if ref is None and contract.objective.uses_reference_model:
            raise LossContractError(f"objective.beta={contract.objective.beta} puts the reference KL in the loss, so ref_local_logits is required")
        for name, t in (("action_ids", action_ids), ("old_logps", old_logps)):
            if t.dim() != 1 or t.shape[0] != n:
                raise LossContractError(f"{name} must be 1-D with one entry per owned token slot; got {tuple(t.shape)} for {n} slots")
        if rewards.dim() != 1 or rewards.shape[0] != sh.local_num_sequences:
            raise LossContractError(f"rewards must hold one entry per sequence this rank owns; got {tuple(rewards.shape)} for "
                                    f"{sh.local_num_sequences} sequences")
        if contract.logprob.mask.num_tokens != n:
            raise LossContractError("the log-prob contract must describe exactly this rank's token slots")
        if sh.dp_world_size > 1:
            dist = _dist_for(sh.dp_world_size)
            if dist.get_world_size(group=dp_group) != sh.dp_world_size:
                raise LossContractError(f"dp_group world size {dist.get_world_size(group=dp_group)} does not match the contract "
                                        f"dp_world_size={sh.dp_world_size}; pass the DP subgroup, not the global group")
            if dist.get_rank(group=dp_group) != sh.dp_rank:
                raise LossContractError(f"dp_group rank {dist.get_rank(group=dp_group)} does not match the contract dp_rank={sh.dp_rank}")

    @staticmethod
    def _preflight(contract: GRPOLossContract, dp_group) -> None:
        """Every DP rank must hold the same contract up to its own rank (objective, reduction, shard table, groups)."""
        sh = contract.sharding
        if sh.dp_world_size == 1:
            return
        dist = _dist_for(sh.dp_world_size)
        mine = contract.cross_rank_fingerprint()               # rank fields, local bounds and the local mask are left out
        seen = [None] * sh.dp_world_size
        dist.all_gather_object(seen, (sh.dp_rank, mine), group=dp_group)
        if sorted(r for r, _ in seen) != list(range(sh.dp_world_size)):
            raise LossContractError(f"the DP ranks of the group do not match the contract's ranks: {[r for r, _ in seen]}")
        if len({h for _, h in seen}) != 1:
            raise LossContractError(f"the DP ranks hold different loss contracts: {seen}")

    def apply(self, policy_local_logits: torch.Tensor, action_ids: torch.Tensor, old_logps: torch.Tensor, rewards: torch.Tensor, *,
              contract: GRPOLossContract, ref_local_logits: torch.Tensor | None = None, tp_group: Any = None, dp_group: Any = None,
              num_vocab_tiles: int | None = None, validate: bool = True) -> GRPOLossResult:
        if not isinstance(contract, GRPOLossContract):
            raise LossContractError("contract must be a GRPOLossContract")
        self._validate(policy_local_logits, ref_local_logits, action_ids, old_logps, rewards, contract, dp_group)
        if validate:
            self._preflight(contract, dp_group)
        sh, obj = contract.sharding, contract.objective
        kw = {} if num_vocab_tiles is None else {"num_vocab_tiles": num_vocab_tiles}
        logp, _ = self._logprob.apply(policy_local_logits, action_ids, contract=contract.logprob, tp_group=tp_group, validate=validate, **kw)
        active = torch.tensor(contract.logprob.mask.active_mask, dtype=torch.bool, device=policy_local_logits.device)
        ratio = (logp - old_logps.float()).masked_fill(~active, 0.0).exp()
        if ref_local_logits is None:
            kl_terms = torch.zeros_like(logp)
        else:
            with torch.no_grad():
                logp_ref, _ = self._logprob.apply(ref_local_logits, action_ids, contract=contract.logprob, tp_group=tp_group,
                                                  validate=False, **kw)
            diff = (logp_ref - logp).masked_fill(~active, 0.0)
            kl_terms = (diff.exp() - diff - 1.0) if obj.kl_estimator is KLEstimator.K3_UNBIASED else -diff
            kl_terms = kl_terms.masked_fill(~active, 0.0)
        global_rewards = _gather_rows(rewards.float().detach(), contract, dp_group)
        advantages = group_advantages_from_contract(global_rewards, contract)
        L = sh.padded_seq_len
        adv_tok = advantages[sh.local_sequence_start:sh.local_sequence_end].reshape(-1, 1).expand(sh.local_num_sequences, L).reshape(-1)
        unclipped = ratio * adv_tok
        clipped = ratio.clamp(obj.clip.lower_bound, obj.clip.upper_bound) * adv_tok
        pol_terms = (-torch.minimum(unclipped, clipped)).masked_fill(~active, 0.0)
        # fixed extents: [local sequences, L] -> [local sequences] -> gathered [num_sequences] -> scalar, at every DP degree
        seq = lambda t: _ordered_sum(t.reshape(sh.local_num_sequences, L), L)          # noqa: E731
        per_pol = _gather_rows(seq(pol_terms), contract, dp_group)
        per_kl = _gather_rows(seq(kl_terms), contract, dp_group)
        counts = _gather_rows(active.reshape(sh.local_num_sequences, L).sum(1), contract, dp_group)
        total_active = int(counts.sum())
        if validate and total_active == 0:
            raise LossContractError("the global batch holds no active tokens; the loss normalizer would divide by zero")

        def normalized(v: torch.Tensor) -> torch.Tensor:
            norm = contract.reduction.token_normalizer
            n = sh.num_sequences
            if norm is TokenNormalizer.PER_SEQUENCE_THEN_MEAN:
                per = torch.where(counts > 0, v / counts.clamp_min(1).to(v.dtype), torch.zeros_like(v))
                return _ordered_sum(per.reshape(1, n), n)[0] / max(1, int((counts > 0).sum()))
            total = _ordered_sum(v.reshape(1, n), n)[0]
            if norm is TokenNormalizer.FIXED_CONSTANT:
                return total / float(contract.reduction.fixed_normalizer_constant)
            return total / float(max(1, total_active))

        policy_loss, kl = normalized(per_pol), normalized(per_kl)
        prov = {"backend_id": BACKEND_ID, "implementation_kind": "reference", "padded_seq_len": int(L), "num_sequences": int(sh.num_sequences),
                "global_active_tokens": total_active, "reference_model_used": ref_local_logits is not None,
                "token_normalizer": contract.reduction.token_normalizer.value, "requested_contract": contract.to_dict(),
                "cross_rank_fingerprint": contract.cross_rank_fingerprint()}
        return GRPOLossResult(policy_loss + obj.beta * kl, policy_loss, kl, advantages, per_pol.detach(), per_kl.detach(), counts.detach(), prov)


__all__ = ["BACKEND_ID", "ContractGRPOLossOp", "DistributedGRPOLossOp", "GRPOLossResult", "group_advantages_from_contract"]
