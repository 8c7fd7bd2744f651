"""Contract-driven distributed GRPO loss on the CPU: against the plain formula, and with 2 gloo ranks as data-parallel
or tensor-parallel shards against one rank, bit for bit (scalars, per-sequence vectors and gradients)."""
import datetime
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rl_kernel_b200.contracts.operators.logprob import LogprobContract, LogprobDType
from rl_kernel_b200.contracts.operators.loss import (AdvantageNormalizer, AdvantageSpec, ClipSpec, GRPOLossContract, KLEstimator,
                                                     LossContractError, LossReductionSpec, LossShardingSpec, ObjectiveSpec, TokenNormalizer)
from rl_kernel_b200.reference.loss.distributed_grpo_loss import ContractGRPOLossOp, group_advantages_from_contract

N_SEQ, L, V, VP, G = 8, 6, 200, 256, 4


def _data(seed=0):
    g = torch.Generator().manual_seed(seed)
    pol = torch.randn(N_SEQ * L, VP, generator=g) * 2
    ref = pol + 0.3 * torch.randn(N_SEQ * L, VP, generator=g)
    ids = torch.randint(0, V, (N_SEQ * L,), generator=g)
    old = torch.log_softmax(pol[:, :V], -1).gather(1, ids[:, None])[:, 0] + 0.2 * torch.randn(N_SEQ * L, generator=g)
    rewards = torch.randn(N_SEQ, generator=g)
    lens = torch.randint(2, L + 1, (N_SEQ,), generator=g)
    mask = (torch.arange(L)[None, :] < lens[:, None]).reshape(-1)
    return pol, ref, ids, old, rewards, mask


def _contract(mask, *, dp_rank=0, dp=1, tp_rank=0, tp=1, normalizer=TokenNormalizer.GLOBAL_ACTIVE_TOKENS, adv=AdvantageNormalizer.MEAN_STD_POPULATION,
              kl=KLEstimator.K3_UNBIASED, beta=0.05, fixed=None):
    sh = LossShardingSpec.even(dp_rank=dp_rank, dp_world_size=dp, num_sequences=N_SEQ, padded_seq_len=L, samples_per_prompt=G)
    a, e = sh.local_sequence_start * L, sh.local_sequence_end * L
    lp = LogprobContract.for_tokens(e - a, real_vocab_size=V, padded_vocab_size=VP, tp_rank=tp_rank, tp_world_size=tp, temperature=1.0,
                                    active_mask=mask[a:e], dtype=LogprobDType.FP32)
    return GRPOLossContract(lp, sh, ObjectiveSpec(ClipSpec(0.2, 0.3), AdvantageSpec(normalizer=adv), kl_estimator=kl, beta=beta),
                            LossReductionSpec(token_normalizer=normalizer, fixed_normalizer_constant=fixed))


@pytest.mark.parametrize("normalizer,adv,kl", [(TokenNormalizer.GLOBAL_ACTIVE_TOKENS, AdvantageNormalizer.MEAN_STD_POPULATION, KLEstimator.K3_UNBIASED),
                                               (TokenNormalizer.PER_SEQUENCE_THEN_MEAN, AdvantageNormalizer.MEAN_ONLY, KLEstimator.K1_LOG_RATIO),
                                               (TokenNormalizer.FIXED_CONSTANT, AdvantageNormalizer.MEAN_STD_POPULATION, KLEstimator.K3_UNBIASED)])
def test_single_rank_matches_the_plain_formula(normalizer, adv, kl):
    pol, ref, ids, old, rewards, mask = _data()
    c = _contract(mask, normalizer=normalizer, adv=adv, kl=kl, fixed=37 if normalizer is TokenNormalizer.FIXED_CONSTANT else None)
    res = ContractGRPOLossOp()(pol, ids, old, rewards, contract=c, ref_local_logits=ref)
    loss, policy_loss, klv = res                                            # unpacks like the tuple of the simple operators
    lp = torch.log_softmax(pol[:, :V], -1).gather(1, ids[:, None])[:, 0]
    lr = torch.log_softmax(ref[:, :V], -1).gather(1, ids[:, None])[:, 0]
    r = rewards.view(-1, G)
    a = r - r.mean(1, keepdim=True)
    if adv is AdvantageNormalizer.MEAN_STD_POPULATION:
        a = a / (r.std(1, unbiased=False, keepdim=True) + 1e-6)
    a = a.reshape(-1)
    assert (res.advantages - a).abs().max() < 1e-5 and torch.equal(group_advantages_from_contract(rewards, c), res.advantages)
    ratio = (lp - old).exp()
    at = a.repeat_interleave(L)
    pt = -torch.minimum(ratio * at, ratio.clamp(0.8, 1.3) * at) * mask
    d = lr - lp
    kt = ((d.exp() - d - 1) if kl is KLEstimator.K3_UNBIASED else -d) * mask
    cnt = mask.view(N_SEQ, L).sum(1)
    if normalizer is TokenNormalizer.GLOBAL_ACTIVE_TOKENS:
        wp, wk = pt.sum() / mask.sum(), kt.sum() / mask.sum()
    elif normalizer is TokenNormalizer.FIXED_CONSTANT:
        wp, wk = pt.sum() / 37, kt.sum() / 37
    else:
        wp, wk = (pt.view(N_SEQ, L).sum(1) / cnt).mean(), (kt.view(N_SEQ, L).sum(1) / cnt).mean()
    assert abs(float(policy_loss - wp)) < 1e-5 and abs(float(klv - wk)) < 1e-5 and abs(float(loss - (wp + 0.05 * wk))) < 1e-5
    assert torch.equal(res.per_sequence_active_tokens, cnt) and res.provenance["global_active_tokens"] == int(mask.sum())
    assert (res.per_sequence_policy - pt.view(N_SEQ, L).sum(1)).abs().max() < 1e-5


def test_invocation_checks():
    pol, ref, ids, old, rewards, mask = _data()
    c, op = _contract(mask), ContractGRPOLossOp()
    with pytest.raises(LossContractError, match="ref_local_logits is required"):
        op(pol, ids, old, rewards, contract=c)
    with pytest.raises(LossContractError, match="token slots"):
        op(pol[:-1], ids, old, rewards, contract=c, ref_local_logits=ref)
    with pytest.raises(LossContractError, match="one entry per sequence"):
        op(pol, ids, old, rewards[:-1], contract=c, ref_local_logits=ref)
    with pytest.raises(LossContractError, match="action_ids"):
        op(pol, ids[:-1], old, rewards, contract=c, ref_local_logits=ref)
    with pytest.raises(LossContractError, match="must be a GRPOLossContract"):
        op(pol, ids, old, rewards, contract=None)
    with pytest.raises(LossContractError, match="no active tokens"):
        op(pol, ids, old, rewards, contract=_contract(torch.zeros_like(mask)), ref_local_logits=ref)
    with pytest.raises(LossContractError, match="initialized process group"):
        op(pol[:N_SEQ * L // 2], ids[:N_SEQ * L // 2], old[:N_SEQ * L // 2], rewards[:N_SEQ // 2], contract=_contract(mask, dp=2),
           ref_local_logits=ref[:N_SEQ * L // 2])
    assert float(op(pol, ids, old, rewards, contract=_contract(mask, beta=0.0)).kl) == 0.0          # no reference model needed


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out, axis):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    pol, ref, ids, old, rewards, mask = _data()
    op = ContractGRPOLossOp()
    if axis == "dp":
        c = _contract(mask, dp_rank=rank, dp=world)
        a, e = c.sharding.local_sequence_start, c.sharding.local_sequence_end
        p = pol[a * L:e * L].clone().requires_grad_(True)
        res = op(p, ids[a * L:e * L], old[a * L:e * L], rewards[a:e], contract=c, ref_local_logits=ref[a * L:e * L], dp_group=dist.group.WORLD)
    else:
        c = _contract(mask, tp_rank=rank, tp=world)
        per = VP // world
        p = pol[:, rank * per:(rank + 1) * per].clone().requires_grad_(True)
        res = op(p, ids, old, rewards, contract=c, ref_local_logits=ref[:, rank * per:(rank + 1) * per].contiguous(), tp_group=dist.group.WORLD)
    res.loss.backward()
    err = None
    if axis == "dp":
        try:                                          # ranks that disagree on the objective stop before any arithmetic
            bad = _contract(mask, dp_rank=rank, dp=world, beta=0.05 if rank == 0 else 0.06)
            a, e = bad.sharding.local_sequence_start, bad.sharding.local_sequence_end
            op(pol[a * L:e * L], ids[a * L:e * L], old[a * L:e * L], rewards[a:e], contract=bad, ref_local_logits=ref[a * L:e * L],
               dp_group=dist.group.WORLD)
        except LossContractError as exc:
            err = str(exc)
    torch.save({"loss": res.loss.detach(), "policy": res.policy_loss.detach(), "kl": res.kl.detach(), "pp": res.per_sequence_policy,
                "pk": res.per_sequence_kl, "cnt": res.per_sequence_active_tokens, "grad": p.grad, "err": err}, f"{out}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("axis", ["dp", "tp"])
def test_two_ranks_give_the_single_rank_bits(tmp_path, axis):
    out = str(tmp_path / "r")
    mp.spawn(_worker, args=(2, _port(), out, axis), nprocs=2, join=True)
    r0, r1 = (torch.load(f"{out}.{r}", weights_only=False) for r in range(2))
    pol, ref, ids, old, rewards, mask = _data()
    p = pol.clone().requires_grad_(True)
    one = ContractGRPOLossOp()(p, ids, old, rewards, contract=_contract(mask), ref_local_logits=ref)
    one.loss.backward()
    for r in (r0, r1):
        assert torch.equal(r["loss"], one.loss.detach()) and torch.equal(r["policy"], one.policy_loss.detach()) and torch.equal(r["kl"], one.kl.detach())
        assert torch.equal(r["pp"], one.per_sequence_policy) and torch.equal(r["pk"], one.per_sequence_kl) and torch.equal(r["cnt"], one.per_sequence_active_tokens)
    grad = torch.cat([r0["grad"], r1["grad"]], dim=0 if axis == "dp" else 1)
    assert torch.equal(grad, p.grad)
    if axis == "dp":
        assert "different loss contracts" in r0["err"] and "different loss contracts" in r1["err"]
