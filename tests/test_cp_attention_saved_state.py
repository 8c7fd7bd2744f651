"""The explicit attention backward from a saved forward state: equals autograd, does not depend on the CP degree, the
layout or the KV chunking beyond fp32 summation order, refuses operands the state was not saved for; split-KV plan
records of the reference path bind as runtime evidence."""
import pytest
import torch

from rl_kernel_b200.contracts.operators.attention import AttentionContract, SplitKVMode
from rl_kernel_b200.reference.attention.cp_attention import (STRICT_ATTENTION_SCHEDULE_ID, DeterministicCPAttentionReferenceOp,
                                                             backward_from_saved_state, backward_path, backward_path_name,
                                                             build_reference_split_kv_runtime_plan_set, compare_backward_paths,
                                                             save_forward_state, split_kv_execution_plan_provenance)


def _qkv(seed=0, S=256, hq=4, hkv=2, d=16):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(S, h, d, generator=g) for h in (hq, hkv, hkv))
    return q, k, v, torch.randn(S, hq, d, generator=g)


def test_explicit_backward_equals_autograd_of_plain_attention():
    q, k, v, dout = _qkv()
    res = backward_path(q, k, v, dout)
    qa, ka, va = (t.clone().requires_grad_(True) for t in (q, k, v))
    g = q.shape[1] // k.shape[1]
    s = torch.einsum("nhd,chd->hnc", qa, ka.repeat_interleave(g, 1)) / (q.shape[-1] ** 0.5)
    s = s.masked_fill(~torch.ones(256, 256, dtype=torch.bool).tril()[None], float("-inf"))
    out = torch.einsum("hnc,chd->nhd", torch.softmax(s, -1), va.repeat_interleave(g, 1))
    (out * dout).sum().backward()
    assert (res.out - out.detach()).abs().max() < 1e-5
    for got, want in ((res.gradients.dq, qa.grad), (res.gradients.dk, ka.grad), (res.gradients.dv, va.grad)):
        assert (got - want).abs().max() < 2e-5 * want.abs().max() + 1e-5
    assert res.name == "cp1_backward_reference" and res.saved_forward_state.strict_schedule == STRICT_ATTENTION_SCHEDULE_ID
    assert res.provenance["split_kv"][0]["actual_split_boundaries"] == [[0, 256]]


@pytest.mark.parametrize("cp,layout,chunk", [(2, "zigzag", None), (4, "zigzag", 64), (2, "contiguous", 48), (1, "zigzag", 100)])
def test_backward_does_not_depend_on_cp_layout_or_kv_chunking(cp, layout, chunk):
    S = 128 * 2 * cp if layout == "zigzag" else 256
    q, k, v, dout = _qkv(1, S=S)
    ref = backward_path(q, k, v, dout)
    cand = backward_path(q, k, v, dout, cp_world_size=cp, layout=layout, kv_chunk_size=chunk)
    assert cand.name == backward_path_name(cp_world_size=cp, kv_chunk_size=chunk)
    assert torch.equal(cand.out, ref.out) and torch.equal(cand.lse, ref.lse)            # the strict forward is bit-equal
    drift = compare_backward_paths(cand, ref)
    assert drift.dq.max_rel < 1e-5 and drift.dk.max_rel < 1e-5 and drift.dv.max_rel < 1e-5
    assert len(drift.ranks) == cp and drift.to_dict()["candidate"] == cand.name
    modes = {p["actual_split_kv_policy"] for p in cand.provenance["split_kv"]}
    assert modes == {SplitKVMode.DISABLED.value if chunk is None else SplitKVMode.FIXED.value}


def test_saved_state_refuses_other_operands():
    q, k, v, dout = _qkv(2, S=256)
    op = DeterministicCPAttentionReferenceOp(2, "zigzag")
    state = save_forward_state(op, q, k, v)
    backward_from_saved_state(state, q, k, v, dout)
    k2 = k.clone()
    k2[5, 0, 0] += 1.0
    with pytest.raises(ValueError, match="operand k differs"):
        backward_from_saved_state(state, q, k2, v, dout)
    with pytest.raises(ValueError, match="operand q is"):
        backward_from_saved_state(state, q.double(), k, v, dout)
    with pytest.raises(ValueError, match="dout must have the output shape"):
        backward_from_saved_state(state, q, k, v, dout[:10])
    state.out[0, 0, 0] += 1.0
    with pytest.raises(ValueError, match="modified after the forward"):
        backward_from_saved_state(state, q, k, v, dout)
    import dataclasses

    with pytest.raises(ValueError, match="strict schedule"):
        dataclasses.replace(save_forward_state(op, q, k, v), strict_schedule=None)
    with pytest.raises(ValueError, match="FP32"):
        dataclasses.replace(save_forward_state(op, q, k, v), lse=state.lse.double())


def test_reference_split_kv_plans_bind_as_runtime_evidence():
    recs = split_kv_execution_plan_provenance(1000, cp_world_size=4, kv_chunk_size=96, backend="x")
    assert [r["owner_cp_rank"] for r in recs] == [0, 1, 2, 3] and recs[0]["actual_split_boundaries"][:2] == [[0, 96], [96, 192]]
    assert recs[3]["actual_split_boundaries"][-1] == [942, 1000] and recs[0]["split_kv_plan_source"] == "reference_execution"
    with pytest.raises(ValueError):
        split_kv_execution_plan_provenance(0, cp_world_size=1, kv_chunk_size=None, backend="x")
    ps = build_reference_split_kv_runtime_plan_set([512, 512], tp_world_size=2, cp_world_size=2, kv_chunk_size=None)
    assert len(ps.entries) == 2 * 2 * 2 * 2 and ps.batch_size == 2
    with pytest.raises(ValueError, match="at least one KV token per CP owner"):
        build_reference_split_kv_runtime_plan_set([1], tp_world_size=1, cp_world_size=2, kv_chunk_size=None)
    from rl_kernel_b200.contracts.operators.attention import AttentionRole
    from rl_kernel_b200.integrations.common.attention_binding import bind_attention_contracts

    kw = dict(head_dim=128, seq_len=512, batch_size=2, tp_world_size=2, cp_world_size=2, layout="zigzag")
    r, t = AttentionContract.for_layout(8, 2, role=AttentionRole.INFER, **kw), AttentionContract.for_layout(8, 2, role=AttentionRole.TRAIN, **kw)
    res = bind_attention_contracts(rollout_contract=r, training_contract=t, rollout_identity={}, training_identity={},
                                   rollout_backend_id="a", training_backend_id="b", require_full_identity=False,
                                   rollout_split_kv_plan_set=ps, training_split_kv_plan_set=ps)
    assert res.passed, [i.to_dict() for i in res.issues]
    chunked = build_reference_split_kv_runtime_plan_set([512, 512], tp_world_size=2, cp_world_size=2, kv_chunk_size=128)
    res = bind_attention_contracts(rollout_contract=r, training_contract=t, rollout_identity={}, training_identity={},
                                   rollout_backend_id="a", training_backend_id="b", require_full_identity=False,
                                   rollout_split_kv_plan_set=chunked, training_split_kv_plan_set=ps)
    assert not res.passed and res.comparable
