"""Three-tier binding of a rollout and a training attention contract: identity (not comparable), semantics (fails
closed), recorded differences (provenance), and the strict hand-over from executed runtimes."""
import dataclasses

import pytest

from rl_kernel_b200.contracts.operators.attention import (AttentionContract, AttentionDType, AttentionMode, AttentionRole, CPLayout,
                                                          ReductionSpec, SplitKVSpec, build_split_kv_runtime_plan_set)
from rl_kernel_b200.integrations.common.attention_binding import (IDENTITY_FIELDS, AttentionBindingError, AttentionRuntimeReadback,
                                                                  BindingErrorCode, BindingIssue, BindingTier,
                                                                  bind_attention_contracts, bind_attention_runtime_readbacks,
                                                                  first_blocking_issue, identity_fingerprint, summarize_binding)
from rl_kernel_b200.ops.attention.preprocess import FUSED_PREPROCESS_BACKEND_ID
from rl_kernel_b200.ops.attention.projection import AttentionProjectionOp


def _contract(role, **kw):
    args = dict(head_dim=128, seq_len=512, batch_size=2, tp_rank=0, tp_world_size=2, cp_rank=0, cp_world_size=2,
                layout=CPLayout.ZIGZAG, role=role)
    args.update(kw)
    return AttentionContract.for_layout(8, 2, **args)


def _identity(**over):
    ident = {k: f"{k}-v1" for k in IDENTITY_FIELDS}
    ident.update(q_heads=8, kv_heads=2, head_dim=128, rope_theta=1e6, rope_scaling=None, rotary_dim=128, qk_layernorm=True,
                 batch_size=2, padding_side="right", pre_update_state=True)
    ident.update(over)
    return ident


def _plans(contract):
    return build_split_kv_runtime_plan_set([512] * contract.batch_size, tp_world_size=contract.sharding.tp_world_size,
                                           cp_world_size=contract.sharding.cp_world_size, split_kv=contract.split_kv)


def _bind(**over):
    r, t = _contract(AttentionRole.INFER), _contract(AttentionRole.TRAIN)
    kw = dict(rollout_contract=r, training_contract=t, rollout_identity=_identity(), training_identity=_identity(),
              rollout_backend_id="b200.paged", training_backend_id="b200.cp_attention",
              rollout_split_kv_plan_set=_plans(r), training_split_kv_plan_set=_plans(t))
    kw.update(over)
    return bind_attention_contracts(**kw)


def test_matching_pair_passes_and_records_expected_differences():
    res = _bind(rollout_recorded_extra={"preprocess.rope": "x"}, training_recorded_extra={"preprocess.rope": "y"})
    assert res.comparable and res.passed and not res.issues
    assert res.recorded_differences["backend_id"] == {"rollout": "b200.paged", "training": "b200.cp_attention"}
    assert res.recorded_differences["preprocess.rope"] == {"rollout": "x", "training": "y"}
    assert res.identity_fingerprint == identity_fingerprint(_identity()) == identity_fingerprint({**_identity(), "extra": 1})
    assert summarize_binding(res).startswith("attention binding OK") and first_blocking_issue(res) is None
    d = res.to_dict()
    assert d["schema_version"] == "cross_config.attention_binding.v3" and d["provenance"]["lse_domain"] == "attention"
    again = _bind(rollout_recorded_extra={"preprocess.rope": "x"}, training_recorded_extra={"preprocess.rope": "y"})
    assert again.binding_fingerprint == res.binding_fingerprint != _bind().binding_fingerprint


def test_identity_tier_makes_the_pair_not_comparable():
    res = _bind(training_identity=_identity(weight_version="other"))
    assert not res.comparable and not res.passed
    (issue,) = res.issues_by_code(BindingErrorCode.IDENTITY_MISMATCH)
    assert issue.field == "weight_version" and issue.tier is BindingTier.IDENTITY and issue.training == "other"
    assert "NOT COMPARABLE" in summarize_binding(res) and first_blocking_issue(res) is issue
    missing = _identity()
    del missing["tokenizer_fingerprint"]
    res = _bind(rollout_identity=missing)
    assert {i.field for i in res.issues_by_code(BindingErrorCode.IDENTITY_MISSING)} == {"rollout.tokenizer_fingerprint"}
    assert not _bind(rollout_identity=missing, require_full_identity=False).issues_by_code(BindingErrorCode.IDENTITY_MISSING)
    # nullable fields may be absent on both sides
    a, b = _identity(), _identity()
    del a["kv_seq_lens_fingerprint"], b["kv_seq_lens_fingerprint"]
    assert _bind(rollout_identity=a, training_identity=b).passed
    # a different TP rank owns other heads: topology is identity, not provenance
    t = _contract(AttentionRole.TRAIN, tp_rank=1)
    res = _bind(training_contract=t, training_split_kv_plan_set=_plans(t))
    fields = {i.field for i in res.issues_by_code(BindingErrorCode.TOPOLOGY_MISMATCH)}
    assert not res.comparable and {"sharding.tp_rank", "sharding.local_q_head_start"} <= fields


def test_semantic_tier_fails_closed_but_stays_comparable():
    t = _contract(AttentionRole.TRAIN, dtype=AttentionDType.FP16)
    res = _bind(training_contract=t, training_split_kv_plan_set=_plans(t))
    assert res.comparable and not res.passed
    assert [i.field for i in res.issues_by_code(BindingErrorCode.REDUCTION_SEMANTIC_MISMATCH)] == ["dtype"]
    assert "FAILED CLOSED" in summarize_binding(res)
    assert _bind(training_contract=t, training_split_kv_plan_set=_plans(t), allow_dtype_difference=True).passed
    # no runtime evidence of the split-KV plans
    res = _bind(rollout_split_kv_plan_set=None)
    assert res.comparable and not res.passed
    assert [i.field for i in res.issues_by_code(BindingErrorCode.SPLIT_KV_RUNTIME_MISSING)] == ["rollout.split_kv_runtime_plan_set"]
    # different split-KV requests, and plans that do not belong to the contract
    r = dataclasses.replace(_contract(AttentionRole.INFER), split_kv=SplitKVSpec.fixed(128))
    res = _bind(rollout_contract=r, rollout_split_kv_plan_set=_plans(r))
    codes = {i.code for i in res.issues}
    assert BindingErrorCode.SPLIT_KV_MISMATCH in codes and not res.passed
    res = _bind(rollout_split_kv_plan_set=_plans(r))                       # fixed-size plans handed in for a 'disabled' contract
    assert any(i.field == "rollout.split_kv_runtime_plan_set" for i in res.issues_by_code(BindingErrorCode.SPLIT_KV_MISMATCH))
    # findings of the framework probes are threaded through
    probe = BindingIssue(BindingErrorCode.DETERMINISM_INCOMPATIBLE, BindingTier.SEMANTIC, "rollout.enforce_eager", "graphs on")
    res = _bind(determinism_issues=[probe])
    assert res.comparable and not res.passed and res.issues == (probe,)


def test_roles_are_checked_and_the_layer_form_still_works():
    with pytest.raises(AttentionBindingError, match="rollout_contract.role"):
        _bind(rollout_contract=_contract(AttentionRole.TRAIN))
    with pytest.raises(AttentionBindingError, match="training_contract.role"):
        _bind(training_contract=_contract(AttentionRole.INFER))

    class Layer:
        num_heads, num_kv_heads, head_dim = 8, 2, 128

    layer = Layer()
    (c,) = bind_attention_contracts([layer], tp_size=2, cp_size=2)
    assert layer.rl_kernel_attention_contract is c and c.sharding.cp_world_size == 2
    with pytest.raises(TypeError):
        bind_attention_contracts([layer], rollout_contract=c)
    with pytest.raises(TypeError):
        bind_attention_contracts()


def _readback(role, **over):
    c = _contract(role)
    kw = dict(contract=c, actual_knobs={"attention_backend": "b200"}, split_kv_plan_set=_plans(c), source="unit", frozen_scope_verified=True,
              preprocess_backends={"qk_rmsnorm": FUSED_PREPROCESS_BACKEND_ID, "rope": FUSED_PREPROCESS_BACKEND_ID},
              preprocess_probe_id="theta=1e+06", projection_plans=AttentionProjectionOp(8, 1).runtime_readback(), strict_mode=True,
              strict_core_id="b200.blockwise.v1", strict_schedule="ascending_128_key_blocks", native_attention_arithmetic=False,
              strict_split_kv_policy="disabled", actual_backend="b200.cp_attention", communication_backend="symmetric_memory_peer_loads",
              production_ready=True)
    kw.update(over)
    return AttentionRuntimeReadback(**kw)


def _bind_rb(rollout=None, training=None):
    return bind_attention_runtime_readbacks(rollout=rollout or _readback(AttentionRole.INFER), training=training or _readback(AttentionRole.TRAIN),
                                            rollout_identity=_identity(), training_identity=_identity(), rollout_backend_id="b200.paged",
                                            training_backend_id="b200.cp_attention")


def test_runtime_readbacks_bind_and_report_what_each_side_ran():
    res = _bind_rb()
    assert res.passed, [i.to_dict() for i in res.issues]
    assert res.provenance["runtime_readbacks"]["rollout"]["strict_attention"]["core_id"] == "b200.blockwise.v1"
    cases = [
        (dict(frozen_scope_verified=False), BindingErrorCode.DETERMINISM_INCOMPATIBLE, "rollout.frozen_scope_verified"),
        (dict(preprocess_backends={"rope": FUSED_PREPROCESS_BACKEND_ID}), BindingErrorCode.ATTENTION_PREPROCESS_MISSING, "rollout.preprocess.qk_rmsnorm"),
        (dict(preprocess_backends={"qk_rmsnorm": "vendor.rmsnorm", "rope": FUSED_PREPROCESS_BACKEND_ID}),
         BindingErrorCode.ATTENTION_PREPROCESS_MISMATCH, "rollout.preprocess.qk_rmsnorm"),
        (dict(preprocess_fallback=True, preprocess_fallback_reason="probe failed"), BindingErrorCode.ATTENTION_PREPROCESS_FALLBACK,
         "rollout.preprocess.fallback"),
        (dict(projection_plans={"qkv": AttentionProjectionOp(8, 1).runtime_readback()["qkv"]}), BindingErrorCode.ATTENTION_PROJECTION_MISSING,
         "rollout.projection.o_proj"),
        (dict(actual_backend=None), BindingErrorCode.ATTENTION_BACKEND_MISSING, "rollout.runtime.actual_backend"),
        (dict(communication_backend="nccl_ring"), BindingErrorCode.ATTENTION_BACKEND_MISSING, "rollout.runtime.communication_backend"),
        (dict(production_ready=False), BindingErrorCode.ATTENTION_NOT_PRODUCTION_READY, "rollout.runtime.production_ready"),
        (dict(native_attention_arithmetic=True), BindingErrorCode.ATTENTION_NATIVE_ARITHMETIC,
         "rollout.strict_attention.native_attention_arithmetic"),
        (dict(strict_schedule="descending"), BindingErrorCode.ATTENTION_CORE_SCHEDULE, "strict_attention.schedule"),
        (dict(strict_core_id="other.core"), BindingErrorCode.ATTENTION_CORE_MISMATCH, "strict_attention.core_id"),
        (dict(strict_mode=False), BindingErrorCode.ATTENTION_CORE_MISMATCH, "strict_attention.enabled"),
        (dict(preprocess_probe_id="theta=10000"), BindingErrorCode.ATTENTION_PREPROCESS_MISMATCH, "preprocess.probe_id"),
    ]
    for over, code, fld in cases:
        res = _bind_rb(rollout=_readback(AttentionRole.INFER, **over))
        assert res.comparable and not res.passed, over
        assert fld in {i.field for i in res.issues_by_code(code)}, (over, [i.to_dict() for i in res.issues])
    plans = dict(AttentionProjectionOp(8, 1).runtime_readback())
    plans["o_proj"] = {**plans["o_proj"], "split_k": True, "canonical_k_chunks": 4}
    res = _bind_rb(training=_readback(AttentionRole.TRAIN, projection_plans=plans))
    assert {i.field for i in res.issues_by_code(BindingErrorCode.ATTENTION_CORE_SPLIT_K)} == {"training.projection.o_proj.split_k"}
    assert "projection.o_proj.canonical_k_chunks" in {i.field for i in res.issues_by_code(BindingErrorCode.ATTENTION_PROJECTION_MISMATCH)}


def test_readback_validation():
    with pytest.raises(ValueError, match="fallback_reason"):
        _readback(AttentionRole.INFER, preprocess_fallback=True)
    with pytest.raises(TypeError, match="SplitKVRuntimePlanSet"):
        _readback(AttentionRole.INFER, split_kv_plan_set=None)
    with pytest.raises(ValueError, match="strict_split_kv_policy"):
        _readback(AttentionRole.INFER, strict_split_kv_policy="sometimes")
    with pytest.raises(ValueError, match="source"):
        _readback(AttentionRole.INFER, source=" ")
    other = build_split_kv_runtime_plan_set([512] * 3, tp_world_size=2, cp_world_size=2, split_kv=SplitKVSpec.disabled())
    with pytest.raises(ValueError, match="batch_size"):
        _readback(AttentionRole.INFER, split_kv_plan_set=other)
    rb = _readback(AttentionRole.INFER)
    with pytest.raises(TypeError):
        rb.actual_knobs["x"] = 1                                          # frozen views
    assert rb.split_kv_fallback is False and rb.to_dict()["runtime_backend"]["production_ready"] is True
    assert ReductionSpec().merge.value == "online_softmax_lse" and AttentionMode.PREFILL.value
