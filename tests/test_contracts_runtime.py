"""Contracts, registry, policy/plan and provenance on CPU."""
import pytest
import torch

from rl_engine.contracts import (AttentionContract, GRPOLossContract, LogprobContract, ShardingSpec,
                                 resolve_tolerance)
from rl_engine.contracts.operators.attention import B200_ATTENTION_CAPABILITY, CPLayout, ReductionSpec
from rl_engine.contracts.operators.logprob import VocabShardingSpec
from rl_engine.runtime.plan import IntegrationPlan
from rl_engine.runtime.policy import RLKernelMode
from rl_engine.runtime.registry import KernelRegistry, kernel_registry, resolve_logp_op_type
from rl_engine.runtime.semantic_registry import semantic_catalog


def test_alias_package_is_same_module():
    import rl_engine.runtime.registry as a
    import rl_kernel_b200.runtime.registry as b

    assert a is b and a.kernel_registry is b.kernel_registry


def test_attention_contract_validation_and_fingerprint():
    c1 = AttentionContract(32, 8, sharding=ShardingSpec(4, 2, CPLayout.ZIGZAG))
    c2 = AttentionContract(32, 8, sharding=ShardingSpec(4, 2, CPLayout.ZIGZAG))
    c3 = AttentionContract(32, 8, sharding=ShardingSpec(4, 2, CPLayout.CONTIGUOUS))
    assert c1.cross_rank_fingerprint() == c2.cross_rank_fingerprint() != c3.cross_rank_fingerprint()
    assert B200_ATTENTION_CAPABILITY.incompatibilities(c1) == []
    assert B200_ATTENTION_CAPABILITY.incompatibilities(AttentionContract(8, 2, head_dim=64))
    with pytest.raises(ValueError):
        ShardingSpec(4, 4, CPLayout.ZIGZAG)           # 16 ranks
    with pytest.raises(ValueError):
        ShardingSpec(1, 2, CPLayout.NONE)
    with pytest.raises(ValueError):
        ReductionSpec(split_kv=True)
    with pytest.raises(ValueError):
        AttentionContract(32, 8, causal=False)


def test_logprob_and_loss_contracts():
    LogprobContract(sharding=VocabShardingSpec(8, 151936, 152576))
    with pytest.raises(ValueError):
        VocabShardingSpec(8, 151936, 152064)          # tiles would straddle shards
    with pytest.raises(ValueError):
        LogprobContract(temperature=0.0)
    with pytest.raises(ValueError):
        GRPOLossContract(samples_per_prompt=1)
    t = resolve_tolerance("det_gemm", torch.bfloat16)
    gold = torch.randn(4, 64) * 10
    assert t.check(gold * (1 + 1e-3), gold)[0] and not t.check(gold + gold.abs().max() * 0.05, gold)[0]


def test_plan_and_mode(monkeypatch):
    p = IntegrationPlan.from_env({"RL_KERNEL_ATTENTION_CASE": "R/R", "RL_KERNEL_FFN_CASE": "P/R", "RL_KERNEL_LOGP_CASE": "r/r"})
    assert p.side("rollout") == {"attention": True, "ffn": False, "logp": True}
    assert not p.bitwise_guarantee and IntegrationPlan.uniform("R/R").bitwise_guarantee
    with pytest.raises(ValueError):
        IntegrationPlan.from_env({"RL_KERNEL_LOGP_CASE": "X/Y"})
    assert RLKernelMode.parse("STRICT") is RLKernelMode.STRICT
    with pytest.raises(ValueError):
        RLKernelMode.parse("bogus")


def test_registry_resolution_and_provenance(monkeypatch):
    reg = KernelRegistry()
    op = reg.get_op("det_gemm")
    a, b = torch.randn(4, 32), torch.randn(32, 8)
    assert torch.allclose(op(a, b), a @ b, atol=1e-4)
    assert reg.last_resolution.op_name == "det_gemm"
    assert resolve_logp_op_type("auto", require_batch_invariant=True) == "batch_invariant_logp"
    with pytest.raises(ValueError):
        resolve_logp_op_type("nope")
    with pytest.raises(KeyError):
        reg.get_op("does_not_exist")
    with pytest.raises(ValueError):
        reg.get_attention_op("auto", contract=AttentionContract(32, 8, sharding=ShardingSpec(1, 2, CPLayout.ZIGZAG)))
    assert reg.provenance()[0]["op"] == "det_gemm"
    assert kernel_registry.get_logprob_op("linear", contract=LogprobContract(temperature=0.7)).inv_temp == pytest.approx(1 / 0.7)


def test_semantic_session_fails_closed():
    s = semantic_catalog.session("t")
    s.observe("attention", "reference", "layer0")
    s.observe("selected_logprob", "reference", "head", fallback=True)
    with pytest.raises(RuntimeError):
        s.assert_no_fallback()
    with pytest.raises(KeyError):
        s.observe("attention", "unknown-backend")
    assert s.readback()["records"]


def test_profiler_reports_blocked_without_a_gpu_and_serialises(tmp_path):
    import json

    import torch

    from rl_kernel_b200.benchmarks.common import PerformanceProfiler, WORKLOAD_REGISTRY

    assert {"det_gemm_4096x12288x4096", "attention_fwd_8x1536", "linear_logp_fwd_4096x151936"} <= set(WORKLOAD_REGISTRY)
    if torch.cuda.is_available():
        return
    prof = PerformanceProfiler(device=torch.device("cpu"), iters=1)
    r = prof.run("rmsnorm_fwd_12288x4096")
    assert r.status == "blocked" and "CUDA" in r.reason
    out = json.loads(prof.to_json(str(tmp_path / "p.json")))
    assert out[0]["name"] == "rmsnorm_fwd_12288x4096" and out[0]["ms"] is None
    prof.to_csv(str(tmp_path / "p.csv"))
