"""Contracts, registry, policy/plan and provenance on CPU."""
import pytest
import torch

from rl_engine.contracts import (AttentionContract, AttentionContractError, GRPOLossContract, LogprobContract,
                                 LogprobContractError, LossContractError, resolve_tolerance)
from rl_engine.contracts.operators.attention import (B200_ATTENTION_CAPABILITY, REFERENCE_ATTENTION_CAPABILITY,
                                                     AttentionMode, CPLayout, KVCacheSpec, ReductionSpec, ShardingSpec,
                                                     SplitKVSpec, build_split_kv_runtime_plan_set,
                                                     validate_cross_config_alignment, validate_split_kv_plan_set_alignment)
from rl_engine.contracts.operators.logprob import (B200_LOGPROB_CAPABILITY, MaskSpec, VocabShardingSpec)
from rl_engine.contracts.operators.logprob import ShardingSpec as VocabSharding
from rl_engine.contracts.operators.loss import B200_LOSS_CAPABILITY, KLEstimator
from rl_engine.runtime.plan import IntegrationPlan
from rl_engine.runtime.policy import RLKernelMode
from rl_engine.runtime.registry import KernelRegistry, kernel_registry, resolve_logp_op_type
from rl_engine.runtime.semantic_registry import semantic_catalog


def test_alias_package_is_same_module():
    import rl_engine.runtime.registry as a
    import rl_kernel_b200.runtime.registry as b

    assert a is b and a.kernel_registry is b.kernel_registry


def _attn(cp_rank=0, layout=CPLayout.ZIGZAG, tp_rank=0, **kw):
    return AttentionContract.for_layout(32, 8, seq_len=4096, batch_size=2, tp_rank=tp_rank, tp_world_size=4, cp_rank=cp_rank,
                                        cp_world_size=2, layout=layout, **kw)


def test_attention_contract_validation_and_fingerprint():
    c1, c2, c3 = _attn(0), _attn(1, tp_rank=3), _attn(0, CPLayout.CONTIGUOUS)
    # ranks of one invocation agree; another layout is another invocation only through its block tables,
    # which are rank-local -- so the rank-independent identity is the same and the local tables differ
    assert c1.cross_rank_fingerprint() == c2.cross_rank_fingerprint()
    assert c1.sharding.global_block_indices != c3.sharding.global_block_indices
    assert c2.sharding.global_block_token_starts[0] == 1024 and c2.sharding.local_sequence_length == 2048
    assert B200_ATTENTION_CAPABILITY.incompatibilities(c1) == ()
    assert "head_dim=64 is unsupported" in B200_ATTENTION_CAPABILITY.incompatibilities(
        AttentionContract.for_layout(8, 2, head_dim=64, seq_len=256))
    assert REFERENCE_ATTENTION_CAPABILITY.supports(AttentionContract.for_layout(8, 2, head_dim=64, seq_len=256))
    validate_cross_config_alignment(c1, c3)
    with pytest.raises(AttentionContractError, match="head layouts"):
        validate_cross_config_alignment(c1, AttentionContract.for_layout(16, 8, seq_len=4096, batch_size=2))
    with pytest.raises(AttentionContractError):
        ShardingSpec.for_layout(num_q_heads=32, num_kv_heads=8, seq_len=1001, cp_world_size=4, layout="zigzag")
    with pytest.raises(AttentionContractError):
        ShardingSpec.for_layout(num_q_heads=32, num_kv_heads=8, seq_len=1024, cp_world_size=1, layout="zigzag")
    with pytest.raises(AttentionContractError):
        ShardingSpec.for_layout(num_q_heads=32, num_kv_heads=6, seq_len=1024, tp_world_size=4)      # 6 kv heads over TP4
    with pytest.raises(AttentionContractError):
        ReductionSpec(acc_dtype="bf16")
    with pytest.raises(AttentionContractError, match="causal_offsets"):
        AttentionContract("train", "prefill", "bf16", 1, 128, 128, True, None,
                          ShardingSpec.for_layout(num_q_heads=8, num_kv_heads=2, seq_len=128))
    with pytest.raises(AttentionContractError, match="kv_cache"):
        AttentionContract.for_layout(8, 2, seq_len=128, mode=AttentionMode.DECODE)


def test_split_kv_plans_and_paged_cache_identity():
    with pytest.raises(AttentionContractError):
        SplitKVSpec.auto(strict_consistency=True)
    plan = SplitKVSpec.fixed(256).resolve(1000, backend="t")
    assert plan.boundaries == ((0, 256), (256, 512), (512, 768), (768, 1000)) and plan.actual_split_count == 4
    assert SplitKVSpec.disabled().resolve(77, backend="t").boundaries == ((0, 77),)
    a = build_split_kv_runtime_plan_set([1000, 513], tp_world_size=2, cp_world_size=2, split_kv=SplitKVSpec.fixed(256))
    b = build_split_kv_runtime_plan_set([1000, 513], tp_world_size=2, cp_world_size=2, split_kv=SplitKVSpec.fixed(128))
    validate_split_kv_plan_set_alignment(a, a)
    assert len(a.entries) == 2 * 2 * 2 * 2 and a.to_dict()["coverage"].startswith("complete")
    with pytest.raises(AttentionContractError, match="differs"):
        validate_split_kv_plan_set_alignment(a, b)
    kc = KVCacheSpec.contiguous([700, 650], 128, shared_prefix_tokens=512)
    assert kc.block_table == ((0, 1, 2, 3, 4, 5), (0, 1, 2, 3, 6, 7)) and kc.shared_prefix_page_count == 4
    with pytest.raises(AttentionContractError, match="shared across sequences"):
        KVCacheSpec((9, 9), (10, 10), ((0,), (0,)), tuple(range(10)) * 2, 16)                # a writable page used twice
    with pytest.raises(AttentionContractError, match="trailing"):
        KVCacheSpec((19,), (20,), ((0, -1, 1),), tuple(range(20)), 16)
    d = AttentionContract.for_layout(32, 8, seq_len=700, batch_size=2, mode=AttentionMode.DECODE, kv_cache=kc, role="infer")
    assert B200_ATTENTION_CAPABILITY.supports(d) and d.to_dict()["kv_cache"]["shared_prefix_page_count"] == 4


def test_logprob_and_loss_contracts():
    c0 = LogprobContract.for_tokens(6, real_vocab_size=151936, padded_vocab_size=152576, tp_rank=0, tp_world_size=8)
    c5 = LogprobContract.for_tokens(6, real_vocab_size=151936, padded_vocab_size=152576, tp_rank=5, tp_world_size=8)
    assert c0.cross_rank_fingerprint() == c5.cross_rank_fingerprint() and c0.to_dict() != c5.to_dict()
    assert c5.sharding.local_vocab_start == 5 * 19072 and c5.sharding.owner_rank(151935) == 7
    assert B200_LOGPROB_CAPABILITY.incompatibilities(c0) == ()
    ragged = LogprobContract("train", "bf16", MaskSpec.all_active(4), VocabSharding(0, 2, ((0, 1000), (1000, 2048)), 2000, 2048))
    assert any("tile boundaries" in w for w in B200_LOGPROB_CAPABILITY.incompatibilities(ragged))
    with pytest.raises(LogprobContractError, match="contiguous"):
        VocabSharding(0, 2, ((0, 10), (11, 20)), 20, 20)
    with pytest.raises(LogprobContractError, match="collide"):
        LogprobContract("train", "bf16", MaskSpec(2, (True, False), ignore_index=5), VocabSharding.even(
            tp_rank=0, tp_world_size=1, real_vocab_size=10, padded_vocab_size=10))
    with pytest.raises(LogprobContractError):
        MaskSpec(2, (True, 1))
    with pytest.raises(LogprobContractError):
        c0.sharding.owner_rank(152000)                        # padding id
    with pytest.raises(ValueError):
        VocabShardingSpec(8, 151936, 152064)                  # tiles would straddle shards
    with pytest.raises(LogprobContractError):
        LogprobContract.for_tokens(4, real_vocab_size=100, temperature=0.0)
    g1 = GRPOLossContract.simple(num_sequences=64, padded_seq_len=16, dp_rank=1, dp_world_size=4, tp_rank=1, tp_world_size=2,
                                 padded_vocab_size=152576)
    g0 = GRPOLossContract.simple(num_sequences=64, padded_seq_len=16, dp_rank=0, dp_world_size=4, tp_rank=0, tp_world_size=2,
                                 padded_vocab_size=152576)
    assert g0.cross_rank_fingerprint() == g1.cross_rank_fingerprint() and g1.sharding.local_sequence_start == 16
    assert B200_LOSS_CAPABILITY.incompatibilities(g0) == ()
    assert B200_LOSS_CAPABILITY.incompatibilities(GRPOLossContract.simple(
        num_sequences=8, padded_seq_len=4, kl_estimator=KLEstimator.K1_LOG_RATIO)) == ("kl_estimator=k1_log_ratio is unsupported",)
    with pytest.raises(LossContractError):
        GRPOLossContract.simple(num_sequences=8, padded_seq_len=4, samples_per_prompt=1)
    with pytest.raises(LossContractError, match="token slots"):
        GRPOLossContract(LogprobContract.for_tokens(5, real_vocab_size=100), g0.sharding)
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
        reg.get_attention_op("auto", contract=AttentionContract.for_layout(32, 8, seq_len=512, cp_world_size=2, layout="zigzag"))
    assert reg.provenance()[0]["op"] == "det_gemm"
    assert kernel_registry.get_logprob_op("linear", contract=LogprobContract.for_tokens(4, real_vocab_size=1024, temperature=0.7)).inv_temp == pytest.approx(1 / 0.7)


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


def test_semantic_resolution_overrides_and_module_executor():
    import torch

    from rl_engine.runtime.executor import (ModuleForwardExecutor, StatelessForwardConfig, StatelessForwardInputs, collect_stateless_metrics,
                                            score_rewards, summarize_tensor_tree)
    from rl_engine.runtime.operators import OperatorBridge, OperatorOverride
    from rl_engine.runtime.semantic_registry import (OperatorRequirements, OperatorResolutionError, OperatorResolutionPolicy,
                                                     implementation_fingerprint, semantic_catalog)
    from rl_engine.validation.fixtures.cpu_cross_config import SyntheticCpuCausalLM

    cpu = OperatorRequirements("selected_logprob", device_type="cpu", dtype="float32")
    r = semantic_catalog.resolve(cpu)
    assert r.actual_backend == "reference" and not r.fallback
    with pytest.raises(OperatorResolutionError) as e:
        semantic_catalog.resolve(cpu, backend="b200-tcgen05")
    assert len(e.value.trace.decisions) == 2 and "cpu" in str(e.value)
    r2 = semantic_catalog.resolve(cpu, backend="b200-tcgen05", policy=OperatorResolutionPolicy.permissive())
    assert r2.fallback and r2.actual_backend == "reference"
    op = semantic_catalog.instantiate(r2)
    prov = semantic_catalog.instance_provenance(r2, op)
    assert prov.backend_id == "reference" and len(prov.implementation_fingerprint) == 64 and prov.native_library_sha256 is None
    assert implementation_fingerprint(type(op)) == implementation_fingerprint(type(op)) != implementation_fingerprint(OperatorBridge)
    with pytest.raises(OperatorResolutionError):
        semantic_catalog.resolve(OperatorRequirements("no_such_op"))
    bridge = OperatorBridge()
    ov = OperatorOverride.for_target("selected_logprob", "training", "reference")
    res = bridge.resolve_override(ov, requirements={"rollout": cpu, "training": cpu})
    assert res.for_target("training").requested_backend == "reference" and res.for_target("rollout").requested_backend is None
    assert OperatorOverride("attention", rollout_backend="auto").rollout_backend is None
    # nn.Module scoring with an attention-backend fallback chain
    lm = SyntheticCpuCausalLM(vocab_size=512, hidden=32)

    class Picky(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.inner, self.config = lm, type("Cfg", (), {"use_cache": True, "_attn_implementation": "eager"})()

        def forward(self, ids, **kw):
            if self.config._attn_implementation == "flash_attention_2":
                raise ImportError("flash_attn is not installed")
            assert self.config.use_cache is False
            return {"logits": self.inner(ids)}

    model = Picky()
    ids = torch.randint(0, 512, (5, 12), generator=torch.Generator().manual_seed(0))
    cm = torch.zeros(5, 12, dtype=torch.bool)
    cm[:, 6:] = True
    ex = ModuleForwardExecutor(model, StatelessForwardConfig(micro_batch=2, attention_backend="flash_attention_2"))
    out = ex.score(StatelessForwardInputs(ids, completion_mask=cm))
    assert out.attention_backend == "sdpa" and "flash_attn" in out.fallback_reason and model.config.use_cache is True
    ref = torch.log_softmax(lm(ids)[:, :-1], -1).gather(-1, ids[:, 1:, None])[..., 0]
    assert torch.allclose(out.outputs.selected_logprobs[:, 5:], ref[:, 5:], atol=1e-5) and float(out.outputs.selected_logprobs[:, :5].abs().max()) == 0.0
    assert out.metrics["micro_batches"] == 3 and collect_stateless_metrics(out, out)["calls"] == 2
    assert summarize_tensor_tree({"a": torch.zeros(4), "b": [torch.zeros(2, 2)]}).tensors == 2
    rewards = score_rewards(lambda x, **kw: {"scores": x.float().sum(-1, keepdim=True)}, ids, micro_batch=2)
    assert rewards.shape == (5,)
    with pytest.raises(ValueError):
        StatelessForwardConfig(use_cache=True)


def test_numerical_contract_surface():
    import copy

    import torch

    from rl_engine.contracts import numerical as N

    c = N.load_contract()
    N.validate_contract_schema(c)
    pol = N.resolve_dtype_policy()
    assert pol.execution_dtype == "bfloat16" and pol.tf32_candidate_execution == "disabled" and "b200_bf16" in pol.backend_profiles
    t = N.resolve_judgment_tolerance("forward_accuracy", "logprob", torch.bfloat16, arch_key="sm100")
    assert (t.mode, t.atol, t.rtol, t.comparison_rhs_role) == ("tolerance", 0.06, 0.0, "fp32_reference") and N.resolve_logprob_threshold("bf16") == 0.06
    inv = N.resolve_judgment_tolerance("forward_invariance", "attention", "bfloat16")
    assert inv.mode == "bitwise" and inv.check(torch.ones(2), torch.ones(2))[0] and not inv.check(torch.ones(2), torch.ones(2) + 1e-7)[0]
    assert N.resolve_tolerance_support("gradient_accuracy", "reduction", "fp16").status == "optional"
    with pytest.raises(N.ContractResolveError):
        N.resolve_judgment_tolerance("forward_accuracy", "reduction", "float8")
    with pytest.raises(N.ContractResolveError):
        N.assert_comparison_roles("forward_accuracy", "baseline", "fp32_reference")
    N.assert_comparison_roles("train_infer_logprob_parity", "training_style_teacher_forcing", "inference_style_rollout_decode")
    good = N.BackendProvenance("b200_bf16", "b200-tcgen05", "b200-tcgen05", "bfloat16", "float32", "bfloat16", "float32", False, False)
    N.validate_backend_provenance(good)
    for bad in (dict(candidate_tf32_enabled=True), dict(actual_backend="reference"), dict(execution_dtype="float32"), dict(backend_profile="rocm")):
        with pytest.raises(N.ContractResolveError):
            N.validate_backend_provenance(N.BackendProvenance(**{**good.to_dict(), **bad}))
    lp = -torch.rand(4, 8)
    agg = N.compute_logprob_aggregates(lp + 0.01, lp, torch.ones(4, 8, dtype=torch.bool))
    v = N.judge_logprob_aggregates(agg, "bfloat16")
    assert v.passed and abs(agg.max_abs_dlogp - 0.01) < 1e-6 and agg.clipfrac0 == 0.0 and agg.comparison_lhs_role == "training_style_teacher_forcing"
    assert not N.judge_logprob_aggregates(agg, "float32").passed
    far = lp.clone()
    far[0, 0] += 0.5
    assert not N.judge_logprob_aggregates(N.compute_logprob_aggregates(far, lp), "bfloat16").passed
    with pytest.raises(N.ContractResolveError):
        N.compute_logprob_aggregates(lp, lp, torch.zeros(4, 8, dtype=torch.bool))
    nan = lp.clone()
    nan[1, 1] = float("nan")
    with pytest.raises(N.ContractResolveError):
        N.compute_logprob_aggregates(nan, lp)
    broken = copy.deepcopy(c)
    broken["policy"]["backend_private_tolerance_relaxation"] = True
    with pytest.raises(N.ContractSchemaError):
        N.validate_contract_schema(broken)
    broken = copy.deepcopy(c)
    broken["judgments"]["forward_invariance"]["by_op_class"]["attention"]["bfloat16"]["atol"] = 1e-6
    with pytest.raises(N.ContractSchemaError):
        N.validate_contract_schema(broken)
    assert N.default_clip_interval() == (0.8, 1.2) and len(N.tolerance_contract_fingerprint()) == 64
