"""Framework bindings exercised with stand-in classes (no vLLM / Megatron / DeepSpeed / Ray needed)."""
import types

import pytest
import torch

from rl_engine.integrations.common.ray_actor_manager import RayActorManager
from rl_engine.integrations.common.runtime import FrameworkOperatorIntegration
from rl_engine.integrations.common.weights import LocalTensorCopyBridge, WeightPublisher
from rl_engine.integrations.engines.rollout.vllm.runtime import install_vllm_integration
from rl_engine.integrations.engines.train.contract import RolloutStageResult
from rl_engine.integrations.engines.train.deepspeed.adapter import DeepSpeedTrainingWorker
from rl_engine.integrations.engines.train.megatron.runtime import (CanonicalColumnProjection,
                                                                   DeterministicTPOutputProjection,
                                                                   install_megatron_integration)
from rl_engine.runtime.plan import IntegrationPlan


class FakeAttention:
    num_heads, num_kv_heads, head_dim = 4, 2, 64

    def forward(self, q, k, v, **kw):
        raise AssertionError("original attention must not run")


class FakeModel:
    def __init__(self):
        self.lm_head = types.SimpleNamespace(weight=torch.randn(64, 16))

    def compute_logits(self, hidden_states):
        return hidden_states @ self.lm_head.weight.t()


class FakeSampler:
    def forward(self, logits, sampling_metadata=None):
        return types.SimpleNamespace(sampled_token_ids=logits.argmax(-1))


def test_vllm_binding_routes_attention_and_logp():
    integ = install_vllm_integration(attention_cls=FakeAttention, model_cls=FakeModel, sampler_cls=FakeSampler,
                                     plan=IntegrationPlan.uniform("R/R"))
    T = 24
    q, k, v = torch.randn(T, 4 * 64), torch.randn(T, 2 * 64), torch.randn(T, 2 * 64)
    out = FakeAttention().forward(q, k, v, cu_seqlens=[0, 10, 24])
    assert out.shape == (T, 256)
    model, sampler = FakeModel(), FakeSampler()
    hidden = torch.randn(5, 16)
    res = sampler.forward(model.compute_logits(hidden))
    want = torch.log_softmax(hidden @ model.lm_head.weight.t(), -1).gather(1, res.sampled_token_ids[:, None])[:, 0]
    assert torch.allclose(res.rl_kernel_logprobs, want, atol=1e-4)
    rb = integ.readback()
    assert rb["modules"]["attention"]["calls"] == 1 and rb["modules"]["logp"]["calls"] == 1
    with pytest.raises(RuntimeError):
        integ.assert_strict_ready()          # the plan also wants an ffn operator, none was installed


def test_plan_gates_installation(tmp_path, monkeypatch):
    integ = FrameworkOperatorIntegration("vllm", "rollout", IntegrationPlan.uniform("P/R"))
    with pytest.raises(RuntimeError):
        integ.install("attention", object())
    monkeypatch.setenv("RL_KERNEL_READBACK_DIR", str(tmp_path))
    assert integ.persist_readback().exists()


def test_megatron_projections_tp_simulated():
    torch.manual_seed(0)
    H, I = 64, 128
    x = torch.randn(6, H)
    w1, w2 = torch.randn(I, H), torch.randn(H, I)
    full = DeterministicTPOutputProjection(w2.clone(), canonical_tp=8, tp_size=1)(CanonicalColumnProjection(w1.clone())(x))
    from rl_engine.distributed import balanced_tree_sum

    parts = []
    for r in range(2):
        col = CanonicalColumnProjection(w1[r * 64:(r + 1) * 64].clone())
        row = DeterministicTPOutputProjection(w2[:, r * 64:(r + 1) * 64].clone(), canonical_tp=8, tp_size=2)
        parts.append(row(col(x)))
    assert torch.equal(balanced_tree_sum(parts), full)


class FakeEngine:
    def __init__(self):
        self.module = torch.nn.ModuleDict({"emb": torch.nn.Embedding(32, 16), "lm_head": torch.nn.Linear(16, 32, bias=False)})
        self.opt = torch.optim.SGD(self.module.parameters(), lr=0.1)

    def backward(self, loss):
        loss.backward()

    def step(self):
        self.opt.step()
        self.opt.zero_grad()


def test_deepspeed_worker_trains_and_publishes():
    eng = FakeEngine()
    bridge = LocalTensorCopyBridge()
    w = DeepSpeedTrainingWorker(eng, WeightPublisher(bridge), hidden_fn=lambda m, ids: m["emb"](ids),
                                lm_head_name="lm_head.weight", kl_coef=0.0)
    B, P, R = 4, 3, 5
    tokens = torch.randint(0, 32, (B, P + R))
    with torch.no_grad():
        h = eng.module["emb"](tokens)[:, P - 1:P - 1 + R]
        old = torch.log_softmax(h @ eng.module["lm_head"].weight.t(), -1).gather(-1, tokens[:, P:, None])[..., 0]
    ro = RolloutStageResult(tokens, torch.ones(B, R, dtype=torch.bool), old, torch.tensor([1.0, 0.0, 1.0, 1.0]), P, 2)
    before = eng.module["lm_head"].weight.detach().clone()
    res = w.train(ro)
    assert res.tokens_compared == B * R and not torch.equal(before, eng.module["lm_head"].weight)
    m = w.publish_weights(1)
    assert "lm_head.weight" in m.tensors and m.metadata["layout"]["kind"] == "full-state"


class FakeRay:
    class _Ref:
        def __init__(self, v):
            self.v = v

    def remote(self, **kw):
        ray = self

        def deco(cls):
            class Handle:
                def __init__(self, obj):
                    for name in ("call", "health"):
                        fn = getattr(obj, name)
                        setattr(self, name, types.SimpleNamespace(remote=lambda *a, _f=fn, **k: ray._Ref(_f(*a, **k))))

            return types.SimpleNamespace(remote=lambda *a, **k: Handle(cls(*a, **k)))

        return deco

    def get(self, ref):
        return ref.v

    def kill(self, actor):
        pass


def test_ray_actor_manager_with_fake_ray():
    mgr = RayActorManager(ray_module=FakeRay())

    class W:
        def __init__(self, k):
            self.k = k

        def ping(self, x):
            return x * self.k

    mgr.spawn("a", "rollout", W, 2)
    mgr.spawn("b", "rollout", W, 3)
    assert mgr.call("a", "ping", 5) == 10 and mgr.broadcast("rollout", "ping", 1) == {"a": 2, "b": 3}
    assert mgr.health_check() == {"a": True, "b": True}
    with pytest.raises(ValueError):
        mgr.spawn("a", "rollout", W, 1)
    mgr.shutdown()
    assert not mgr.workers


def test_vime_providers_over_structural_requests():
    from types import SimpleNamespace as NS

    import torch

    from rl_engine.integrations.vime import attention as att, linear_logp_provider as llp, logp

    g = torch.Generator().manual_seed(0)
    T, V, H = 9, 1024, 64
    logits, tg = torch.randn(T, V, generator=g), torch.randint(0, 1000, (T,), generator=g)
    md = {"real_vocab_size": 1000, "padded_vocab_size": 1024}
    r = logp.provider(NS(logits=logits, target_ids=tg, metadata=md, context_parallel=NS(world_size=1, rank=0, layout="single"),
                         tensor_parallel_group=None, with_entropy=True))
    ref = torch.log_softmax(logits[:, :1000], -1).gather(1, tg[:, None])
    assert (r.selected_logprobs - ref).abs().max() < 1e-5 and r.entropy.shape == (T,) and not r.provenance["cp_row_ownership"]["cp_is_merge_axis"]
    keep = torch.rand(T, V, generator=g) > 0.5
    keep[torch.arange(T), tg] = True
    r2 = logp.provider(NS(logits=logits, target_ids=tg, metadata=md, log_prob_keep_mask=keep))
    ref2 = torch.log_softmax(logits.masked_fill(~keep, float("-inf"))[:, :1000], -1).gather(1, tg[:, None])
    assert (r2.selected_logprobs - ref2).abs().max() < 1e-5 and r2.provenance["execution"]["top_p_replay"]
    for bad in (NS(logits=logits, target_ids=tg, metadata={"real_vocab_size": 1000, "padded_vocab_size": 2048}),
                NS(logits=logits, target_ids=tg[:-1], metadata=md),
                NS(logits=logits, target_ids=tg, metadata=md, context_parallel=NS(world_size=2, rank=0, layout="single"))):
        try:
            logp.provider(bad)
            raise AssertionError("accepted an inconsistent request")
        except logp.SelectedLogprobProviderUnavailable as exc:
            assert exc.selected_logprob_provider_unavailable
    hid = torch.randn(T, H, generator=g)
    W = torch.zeros(V, H)
    W[:1000] = torch.randn(1000, H, generator=g) * 0.1
    r3 = llp.provider(NS(hidden=hid, weight=W, target_ids=tg, metadata=md, temperature=0.7))
    ref3 = torch.log_softmax((hid @ W.t())[:, :1000] / 0.7, -1).gather(1, tg[:, None])
    assert (r3.selected_logprobs - ref3).abs().max() < 1e-5 and not r3.provenance["execution"]["logits_materialized"]
    q, k, v = torch.randn(32, 4, 16, generator=g), torch.randn(32, 2, 16, generator=g), torch.randn(32, 2, 16, generator=g)
    r4 = att.attention_provider(NS(q=q, k=k, v=v, metadata={"global_sequence_length": 16, "num_sequences": 2}))
    assert r4.out.shape == q.shape and r4.lse.shape == (32, 4)
    try:
        att.attention_provider(NS(q=q, k=k, v=v, sliding_window=(128, 0), metadata={"global_sequence_length": 16, "num_sequences": 2}))
        raise AssertionError("accepted a sliding window")
    except att.AttentionProviderUnavailable:
        pass


def test_rollout_payload_contract_round_trip():
    from types import SimpleNamespace as NS

    import pytest
    import torch

    from rl_engine.integrations.engines.train import contract as C

    def completion(ids, lps):
        return NS(token_ids=ids, logprobs=[{t: NS(logprob=l)} for t, l in zip(ids, lps)])

    payload = [NS(prompt_token_ids=[5, 6, 7], outputs=[completion([1, 2], [-0.1, -0.2]), completion([3], [-0.3])]),
               {"prompt_token_ids": [8, 9, 10], "outputs": [{"token_ids": [4, 4, 4], "rollout_logprobs": [-1.0, -1.1, -1.2]},
                                                            {"token_ids": [2, 1], "rollout_logprobs": [-0.5, -0.6]}]}]
    assert C.extract_rollout_candidate_groups(payload) == [[[1, 2], [3]], [[4, 4, 4], [2, 1]]]
    assert C.extract_rollout_token_groups(payload) == [[5, 6, 7], [8, 9, 10]]
    with pytest.raises(ValueError):
        C.extract_rollout_reward_groups(payload)
    inp = C.build_stateless_inputs_from_rollout_payload(payload, pad_token_id=0)
    assert inp.input_ids.shape == (4, 6) and inp.completion_mask.sum().item() == 8 and inp.attention_mask[1].tolist() == [True] * 4 + [False] * 2
    ref = torch.arange(24, dtype=torch.float32).view(4, 6)
    C.attach_stateless_scores_to_payload(payload, rewards=torch.tensor([1.0, 0.0, 0.5, 0.5]), reference_logps=ref, completion_mask=inp.completion_mask)
    assert C.extract_rollout_reward_groups(payload) == [[1.0, 0.0], [0.5, 0.5]]
    assert C.extract_rollout_reference_logp_groups(payload)[1][0] == [15.0, 16.0, 17.0]
    adv = C.compute_group_relative_advantages(C.extract_rollout_reward_groups(payload))
    assert abs(adv[0][0] - 1.0) < 1e-5 and adv[1] == [0.0, 0.0]
    res = C.make_rollout_result(payload, pad_token_id=0, weight_version=3)
    assert res.tokens.shape == (4, 6) and res.response_mask.sum().item() == 8 and abs(float(res.rollout_logp[2, 2]) + 1.2) < 1e-6
    assert res.samples_per_prompt == 2 and res.prompt_len == 3
    assert C.broadcast_sequence_advantages(torch.tensor([2.0, -1.0]), torch.tensor([[1, 1, 0], [1, 0, 0]])).tolist() == [[2.0, 2.0, 0.0], [-1.0, 0.0, 0.0]]
    assert C.objective_reference_logps(None, torch.zeros(2), 0.0) is None
    with pytest.raises(ValueError):
        C.objective_reference_logps(None, torch.zeros(2), 0.1)
    with pytest.raises(ValueError):
        C.TorchRLTrainingConfig(clip_eps=1.5)


def test_training_batch_from_rollout_payload_or_synthetic():
    from rl_kernel_b200.integrations.engines.train.contract import batch_from_candidate_groups, batch_from_rollout_or_synthetic

    payload = {"groups": [{"prompt_token_ids": [1, 2, 3],
                           "candidates": [{"token_ids": [4, 5, 6, 7], "reward": 1.0, "logprobs": [-.1, -.2, -.3, -.4]},
                                          {"token_ids": [8, 9], "reward": 0.0, "logprobs": [-.5, -.6]}]}]}
    b, prov = batch_from_rollout_or_synthetic(payload, completion_len=4)
    assert prov == {"training_data_source": "rollout_payload", "reward_source": "payload_rewards", "reference_logp_source": "zeros",
                    "old_logp_source": "payload_rollout_logps", "rollout_prompt_groups": 1, "rollout_sequences": 2, "rollout_tokens": 6}
    assert b.input_ids.tolist() == [[1, 2, 3, 4, 5, 6, 7], [1, 2, 3, 8, 9, 0, 0]] and b.completion_mask.tolist() == [[True] * 4, [True, True, False, False]]
    assert torch.allclose(b.old_logps[1], torch.tensor([-.5, -.6, 0, 0])) and b.prompt_len == 3 and b.valid_indices.tolist() == [0, 1, 2, 3, 4, 5]
    assert b.advantages[0, 0] > 0 > b.advantages[1, 0] and (b.advantages[1, 2:] == 0).all()             # group-relative, masked
    for c in payload["groups"][0]["candidates"]:
        c["reference_logprobs"] = [-1.0] * len(c["token_ids"])
        del c["reward"]
    b, prov = batch_from_rollout_or_synthetic(payload, completion_len=3)                                  # completions cut to 3
    assert prov["reward_source"] == "token_id_proxy" and prov["reference_logp_source"] == "payload_reference_logps"
    assert b.completion_len == 3 and (b.ref_logps[0] == -1).all() and b.ref_logps[1].tolist() == [-1.0, -1.0, 0.0]
    s1, p1 = batch_from_rollout_or_synthetic(None, iteration=3, seed=10)
    s2, _ = batch_from_rollout_or_synthetic({}, iteration=3, seed=10)
    assert p1["training_data_source"] == "synthetic_fallback" and torch.equal(s1.input_ids, s2.input_ids)
    assert not torch.equal(s1.input_ids, batch_from_rollout_or_synthetic(None, iteration=4, seed=10)[0].input_ids)
    with pytest.raises(ValueError):
        batch_from_candidate_groups([[]])
    with pytest.raises(ValueError, match="one length"):
        batch_from_candidate_groups([[[1]], [[2]]], [[1, 2], [3]])
    uneven = batch_from_candidate_groups([[[1, 2], [3]], [[4]]], reward_groups=[[1.0, 0.0], [0.5]])
    assert uneven.metadata["samples_per_prompt"] is None and uneven.metadata["group_sizes"] == [2, 1] and uneven.advantages[2].abs().max() == 0


def test_deepspeed_engine_construction_with_a_stand_in_module(tmp_path):
    import types

    from rl_kernel_b200.integrations.common.weights import make_weight_bridge
    from rl_kernel_b200.integrations.engines.train.deepspeed import adapter as ds

    cfg = ds.DeepSpeedTrainingConfig(zero_stage=3, micro_batch_size=4, dtype=torch.float32,
                                     deepspeed_config={"zero_optimization": {"stage3_param_persistence_threshold": 0}, "wall_clock_breakdown": True})
    conf = ds.resolved_deepspeed_config(cfg)
    assert conf["zero_optimization"] == {"stage": 3, "overlap_comm": False, "contiguous_gradients": True, "reduce_scatter": True,
                                         "stage3_param_persistence_threshold": 0}
    assert conf["bf16"] == {"enabled": False} and conf["wall_clock_breakdown"] is True and conf["communication_data_type"] == "fp32"
    assert ds.resolved_zero_stage(conf) == 3 and ds.resolved_zero_stage({"zero_optimization": False}, fallback=2) == 0
    assert ds.resolved_zero_stage({}, fallback=2) == 2
    with pytest.raises(ValueError):
        ds.DeepSpeedTrainingConfig(zero_stage=4)
    with pytest.raises(ds.DeepSpeedUnavailableError):
        ds.load_deepspeed()                                                   # not installed in this environment
    # toolkit discovery: a directory with bin/nvcc and include/cuda.h is taken, PATH is extended, an explicit value wins
    root = tmp_path / "cu"
    (root / "bin").mkdir(parents=True)
    (root / "include").mkdir()
    (root / "bin" / "nvcc").write_text("")
    (root / "include" / "cuda.h").write_text("")
    assert ds.looks_like_cuda_home(root) and not ds.looks_like_cuda_home(tmp_path)
    assert ds.configure_cuda_home({"CUDA_HOME": "/somewhere"}) == "/somewhere"
    # output readers
    h = torch.randn(2, 5, 16)
    out = types.SimpleNamespace(last_hidden_state=h, logits=torch.randn(2, 5, 64))
    assert ds.extract_hidden_states(out, expected_hidden_dim=16) is h and ds.extract_logits(out).shape[-1] == 64
    assert ds.extract_hidden_states({"hidden_states": (torch.zeros(1), h)}) is h and ds.extract_hidden_states((torch.randn(2, 5, 64), h), expected_hidden_dim=16) is h
    with pytest.raises(TypeError, match="width 16"):
        ds.extract_hidden_states(types.SimpleNamespace(logits=torch.randn(2, 5, 64)), expected_hidden_dim=16)
    assert ds.first_initialize_result((1, 2, 3)) == 1 and ds.first_initialize_result("e") == "e"
    with pytest.raises(RuntimeError):
        ds.first_initialize_result(())

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(32, 16)
            self.lm_head = torch.nn.Linear(16, 32, bias=False)

        def forward(self, ids):
            return types.SimpleNamespace(last_hidden_state=self.emb(ids), logits=None)

    class Engine:
        def __init__(self, model, config):
            self.module, self.config = model, config
            self.opt = torch.optim.SGD(model.parameters(), lr=0.1)

        def backward(self, loss):
            loss.backward()

        def step(self):
            self.opt.step()
            self.opt.zero_grad()

    seen = {}

    def initialize(model, model_parameters, config, **kw):
        seen.update(config=config, kw=kw, n=len(list(model_parameters)))
        return Engine(model, config), None, None, None

    fake = types.SimpleNamespace(initialize=initialize, zero=types.SimpleNamespace(GatheredParameters=lambda params, modifier_rank=None: __import__("contextlib").nullcontext()))
    worker = ds.build_deepspeed_worker(Tiny(), make_weight_bridge("local-clone", source_worker="t", source_rank=0), cfg, deepspeed_module=fake)
    assert seen["config"]["zero_optimization"]["stage"] == 3 and seen["n"] == 2 and worker.gather_context is not None
    from rl_kernel_b200.integrations.engines.train.contract import RolloutStageResult

    tokens = torch.randint(0, 32, (4, 3 + 5))
    roll = RolloutStageResult(tokens, torch.ones(4, 5, dtype=torch.bool), torch.full((4, 5), -3.0), torch.tensor([1.0, 0.0, 0.5, 0.2]), 3, 2)
    before = worker.engine.module.lm_head.weight.detach().clone()
    res = worker.train(roll)
    assert res.tokens_compared == 20 and not torch.equal(worker.engine.module.lm_head.weight, before)
    manifest = worker.publish_weights(1)
    assert manifest.weight_version == 1


def test_megatron_install_records_hooks_patches_linears_and_uninstalls():
    from rl_kernel_b200.integrations.engines.train.megatron.runtime import (MegatronUnavailable, resolve_megatron_classes,
                                                                           uninstall_megatron_integration)

    class Column(torch.nn.Module):
        def __init__(self, w, bias=None, skip_bias_add=False):
            super().__init__()
            self.weight, self.bias, self.skip_bias_add = torch.nn.Parameter(w), bias, skip_bias_add

        def forward(self, x):
            return "framework", None

    class Row(Column):
        pass

    class Out(torch.nn.Module):
        def __init__(self, w):
            super().__init__()
            self.weight = torch.nn.Parameter(w)

    class Norm(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight, self.eps = torch.nn.Parameter(torch.ones(16)), 1e-6

        def forward(self, x):
            return "framework"

    integ = install_megatron_integration(column_linear_cls=Column, row_linear_cls=Row, output_layer_cls=Out, norm_cls=Norm,
                                         plan=IntegrationPlan.uniform("R/R"))
    rb = integ.readback()
    assert rb["installed_hooks"]["logp"].endswith("Out.selected_logprobs") and rb["installed_hooks"]["attention"].endswith("Row.forward")
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 5, 16, generator=g)
    w1, w2, b = torch.randn(32, 16, generator=g), torch.randn(16, 32, generator=g), torch.randn(32, generator=g)
    y, bias = Column(w1, b, skip_bias_add=True)(x)
    assert y.shape == (2, 5, 32) and bias is b and torch.allclose(y, x @ w1.t(), atol=1e-4)
    y2, none = Column(w1, b)(x)
    assert none is None and torch.allclose(y2, x @ w1.t() + b, atol=1e-4)
    z, _ = Row(w2)(y)
    assert z.shape == (2, 5, 16) and torch.allclose(z, y @ w2.t(), atol=1e-3)
    assert torch.allclose(Norm()(x), x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6), atol=1e-5)
    hidden, tg = torch.randn(7, 16, generator=g), torch.randint(0, 32, (7,), generator=g)
    lp = Out(w1).selected_logprobs(hidden, tg)
    assert torch.allclose(lp, torch.log_softmax(hidden @ w1.t(), -1).gather(1, tg[:, None])[:, 0], atol=1e-4)
    assert integ.readback()["operators"]["logp"]["call_count"] == 1
    # installing again does not stack wrappers; uninstalling restores the framework's own methods and removes added ones
    again = install_megatron_integration(column_linear_cls=Column, row_linear_cls=Row, output_layer_cls=Out, norm_cls=Norm,
                                         plan=IntegrationPlan.uniform("R/R"))
    assert uninstall_megatron_integration(again) == 4 and uninstall_megatron_integration(integ) == 0
    assert Column(w1)(x) == ("framework", None) and Norm()(x) == "framework" and not hasattr(Out, "selected_logprobs")
    with pytest.raises(MegatronUnavailable):
        resolve_megatron_classes()


def test_vllm_operators_provenance_page_validation_and_packed_ffn_binding():
    import types

    from rl_kernel_b200.integrations.engines.rollout.vllm.operators import PAGE, VllmAttentionOperator, VllmFFNOperator, VllmLogpOperator

    g = torch.Generator().manual_seed(0)
    # FFN: weights are read out of an engine-style MLP module ([gate; up] rows) and give silu(gate) * up @ down
    H, I = 32, 64
    mlp = types.SimpleNamespace(gate_up_proj=types.SimpleNamespace(weight=torch.randn(2 * I, H, generator=g) * 0.2),
                                down_proj=types.SimpleNamespace(weight=torch.randn(H, I, generator=g) * 0.2))
    ffn = VllmFFNOperator(canonical_tp=8, tp_size=1)
    assert ffn.bind_packed_inference(mlp) == (H, I) and mlp.rlk_w_gu.shape == (2 * I, H) and mlp.rlk_ffn_version == 1
    x = torch.randn(5, H, generator=g)
    gate, up = mlp.gate_up_proj.weight[:I], mlp.gate_up_proj.weight[I:]
    want = (torch.nn.functional.silu(x @ gate.t()) * (x @ up.t())) @ mlp.down_proj.weight.t()
    assert torch.allclose(ffn(mlp, x), want, atol=1e-4) and ffn.provenance["calls"] == 1 and ffn.provenance["local_k_chunks"] == 8
    fresh = types.SimpleNamespace(gate_up_proj=mlp.gate_up_proj, down_proj=mlp.down_proj)
    assert torch.allclose(VllmFFNOperator()(fresh, x), want, atol=1e-4) and hasattr(fresh, "rlk_w_gu")      # bound on first use
    with pytest.raises(ValueError, match="canonical shards"):
        VllmFFNOperator(canonical_tp=8).bind_packed_inference(types.SimpleNamespace(
            gate_up_proj=types.SimpleNamespace(weight=torch.zeros(2 * 12, H)), down_proj=types.SimpleNamespace(weight=torch.zeros(H, 12))))
    # log-prob operator
    lp_op = VllmLogpOperator(temperature=0.5, real_vocab=40)
    w, hid, ids = torch.randn(48, H, generator=g), torch.randn(6, H, generator=g), torch.randint(0, 40, (6,), generator=g)
    got = lp_op(hid, w, ids)
    assert torch.allclose(got, torch.log_softmax((hid @ w[:40].t()) / 0.5, -1).gather(1, ids[:, None])[:, 0], atol=1e-4)
    assert lp_op.provenance["calls"] == 1 and lp_op.provenance["real_vocab_size"] == 40 and lp_op.provenance["runtime_platform"] == "cpu-reference"
    # attention over a block cache: provenance and the one-time page / slot validation
    hq, hkv, d, nb = 4, 2, 16, 6
    layer = types.SimpleNamespace(num_heads=hq, num_kv_heads=hkv, head_dim=d, head_size=d, scale=None)
    cache = torch.zeros(2, nb, PAGE, hkv, d)
    n = 5
    q, k, v = (torch.randn(n, h * d, generator=g) for h in (hq, hkv, hkv))
    md = types.SimpleNamespace(num_actual_tokens=n, slot_mapping=torch.arange(n) + 2 * PAGE, block_table=torch.tensor([[2, 0, 0]]),
                               seq_lens=torch.tensor([n]), query_start_loc=torch.tensor([0, n]))
    op = VllmAttentionOperator()
    out = op(layer, q, k, v, kv_cache=cache, attn_metadata=md)
    from rl_kernel_b200.ops.attention.attention import causal_attention

    assert torch.allclose(out, causal_attention(q.view(n, hq, d), k.view(n, hkv, d), v.view(n, hkv, d), [0, n]).reshape(n, hq * d), atol=1e-5)
    prov = op.provenance
    assert prov["calls"]["paged"] == 1 and prov["phase"] == "prefill_or_mixed" and prov["split_kv"] == "disabled" and prov["kv_block"] == PAGE
    bad = types.SimpleNamespace(num_actual_tokens=n, slot_mapping=torch.arange(n) + 2 * PAGE, block_table=torch.tensor([[9, 0]]),
                                seq_lens=torch.tensor([n]), query_start_loc=torch.tensor([0, n]))
    with pytest.raises(ValueError, match="outside the pool of 6 pages"):
        VllmAttentionOperator()(layer, q, k, v, kv_cache=cache, attn_metadata=bad)
    off = types.SimpleNamespace(num_actual_tokens=n, slot_mapping=torch.arange(n) + nb * PAGE, block_table=torch.tensor([[2, 0, 0]]),
                                seq_lens=torch.tensor([n]), query_start_loc=torch.tensor([0, n]))
    with pytest.raises(ValueError, match="token slots"):
        VllmAttentionOperator()(layer, q, k, v, kv_cache=cache, attn_metadata=off)
    short = types.SimpleNamespace(num_actual_tokens=1, slot_mapping=torch.tensor([PAGE * 3]), block_table=torch.tensor([[1, 2]]),
                                  seq_lens=torch.tensor([3 * PAGE]), query_start_loc=torch.tensor([0, 1]))
    with pytest.raises(ValueError, match="needs 3 pages"):
        VllmAttentionOperator()(layer, q[:1], k[:1], v[:1], kv_cache=cache, attn_metadata=short)


def test_ray_manager_specs_options_typed_handles_and_runtime():
    from rl_kernel_b200.integrations.common.ray_actor_manager import (RayActorOptions, RayRuntimeConfig, RayUnavailableError, RayWorkerSpec,
                                                                      load_ray)

    opts = RayActorOptions(num_gpus=0.5, resources={"nvlink_domain": 1}, name="trainer-0", max_restarts=2)
    assert opts.to_ray_options() == {"num_gpus": 0.5, "name": "trainer-0", "max_restarts": 2, "resources": {"nvlink_domain": 1}}
    assert RayRuntimeConfig(init_kwargs={"num_cpus": 4}).resolved_init_kwargs() == {"ignore_reinit_error": True, "num_cpus": 4}
    with pytest.raises(RayUnavailableError):
        load_ray()

    class Ray(FakeRay):
        def __init__(self):
            self.inits, self.shutdowns, self.options = [], 0, []

        def init(self, **kw):
            self.inits.append(kw)

        def shutdown(self):
            self.shutdowns += 1

        def remote(self, **kw):
            self.options.append(kw)
            return super().remote(**kw)

    class Trainer:
        def __init__(self, scale):
            self.scale, self.released = scale, []

        def train(self, rollout):
            return rollout * self.scale

        def publish_weights(self, weight_version, tag=None):
            return {"weight_version": weight_version, "tag": tag}

        def release_weights(self, update_id):
            self.released.append(update_id)
            return list(self.released)

        def health_check(self):
            return {"step": 7}

    class Rollout:
        def rollout(self, spec):
            return [spec] * 2

        def update_weights(self, manifest):
            return manifest["weight_version"]

        def release_weights(self):
            return "released"

    ray = Ray()
    with RayActorManager(ray_module=ray, runtime=RayRuntimeConfig(shutdown_ray_on_close=True)) as mgr:
        t = mgr.create_training_worker(RayWorkerSpec(Trainer, args=(3,), actor_options=opts))
        r = mgr.create_rollout_worker(RayWorkerSpec(Rollout))
        assert ray.inits == [{"ignore_reinit_error": True}] and ray.options[0]["name"] == "trainer-0" and ray.options[1] == {"num_gpus": 1.0}
        assert t.train(5) == 15 and t.publish_weights(4, tag="x") == {"weight_version": 4, "tag": "x"} and t.release_weights("u1") == ["u1"]
        assert r.rollout("p") == ["p", "p"] and r.update_weights({"weight_version": 4}) == 4 and r.release_weights() == "released"
        assert set(mgr.workers) == {"trainer-0", "rollout-1"} and mgr.health_check() == {"trainer-0": True, "rollout-1": True}
        with pytest.raises(ValueError, match="already exists"):
            mgr.create_training_worker(RayWorkerSpec(Trainer, args=(1,), actor_options=opts))
    assert ray.shutdowns == 1 and not mgr.workers
