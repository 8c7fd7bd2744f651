"""The vLLM-side binding against stand-in classes shaped like vLLM's v1 interfaces: attention over a block KV cache
with block tables, the backend object, LM-head padding, fused-residual RMSNorm, support capture and the samplers."""
import types

import pytest
import torch

from rl_engine.integrations.engines.rollout.vllm import sampling_support
from rl_engine.integrations.engines.rollout.vllm.backend import (BACKEND_NAME, RLKernelAttentionBackend,
                                                                 RLKernelAttentionImpl)
from rl_engine.integrations.engines.rollout.vllm.operators import VllmAttentionOperator, VllmKVCacheView
from rl_engine.integrations.engines.rollout.vllm.runtime import (fused_add_rms_norm, install_vllm_integration,
                                                                 last_rollout_support_threshold, patch_lm_head_padding)
from rl_engine.integrations.engines.rollout.vllm.sampler import (NormalizedRolloutCandidate, VLLMSamplerConfig,
                                                                 VLLMSharedPrefixSampler)
from rl_engine.reference.attention.standard_attn import NativeAttentionOp
from rl_engine.runtime.plan import IntegrationPlan

HQ, HKV, D = 4, 2, 128


def _metadata(block_table, seq_lens, qsl, slots):
    return types.SimpleNamespace(num_actual_tokens=qsl[-1], block_table=torch.tensor(block_table, dtype=torch.int32),
                                 seq_lens=torch.tensor(seq_lens), query_start_loc=torch.tensor(qsl),
                                 slot_mapping=torch.tensor(slots), causal=True, use_cascade=False)


def _slots(table_row, positions):
    return [table_row[p // 128] * 128 + p % 128 for p in positions]


def test_attention_over_block_cache_prefill_then_decode_matches_dense_attention():
    torch.manual_seed(0)
    kv_cache = torch.zeros(2, 8, 128, HKV, D)
    table = [[5, 2, -1], [7, -1, -1]]
    lens = [150, 40]
    K = [torch.randn(n, HKV, D) for n in lens]
    V = [torch.randn(n, HKV, D) for n in lens]
    Q = [torch.randn(n, HQ, D) for n in lens]
    impl = RLKernelAttentionImpl(HQ, D, D ** -0.5, HKV)
    # step 1: both requests prefill (the K/V rows are written by the call itself)
    md = _metadata(table, lens, [0, 150, 190], _slots(table[0], range(150)) + _slots(table[1], range(40)))
    out = torch.empty(190, HQ * D)
    impl.forward(impl, torch.cat(Q).view(190, -1), torch.cat(K).view(190, -1), torch.cat(V).view(190, -1), kv_cache, md, out)
    ref = NativeAttentionOp()
    for i, (a, b) in enumerate([(0, 150), (150, 190)]):
        want = ref(Q[i][None], K[i][None], V[i][None], causal=True)[0]
        assert torch.allclose(out[a:b].view(-1, HQ, D), want, atol=1e-5)
    # step 2: one decode token each; the cache now holds 151 / 41 tokens (request 0 crosses into its second page)
    k1, v1, q1 = torch.randn(2, HKV, D), torch.randn(2, HKV, D), torch.randn(2, HQ, D)
    md = _metadata(table, [151, 41], [0, 1, 2], _slots(table[0], [150]) + _slots(table[1], [40]))
    o = impl.forward(impl, q1.view(2, -1), k1.view(2, -1), v1.view(2, -1), kv_cache, md)
    for i in range(2):
        kk, vv = torch.cat([K[i], k1[i:i + 1]]), torch.cat([V[i], v1[i:i + 1]])
        want = ref(q1[i:i + 1][None], kk[None], vv[None], causal=True)[0]
        assert torch.allclose(o[i].view(1, HQ, D), want, atol=1e-5)
    assert impl.op.calls["paged"] == 2
    # a negative slot is a padding token: nothing is written for it
    before = kv_cache.clone()
    md = _metadata(table, [151, 41], [0, 1, 2], [-1, -1])
    impl.forward(impl, q1.view(2, -1), k1.view(2, -1), v1.view(2, -1), kv_cache, md)
    assert torch.equal(before, kv_cache)
    assert impl.forward(impl, q1.view(2, -1), None, None, kv_cache, None, torch.ones(2, HQ * D)).abs().sum() == 0   # profiling


def test_backend_object_answers_the_engine_and_rejects_what_the_kernel_cannot_do():
    assert RLKernelAttentionBackend.get_name() == BACKEND_NAME and RLKernelAttentionBackend.get_impl_cls() is RLKernelAttentionImpl
    assert RLKernelAttentionBackend.get_supported_kernel_block_sizes() == [128]
    assert RLKernelAttentionBackend.get_kv_cache_shape(10, 128, 2, 128) == (2, 10, 128, 2, 128)
    with pytest.raises(ValueError):
        RLKernelAttentionBackend.get_kv_cache_shape(10, 16, 2, 128)
    with pytest.raises(ValueError, match="--block-size 128"):
        VllmKVCacheView.from_tensor(torch.zeros(2, 4, 16, 2, 128))
    for bad in (dict(sliding_window=1024), dict(alibi_slopes=[0.1]), dict(kv_cache_dtype="fp8"), dict(attn_type="encoder")):
        with pytest.raises(NotImplementedError):
            RLKernelAttentionImpl(HQ, D, 1.0, HKV, **bad)
    with pytest.raises(NotImplementedError):
        RLKernelAttentionImpl(HQ, 64, 1.0, HKV)
    impl = RLKernelAttentionImpl(HQ, D, 1.0, HKV)
    md = types.SimpleNamespace(causal=True, use_cascade=True)
    with pytest.raises(NotImplementedError, match="cascade"):
        impl.forward(impl, torch.zeros(1, HQ * D), None, None, torch.zeros(2, 1, 128, HKV, D), md)


def test_install_patches_a_backend_impl_class_with_the_engine_signature():
    class Impl:
        num_heads, num_kv_heads, head_dim = HQ, HKV, D

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None):
            raise AssertionError("the engine's own kernel must not run")

    integ = install_vllm_integration(attention_impl_cls=Impl, plan=IntegrationPlan.uniform("R/R"))
    kv_cache = torch.zeros(2, 2, 128, HKV, D)
    md = _metadata([[1]], [3], [0, 3], _slots([1], range(3)))
    q, k, v = torch.randn(3, HQ * D), torch.randn(3, HKV * D), torch.randn(3, HKV * D)
    out = Impl().forward(None, q, k, v, kv_cache, md)
    want = NativeAttentionOp()(q.view(1, 3, HQ, D), k.view(1, 3, HKV, D), v.view(1, 3, HKV, D), causal=True)[0]
    assert torch.allclose(out.view(3, HQ, D), want, atol=1e-5) and integ.readback()["modules"]["attention"]["calls"] == 1


class _ShardIdx:
    def __init__(self, start, end):
        self.org_vocab_start_index, self.org_vocab_end_index = start, end


class FakeVocabEmbedding:
    def __init__(self, num_embeddings, embedding_dim, org_num_embeddings=None, padding_size=64, tp_rank=0, tp_size=1):
        org = org_num_embeddings or num_embeddings
        self.org_vocab_size = org
        self.num_embeddings_padded = (num_embeddings + padding_size - 1) // padding_size * padding_size
        per = self.num_embeddings_padded // tp_size
        self.shard_indices = _ShardIdx(tp_rank * per, (tp_rank + 1) * per)
        self.weight = torch.nn.Parameter(torch.full((per, embedding_dim), 7.0), requires_grad=False)
        self.weight.output_dim = 0

    def weight_loader(self, param, loaded_weight):
        raise AssertionError("the engine's loader is only used for tensors that are not a full real-vocabulary table")


class FakeParallelLMHead(FakeVocabEmbedding):
    pass


def test_lm_head_padding_gives_every_tp_rank_the_trainers_vocabulary_shard():
    real, padded = 1500, 2048
    patch_lm_head_padding(FakeParallelLMHead, FakeVocabEmbedding, real_vocab=real, padded_vocab=padded)
    ckpt = torch.randn(real, 8)
    for tp in (1, 2, 4):
        shards = []
        for r in range(tp):
            head = FakeParallelLMHead(real, 8, tp_rank=r, tp_size=tp)        # the model asks for the real size ...
            assert head.num_embeddings_padded == padded and head.org_vocab_size == padded    # ... and gets the padded one
            head.weight_loader(head.weight, ckpt)
            shards.append(head.weight.data)
        full = torch.cat(shards)
        assert full.shape[0] == padded and torch.equal(full[:real], ckpt) and full[real:].abs().sum() == 0
    with pytest.raises(RuntimeError):
        patch_lm_head_padding(type("H2", (FakeVocabEmbedding,), {}), FakeVocabEmbedding, real_vocab=1500, padded_vocab=1536)


def test_fused_residual_norm_and_support_capture():
    x, res, w = torch.randn(5, 64).bfloat16(), torch.randn(5, 64).bfloat16(), (1 + 0.1 * torch.randn(64)).bfloat16()
    y, new_res = fused_add_rms_norm(x, res, w, 1e-6)
    s = (x.float() + res.float()).bfloat16()
    assert torch.equal(new_res, s)
    want = s.float() * torch.rsqrt(s.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert (y.float() - want).abs().max() < 0.05 and fused_add_rms_norm(x, None, w, 1e-6).shape == x.shape
    # support capture: the wrapped filter records which ids stayed finite
    mod = types.SimpleNamespace(apply_top_k_top_p=lambda logits, k, p: logits.masked_fill(logits < logits.topk(3, -1).values[:, -1:], float("-inf")))
    sampling_support.install_capture(mod)
    logits = torch.randn(4, 50)
    with sampling_support.capture_support(True) as cap:
        mod.apply_top_k_top_p(logits, 3, None)
    assert cap["mask"].sum(1).tolist() == [3] * 4
    thr = sampling_support.support_to_threshold(logits, cap["mask"], temperature=0.5)
    assert torch.equal((logits / 0.5 >= thr[:, None]), cap["mask"])
    with sampling_support.capture_support(False) as cap:
        mod.apply_top_k_top_p(logits, 3, None)
    assert cap == {}


def test_sampler_scores_the_sampled_token_over_the_restricted_support():
    class Model:
        def __init__(self):
            self.lm_head = types.SimpleNamespace(weight=(torch.randn(256, 32) * 0.3).bfloat16())

        def compute_logits(self, hidden_states):
            return (hidden_states.float() @ self.lm_head.weight.float().t()).bfloat16()

    class Sampler:
        def forward(self, logits, sampling_metadata=None):
            return types.SimpleNamespace(sampled_token_ids=logits.float().argmax(-1))

    install_vllm_integration(model_cls=Model, sampler_cls=Sampler, plan=IntegrationPlan.uniform("R/R"), temperature=0.8, top_k=5)
    model, sampler = Model(), Sampler()
    hidden = torch.randn(6, 32).bfloat16()
    logits = model.compute_logits(hidden)
    res = sampler.forward(logits)
    z = logits.float() / 0.8
    keep = z >= z.topk(5, -1).values[:, -1:]
    want = torch.log_softmax(z.masked_fill(~keep, float("-inf")), -1).gather(1, res.sampled_token_ids[:, None])[:, 0]
    assert (res.rl_kernel_logprobs - want).abs().max() < 2e-2
    assert last_rollout_support_threshold().shape == (6,)


def test_vllm_shared_prefix_sampler_groups_and_normalises_outputs():
    calls = {}

    class Engine:
        def generate(self, prompts, params):
            calls["prompts"], calls["params"] = prompts, params
            return [types.SimpleNamespace(request_id=str(i), prompt_token_ids=[1, 2], outputs=[types.SimpleNamespace(
                token_ids=[i, i + 1], text=f"t{i}", finish_reason="length", cumulative_logprob=-0.5 * i, logprobs=None)])
                for i in range(len(prompts))]

    cfg = VLLMSamplerConfig.from_model_config({"vllm": {"model": "m", "num_generations": 2}, "sampler": {"num_generations": 3},
                                               "sampling_params": {"temperature": 0.7}})
    assert cfg.num_generations == 3 and cfg.model == "m"
    s = VLLMSharedPrefixSampler(cfg, engine=Engine(), llm_cls=object, sampling_params_cls=dict)
    res = s.generate(["a", {"prompt_token_ids": [5, 6]}], sampling_params={"top_p": 0.9})
    assert calls["prompts"] == ["a", "a", "a", {"prompt_token_ids": [5, 6]}] + [{"prompt_token_ids": [5, 6]}] * 2
    assert calls["params"] == {"temperature": 0.7, "top_p": 0.9}
    n = res["normalized_outputs"]
    assert len(n) == 2 and len(n[0]) == 3 and isinstance(n[1][2], NormalizedRolloutCandidate)
    assert n[1][2].token_ids == [5, 6] and n[1][2].prompt_index == 1 and n[1][2].candidate_index == 2
    assert "raw_output" not in n[0][0].to_dict()
    with pytest.raises(ValueError):
        VLLMSamplerConfig(num_generations=0)
    with pytest.raises(ValueError):
        VLLMSharedPrefixSampler(VLLMSamplerConfig(), llm_cls=object, sampling_params_cls=dict).engine   # no model named
    built = {}

    class LLM:
        def __init__(self, **kw):
            built.update(kw)

    VLLMSharedPrefixSampler(VLLMSamplerConfig(model="x"), llm_cls=LLM, sampling_params_cls=dict).engine
    assert built == {"model": "x", "enable_prefix_caching": True, "block_size": 128}
