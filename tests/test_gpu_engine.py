"""The Qwen3 engine end to end on a B200: accuracy against an fp32 model, rollout == training
log-probs bit for bit, CUDA-graph decode == eager decode, gradients against autograd."""
import pytest
import torch

from tests.gpu_util import dev, sync_and_check

pytestmark = pytest.mark.gpu


def _spec():
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec

    return Qwen3DenseSpec.scaled(layers=2, hidden=1024, ffn=2048, q_heads=8, kv_heads=2, head_dim=128, vocab=4096)


def _gold_forward(spec, ids, W):
    from rl_kernel_b200.reference.attention.standard_attn import NativeAttentionOp

    B, S = ids.shape
    x = W["embed_tokens.weight"][ids]

    def rms(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * w

    inv = 1.0 / (spec.rope_theta ** (torch.arange(0, 128, 2, device=x.device).double() / 128))
    ang = torch.arange(S, device=x.device).double()[:, None] * inv[None]
    cos, sin = ang.cos().float(), ang.sin().float()

    def rope(t):
        a, b = t[..., :64], t[..., 64:]
        c, s = cos[None, :, None], sin[None, :, None]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    for l in range(spec.num_hidden_layers):
        p = f"layers.{l}"
        h = rms(x, W[f"{p}.input_layernorm.weight"])
        q = (h @ W[f"{p}.self_attn.q_proj.weight"].t()).view(B, S, -1, 128)
        k = (h @ W[f"{p}.self_attn.k_proj.weight"].t()).view(B, S, -1, 128)
        v = (h @ W[f"{p}.self_attn.v_proj.weight"].t()).view(B, S, -1, 128)
        q, k = rope(rms(q, W[f"{p}.self_attn.q_norm.weight"])), rope(rms(k, W[f"{p}.self_attn.k_norm.weight"]))
        a = NativeAttentionOp()(q, k, v).reshape(B, S, -1)
        x = x + a @ W[f"{p}.self_attn.o_proj.weight"].t()
        h2 = rms(x, W[f"{p}.post_attention_layernorm.weight"])
        x = x + (torch.nn.functional.silu(h2 @ W[f"{p}.mlp.gate_proj.weight"].t()) *
                 (h2 @ W[f"{p}.mlp.up_proj.weight"].t())) @ W[f"{p}.mlp.down_proj.weight"].t()
    hf = rms(x, W["norm.weight"])
    return hf, hf @ W["lm_head.weight"].t()


def test_forward_accuracy_and_batch_invariance():
    from rl_kernel_b200.models.qwen3 import Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine

    spec = _spec()
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    eng = Qwen3Engine(spec, PackedParams(spec, 0, 1, dev()).load(w), max_positions=512)
    ids = torch.randint(0, spec.vocab_size, (3, 256), generator=torch.Generator().manual_seed(0)).to(dev())
    hf = eng.forward_hidden(ids).clone()
    sync_and_check()
    W = {k: v.float().to(dev()) for k, v in w.items()}
    gh, gl = _gold_forward(spec, ids, W)
    assert (hf.float().view(3, 256, -1) - gh).abs().max().item() < 0.03 * gh.abs().max().item()
    tg = ids[:, 1:].reshape(-1)
    rows = hf.view(3, 256, -1)[:, :-1].reshape(-1, spec.hidden_size).contiguous()
    lp = eng.logp_from_hidden(rows, tg)
    glp = torch.log_softmax(gl[:, :-1], -1).reshape(-1, spec.vocab_size).gather(1, tg[:, None])[:, 0]
    assert (lp - glp).abs().max().item() < 0.06          # the reference's chain-gate bound on |dlogp|
    one = eng.forward_hidden(ids[1:2]).clone()
    sync_and_check()
    assert torch.equal(hf.view(3, 256, -1)[1], one.view(256, -1))
    # weights survive the round trip through the packed, canonical layout
    back = PackedParams(spec, 0, 1, dev()).load(w).export_local()
    for k, v in w.items():
        assert torch.equal(back[k].cpu(), v), k


def test_grpo_step_rollout_equals_training_bitwise():
    from rl_kernel_b200.models.qwen3 import Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    spec = _spec()
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    prompts = torch.randint(0, spec.vocab_size, (2, 128), generator=torch.Generator().manual_seed(5)).to(dev())
    outs = []
    for graph, mb in ((True, 4), (False, 8)):
        cfg = GRPOConfig(num_prompts=2, group_size=4, prompt_len=128, response_len=96, micro_batch_seqs=mb,
                         lr=1e-4, use_cuda_graph=graph)
        tr = GRPOTrainer(spec, cfg, dev(), weights=w)
        for step in range(2):
            out = tr.step(prompts, step_index=step)
            sync_and_check()
            assert tr.mismatch_count(out["train_logp"], out["old_logp"]) == 0
            assert torch.isfinite(out["grad_norm"]).all()
            if step == 0:
                outs.append({k: out[k].clone() for k in ("tokens", "old_logp", "train_logp")})
    # first step (same weights): CUDA-graph decode == eager decode, and the micro-batch size does not
    # change training log-probs (later steps differ: gradient accumulation order depends on it)
    assert torch.equal(outs[0]["tokens"], outs[1]["tokens"])
    assert torch.equal(outs[0]["old_logp"], outs[1]["old_logp"])
    assert torch.equal(outs[0]["train_logp"], outs[1]["train_logp"])


def test_grouped_prompt_attention_in_decode_keeps_the_bits():
    """Decode with a shared prompt: the group's rows walk the prompt blocks in one tile and every
    sequence resumes from the saved row state; tokens, rollout log-probs and training log-probs must
    equal the run in which every sequence walks its prompt blocks itself."""
    from rl_kernel_b200.models.qwen3 import Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    spec = _spec()                      # 8 query heads on 2 KV heads: 4 rows per sequence and KV head
    w = Qwen3DenseWeights.synthetic(spec, seed=7)
    prompts = torch.randint(0, spec.vocab_size, (2, 256), generator=torch.Generator().manual_seed(9)).to(dev())
    outs = []
    for grouped in (True, False):
        cfg = GRPOConfig(num_prompts=2, group_size=8, prompt_len=256, response_len=140, micro_batch_seqs=8,
                         lr=1e-4, use_cuda_graph=grouped)
        tr = GRPOTrainer(spec, cfg, dev(), weights=w)
        tr.rollout_engine.group_prefix_attention = grouped
        out = tr.step(prompts, step_index=0)
        sync_and_check()
        if grouped:
            assert tr._shared is not None and tr._shared.prefix_tiles is not None
        assert tr.mismatch_count(out["train_logp"], out["old_logp"]) == 0
        outs.append({k: out[k].clone() for k in ("tokens", "old_logp")})
    assert torch.equal(outs[0]["tokens"], outs[1]["tokens"])
    assert torch.equal(outs[0]["old_logp"], outs[1]["old_logp"])


def test_captured_decode_graph_draws_new_noise_every_training_step():
    """The decode graph freezes its scalar arguments; the step still has to reach the sampler."""
    from rl_kernel_b200.models.qwen3 import Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    spec = _spec()
    w = Qwen3DenseWeights.synthetic(spec, seed=11)
    prompts = torch.randint(0, spec.vocab_size, (2, 128), generator=torch.Generator().manual_seed(3)).to(dev())
    cfg = GRPOConfig(num_prompts=2, group_size=4, prompt_len=128, response_len=48, micro_batch_seqs=8,
                     use_cuda_graph=True)
    tr = GRPOTrainer(spec, cfg, dev(), weights=w)
    tr.publish_weights()
    t1, _ = tr.rollout(prompts, step_seed=1)
    t2, _ = tr.rollout(prompts, step_seed=2)     # replays the graph captured with step_seed = 1
    t1b, _ = tr.rollout(prompts, step_seed=1)
    sync_and_check()
    assert torch.equal(t1, t1b)
    assert not torch.equal(t1[:, 130:], t2[:, 130:])


def test_gradients_against_autograd():
    from rl_kernel_b200.models.qwen3 import Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine
    from rl_kernel_b200.models.qwen3.weights import unpack_gate_up, unpack_qkv

    spec = _spec()
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    params = PackedParams(spec, 0, 1, dev(), with_grad=True).load(w)
    eng = Qwen3Engine(spec, params, max_positions=512)
    tok = torch.randint(0, spec.vocab_size, (2, 256), generator=torch.Generator().manual_seed(2)).to(dev())
    lp = eng.train_forward_backward(tok, 128, lambda x: torch.full_like(x, -1.0 / x.numel()))
    sync_and_check()
    W = {k: v.float().to(dev()).requires_grad_(True) for k, v in w.items()}
    _, gl = _gold_forward(spec, tok, W)
    lpg = torch.log_softmax(gl[:, 127:255], -1).gather(-1, tok[:, 128:, None])[..., 0]
    (-lpg.mean()).backward()
    assert (lp - lpg).abs().max().item() < 0.06
    gq, gk, gv = unpack_qkv(spec, params.g["l0.wqkv"])
    gg, gu = unpack_gate_up(spec, params.g["l0.wgu"])
    pairs = {"layers.0.self_attn.q_proj.weight": gq, "layers.0.self_attn.k_proj.weight": gk,
             "layers.0.self_attn.v_proj.weight": gv, "layers.0.self_attn.o_proj.weight": params.g["l0.wo"],
             "layers.0.mlp.gate_proj.weight": gg, "layers.0.mlp.up_proj.weight": gu,
             "layers.0.mlp.down_proj.weight": params.g["l0.wd"], "layers.1.mlp.down_proj.weight": params.g["l1.wd"],
             "layers.0.input_layernorm.weight": params.g["l0.ln1"],
             "layers.1.post_attention_layernorm.weight": params.g["l1.ln2"],
             "layers.0.self_attn.q_norm.weight": params.g["l0.qn"], "layers.0.self_attn.k_norm.weight": params.g["l0.kn"],
             "norm.weight": params.g["norm"], "lm_head.weight": params.g["lm_head"][:4096],
             "embed_tokens.weight": params.g["embed"][:4096]}
    for name, got in pairs.items():
        want = W[name].grad
        err = (got.float() - want).abs().max().item()
        assert err < 0.04 * want.abs().max().item() + 1e-5, f"{name}: err {err} vs max {want.abs().max().item()}"


def test_stored_activation_backward_equals_recompute_bitwise():
    """Keeping a layer's intermediates for its backward gives the gradients of the recomputing path
    bit for bit (the tensors that are rebuilt -- both norms and the activation -- repeat the
    forward's arithmetic)."""
    from rl_kernel_b200.models.qwen3 import Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine

    spec = _spec()
    w = Qwen3DenseWeights.synthetic(spec, seed=4)
    tok = torch.randint(0, spec.vocab_size, (3, 320), device=dev())
    out = []
    for stored in (False, True):
        params = PackedParams(spec, 0, 1, dev(), with_grad=True).load(w)
        eng = Qwen3Engine(spec, params, max_positions=512)
        lp = eng.train_forward_backward(tok, 64, lambda x: torch.full_like(x, -1.0 / x.numel()),
                                        store_activations=stored)
        sync_and_check()
        out.append((lp.clone(), params.grad.clone()))
    assert torch.equal(out[0][0], out[1][0])
    assert torch.equal(out[0][1], out[1][1])
    assert out[0][1].float().abs().sum().item() > 0


def test_top_p_rollout_and_training_logprobs_agree_bitwise():
    """With top-k / top-p the rollout draws from, and scores under, a restricted support; the recorded per-token
    thresholds make reference scoring and training evaluate the same distribution: 0 mismatching log-probs, and
    every sampled token lies inside its support."""
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    spec = Qwen3DenseSpec.scaled(layers=2, hidden=1024, ffn=2048, q_heads=8, kv_heads=2, head_dim=128, vocab=4096)
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    cfg = GRPOConfig(num_prompts=2, group_size=4, prompt_len=128, response_len=96, micro_batch_seqs=4, temperature=0.9,
                     top_k=50, top_p=0.8, lr=1e-4)
    tr = GRPOTrainer(spec, cfg, dev(), weights=w)
    prompts = torch.randint(0, spec.vocab_size, (2, 128), generator=torch.Generator().manual_seed(9)).to(dev())
    res = tr.step(prompts, step_index=0)
    sync_and_check()
    assert res["support"] is not None and res["support"].shape == (8, 96) and torch.isfinite(res["support"]).all()
    assert tr.mismatch_count(res["train_logp"], res["old_logp"]) == 0
    assert torch.isfinite(res["old_logp"]).all() and (res["old_logp"] <= 0).all()
    # the same seed without a restriction samples other tokens / other log-probs at some position
    free = GRPOTrainer(spec, GRPOConfig(num_prompts=2, group_size=4, prompt_len=128, response_len=96, micro_batch_seqs=4,
                                        temperature=0.9, lr=1e-4), dev(), weights=w)
    res2 = free.step(prompts, step_index=0)
    assert res2["support"] is None and not torch.equal(res2["old_logp"], res["old_logp"])
    # restricted log-probs are never below the unrestricted ones of the same token (the support only shrinks)
    lp_free = free.score(free.policy, res["tokens"])
    assert (res["old_logp"] >= lp_free - 1e-5).all()


def test_dense_experiment_arm_with_library_logp_reports_the_drift_the_strict_path_removes(tmp_path):
    from rl_kernel_b200.integrations.orchestrators.vime.experiments.dense import run_arm, validate_run, weight_audit

    s = run_arm.run_arm(tmp_path / "arm", phase="short", group="library_logp", seed=1234, num_rollout=2)
    assert s["strict_mismatches"] == 0 and s["library_mismatches"] > 0
    v = validate_run.validate_run(tmp_path / "arm")
    assert v["valid"], v
    again = run_arm.run_arm(tmp_path / "arm", phase="short", group="library_logp", seed=1234, num_rollout=2)
    assert again["tokens"] == s["tokens"]                      # a finished arm is not run twice
