"""End-to-end GRPO step on the CPU reference model: 2-layer Qwen3-style decoder (hidden 256, 4 q /
2 kv heads, head_dim 64, SwiGLU 768, vocab 4096), 2 prompts x group 4, prompt 32 + response 64.
Rollout (prefill + one-token decode with sampling) and the training forward over the finished
sequences must give bitwise equal selected-token log-probs; the GRPO loss then back-propagates
into every weight."""
import torch

from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
from rl_kernel_b200.models.qwen3.reference import Qwen3DenseBIModel
from rl_kernel_b200.reference.loss.grpo_loss import NativeGRPOLossOp, grpo_loss_from_logps
from rl_kernel_b200.utils.bits import bit_mismatch_count

SPEC = Qwen3DenseSpec.scaled(layers=2, hidden=256, ffn=768, q_heads=4, kv_heads=2, head_dim=64, vocab=4096)


def test_cpu_grpo_step_rollout_matches_training_and_trains():
    torch.set_num_threads(2)
    P, R, G, NP = 32, 64, 4, 2
    B, S = NP * G, P + R
    w = Qwen3DenseWeights.synthetic(SPEC, dtype=torch.float32, seed=0)
    model = Qwen3DenseBIModel(SPEC, w)
    gen = torch.Generator().manual_seed(7)
    prompts = torch.randint(0, SPEC.vocab_size, (NP, P), generator=gen).repeat_interleave(G, dim=0)
    # ---- rollout: prefill, then one token at a time against the KV cache
    with torch.no_grad():
        cache = model.allocate_cache(B, S)
        out = model(prompts, kv_cache=cache)
        hidden = out["hidden"].view(B, P, -1)[:, -1]
        tokens, old = [prompts], []
        for t in range(R):
            logits = model.lm_head_logits(hidden)
            nxt = torch.multinomial(torch.softmax(logits.float(), -1), 1, generator=gen)[:, 0]
            old.append(model.selected_logprobs(hidden, nxt))
            tokens.append(nxt[:, None])
            if t + 1 < R:
                hidden = model.decode_step(nxt, torch.full((B,), P + t), cache, return_logits=False)["hidden"].view(B, -1)
        tokens = torch.cat(tokens, dim=1)
        old_logp = torch.stack(old, dim=1)
    # ---- training forward over whole sequences, one sequence per call and all eight at once
    for k in w.keys():
        w[k].requires_grad_(True)
    lp_all = model(tokens, target_ids=tokens, return_logits=False)["selected_logp"][:, P - 1:]
    with torch.no_grad():
        lp_one = model(tokens[5:6], target_ids=tokens[5:6], return_logits=False)["selected_logp"][:, P - 1:]
    assert bit_mismatch_count(lp_all.detach(), old_logp) == 0, "train vs rollout log-probs"
    assert bit_mismatch_count(lp_one, old_logp[5:6]) == 0, "batch 1 vs batch 8"
    # ---- GRPO loss and backward
    rewards = torch.bernoulli(torch.full((B,), 0.5), generator=gen)
    adv = NativeGRPOLossOp().group_advantages(rewards, samples_per_prompt=G)
    mask = torch.ones(B, R, dtype=torch.bool)
    loss, pol, kl = grpo_loss_from_logps(lp_all, old_logp, old_logp, adv, mask, clip_eps=0.2, beta=0.001)
    loss.backward()
    assert torch.isfinite(loss) and float(kl.detach()) == 0.0
    for k in ("embed_tokens.weight", "layers.1.mlp.down_proj.weight", "layers.0.self_attn.q_norm.weight", "lm_head.weight"):
        g = w[k].grad
        assert g is not None and torch.isfinite(g).all()
    if rewards.min() != rewards.max():
        assert w["lm_head.weight"].grad.abs().sum() > 0
