"""Mixture-of-experts kernels (router, dispatch plan, grouped GEMM, combine) against the CPU
restatement of their contract and an fp64 autograd reference."""
import pytest
import torch

from tests.gpu_util import dev, sync_and_check

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _weights(E, H, I, seed=0, grads=False):
    from rl_kernel_b200.ops.moe import MoEWeights

    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s, std: (torch.randn(*s, device=dev(), generator=g) * std).to(BF)  # noqa: E731
    w = MoEWeights(r(E, H, std=0.05), r(E * 2 * I, H, std=0.03), r(E * H, I, std=0.03))
    if grads:
        w.g_router, w.g_w1, w.g_w2 = torch.zeros_like(w.router), torch.zeros_like(w.w1), torch.zeros_like(w.w2)
    return w


def test_router_topk_matches_reference_and_breaks_ties_low():
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.reference.moe import router_topk_reference

    T, E, K = 500, 128, 8
    logits = torch.randn(T, E, device=dev())
    logits[0] = 0.0                      # all tied: experts 0..7 must win
    logits[1, 100:] = 5.0                # 28 tied winners: the lowest 8 of them
    idx = torch.zeros(T, K, dtype=torch.int32, device=dev())
    w = torch.zeros(T, K, device=dev())
    probs = torch.zeros(T, E, device=dev())
    counts = torch.zeros(E, dtype=torch.int32, device=dev())
    nv.moe_router_topk(logits, idx, w, probs, counts)
    sync_and_check()
    ri, rw, rp = router_topk_reference(logits.cpu(), K)
    assert torch.equal(idx.cpu().long(), ri)
    assert idx[0].tolist() == list(range(8)) and idx[1].tolist() == list(range(100, 108))
    assert (w.cpu() - rw).abs().max().item() < 1e-6 and (probs.cpu() - rp).abs().max().item() < 1e-6
    assert torch.equal(counts.cpu().long(), torch.bincount(ri.reshape(-1), minlength=E))
    idx2, w2 = torch.zeros_like(idx[:3]), torch.zeros_like(w[:3])
    nv.moe_router_topk(logits[:3].contiguous(), idx2, w2)
    assert torch.equal(idx2, idx[:3]) and torch.equal(w2, w[:3]), "routing must not depend on the batch"


def test_moe_forward_matches_cpu_contract_and_is_batch_invariant():
    from rl_kernel_b200.ops.moe import MoEBuffers, MoEExperts
    from rl_kernel_b200.reference.moe import moe_dispatch_plan_reference, moe_ffn_reference

    T, H, I, E, K = 384, 512, 256, 32, 4
    wts = _weights(E, H, I)
    x = torch.randn(T, H, device=dev()).to(BF)
    base = torch.randn(T, H, device=dev()).to(BF)
    moe = MoEExperts(MoEBuffers(dev(), hidden=H, inter=I, num_experts=E, top_k=K, max_tokens=T, with_backward=False))
    out = torch.empty_like(x)
    moe.forward(x, wts, out, base)
    sync_and_check()
    ref, ridx, rw = moe_ffn_reference(x.cpu(), wts.router.cpu(), wts.w1.cpu().view(E, 2 * I, H),
                                      wts.w2.cpu().view(E, H, I), K, base.cpu())
    assert torch.equal(moe.idx.cpu().long(), ridx)
    rows, _, total, padded = moe_dispatch_plan_reference([ridx], E)
    assert torch.equal(moe.slot_row.cpu().long().view(T, K), rows[0])
    assert int(moe.b.rows_used.item()) == int(padded.sum())
    err = (out.float().cpu() - ref.float()).abs().max().item()
    assert err < 0.03, err
    # a sub-batch routed alone gives the same bits for its tokens
    T2 = 128
    moe2 = MoEExperts(MoEBuffers(dev(), hidden=H, inter=I, num_experts=E, top_k=K, max_tokens=T2, with_backward=False))
    out2 = torch.empty_like(x[:T2])
    moe2.forward(x[:T2].contiguous(), wts, out2, base[:T2].contiguous())
    sync_and_check()
    assert torch.equal(out2, out[:T2])


def test_moe_backward_matches_fp64_autograd():
    from rl_kernel_b200.ops.moe import MoEBuffers, MoEExperts

    T, H, I, E, K = 256, 512, 256, 32, 4
    wts = _weights(E, H, I, seed=1, grads=True)
    x = torch.randn(T, H, device=dev()).to(BF)
    dout = (torch.randn(T, H, device=dev()) * 0.1).to(BF)
    moe = MoEExperts(MoEBuffers(dev(), hidden=H, inter=I, num_experts=E, top_k=K, max_tokens=T))
    out, dx = torch.empty_like(x), torch.empty_like(x)
    moe.forward(x, wts, out)
    moe.backward(x, dout, wts, dx)
    sync_and_check()
    # fp64 reference with the routing decisions of the kernel
    idx = moe.idx.long()
    xd = x.double().requires_grad_(True)
    wr = wts.router.double().requires_grad_(True)
    w1 = wts.w1.double().view(E, 2 * I, H).requires_grad_(True)
    w2 = wts.w2.double().view(E, H, I).requires_grad_(True)
    p = torch.softmax(xd @ wr.t(), -1)
    sel = torch.gather(p, 1, idx)
    w = sel / sel.sum(-1, keepdim=True)
    y = torch.zeros(T, H, dtype=torch.float64, device=dev())
    for k in range(K):
        e = idx[:, k]
        gu = torch.einsum("th,tnh->tn", xd, w1[e])
        act = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        y = y + w[:, k:k + 1] * torch.einsum("ti,thi->th", act, w2[e])
    (y * dout.double()).sum().backward()

    def close(a, b, name, tol=0.05):
        scale = b.abs().max().item() + 1e-12
        err = (a.double() - b).abs().max().item() / scale
        assert err < tol, f"{name}: relative error {err}"

    close(out, y.detach(), "out", 0.02)
    close(dx, xd.grad, "dx")
    close(wts.g_w1.view(E, 2 * I, H), w1.grad, "dW1")
    close(wts.g_w2.view(E, H, I), w2.grad, "dW2")
    close(wts.g_router, wr.grad, "dWrouter")


def test_moe_engine_rollout_and_training_logp_agree_bitwise():
    """Decode (one token per sequence against the KV cache) and training (full sequences) route
    every token to the same experts and produce the same selected-token log-prob bits."""
    from rl_kernel_b200.models.qwen3_moe import MoEPackedParams, Qwen3MoeEngine, Qwen3MoeSpec

    spec = Qwen3MoeSpec.tiny()
    B, P, R = 4, 128, 24
    S = P + R
    params = MoEPackedParams(spec, 0, 1, dev(), with_grad=True).init_synthetic_(3, std=0.05)
    eng = Qwen3MoeEngine(spec, params, max_tokens=B * S, max_positions=S + 8)
    prompts = torch.randint(0, spec.vocab_size, (B, P), device=dev())
    kv = eng.new_kv_cache(B, S)
    hf = eng.forward_hidden(prompts, kv=kv, tag="p")
    last = hf.view(B, P, -1)[:, P - 1].contiguous()
    keys = torch.arange(B, device=dev(), dtype=torch.int64) * 65536
    dtiles = eng.decode_tiles(B, S)
    toks, lps = [], []
    ids, lp = eng.sample(eng.logits(last), keys + P - 1, temperature=1.0, seed=11)
    for i in range(R):
        toks.append(ids.clone()); lps.append(lp.clone())
        if i == R - 1:
            break
        pos = torch.full((B,), P + i, dtype=torch.int32, device=dev())
        hf = eng.decode_step(ids.clone(), pos, kv, dtiles)
        ids, lp = eng.sample(eng.logits(hf), keys + P + i, temperature=1.0, seed=11)
    tokens = torch.cat([prompts, torch.stack(toks, 1)], 1).contiguous()
    old = torch.stack(lps, 1)
    new = eng.train_forward_backward(tokens, P, lambda x: torch.full_like(x, -1.0 / x.numel()))
    sync_and_check()
    assert torch.equal(new, old), (new - old).abs().max().item()
    assert params.g["l0.w1"].float().abs().sum().item() > 0 and params.g["l1.router"].float().abs().sum().item() > 0
