"""Device operator classes under the reference's import names (rl_engine.backends.cuda.*) against
fp32 PyTorch references of the same operators."""
import math

import pytest
import torch

from tests.gpu_util import dev, sync_and_check

pytestmark = pytest.mark.gpu


def _g(seed):
    return torch.Generator(device="cuda").manual_seed(seed)


def test_rope_op_forward_backward_and_layouts():
    from rl_engine.backends.cuda.rope import RoPESM90Op
    from rl_engine.reference.rope.rope import NativeRoPEOp

    g = _g(1)
    B, H, S, D = 2, 4, 37, 128
    x = torch.randn(B, H, S, D, device=dev(), generator=g).bfloat16().requires_grad_(True)
    pos = torch.stack([torch.arange(S), torch.arange(5, 5 + S)]).to(dev())
    op, ref = RoPESM90Op(), NativeRoPEOp()
    y = op(x, pos, theta=1e6)
    sync_and_check()
    want = ref.forward_fp32(x.detach(), pos, theta=1e6)
    assert torch.equal(y, want.to(torch.bfloat16))                       # fp32 math, one rounding
    gout = torch.randn(B, H, S, D, device=dev(), generator=g).bfloat16()
    y.backward(gout)
    xr = x.detach().float().requires_grad_(True)
    ref.forward_fp32(xr, pos, theta=1e6).backward(gout.float())
    assert (x.grad.float() - xr.grad).abs().max().item() < 2e-2
    # 1-D positions, [S, D] input, fp32 output
    x2 = torch.randn(S, D, device=dev(), generator=g).bfloat16()
    y2 = op.forward_fp32(x2, torch.arange(S, device=dev()))
    assert y2.dtype == torch.float32 and torch.equal(y2, ref.forward_fp32(x2, torch.arange(S, device=dev())))
    # batch invariance: a row alone gives the same bits
    assert torch.equal(op(x.detach()[1:2, :, 3:4], pos[1:2, 3:4]), y.detach()[1:2, :, 3:4])


def test_det_gemm_op_and_lm_head_match_fp32_and_have_gradients():
    from rl_engine.backends.cuda.embedding import SM90LMHeadOp
    from rl_engine.backends.cuda.gemm import DetGemmOp, det_gemm_backend, det_gemm_fallback_reason

    assert det_gemm_backend() == "sm100_tcgen05" and det_gemm_fallback_reason() is None
    g = _g(2)
    M, K, N = 200, 512, 384
    a = (torch.randn(M, K, device=dev(), generator=g) * 0.5).bfloat16().requires_grad_(True)
    b = (torch.randn(K, N, device=dev(), generator=g) * 0.1).bfloat16().requires_grad_(True)
    op = DetGemmOp()
    c = op(a, b)
    sync_and_check()
    ref = a.detach().float() @ b.detach().float()
    assert (c.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item() / 8 + 1e-2
    c32 = op.forward_fp32(a.detach(), b.detach())
    assert c32.dtype == torch.float32 and (c32 - ref).abs().max().item() < 1e-3 * ref.abs().max().item() + 1e-4
    gc = torch.randn(M, N, device=dev(), generator=g).bfloat16()
    c.backward(gc)
    da, db = gc.float() @ b.detach().float().t(), a.detach().float().t() @ gc.float()
    assert (a.grad.float() - da).abs().max().item() < 0.02 * da.abs().max().item() + 1e-2
    assert (b.grad.float() - db).abs().max().item() < 0.02 * db.abs().max().item() + 1e-2
    # batch invariance of a row, and linear() == op(a, w.t())
    assert torch.equal(op(a.detach()[7:8], b.detach()), c.detach()[7:8])
    w = b.detach().t().contiguous()
    assert torch.equal(op.linear(a.detach(), w), c.detach())
    head = SM90LMHeadOp()
    h = a.detach().view(2, 100, K).clone().requires_grad_(True)
    wl = w.clone().requires_grad_(True)
    bias = torch.randn(N, device=dev(), generator=g).bfloat16().requires_grad_(True)
    logits = head(h, wl, bias=bias)
    want = h.detach().float() @ w.float().t() + bias.detach().float()
    assert logits.shape == (2, 100, N) and (logits.float() - want).abs().max().item() < 0.05
    logits.backward(gc.view(2, 100, N))
    assert (bias.grad.float() - gc.float().sum(0)).abs().max().item() < 0.5 and wl.grad.shape == wl.shape
    assert head.forward_fp32(h.detach(), w).dtype == torch.float32


def test_deterministic_attention_op_bhsd_matches_reference_and_pads():
    from rl_engine.backends.cuda.attention import DeterministicAttentionOp, PrefixSharedAttentionOp
    from rl_engine.reference.attention.standard_attn import NativeAttentionOp

    g = _g(3)
    B, HQ, HKV, S, D = 2, 4, 2, 200, 128
    q = torch.randn(B, HQ, S, D, device=dev(), generator=g).bfloat16().requires_grad_(True)
    k = torch.randn(B, HKV, S, D, device=dev(), generator=g).bfloat16().requires_grad_(True)
    v = torch.randn(B, HKV, S, D, device=dev(), generator=g).bfloat16().requires_grad_(True)
    mask = torch.ones(B, S, dtype=torch.bool, device=dev())
    mask[1, 150:] = False
    op = DeterministicAttentionOp()
    o, lse = op.forward_with_lse(q, k, v, causal=True, key_padding_mask=mask)
    sync_and_check()
    ro, rl = NativeAttentionOp()(q.detach().transpose(1, 2).float(), k.detach().transpose(1, 2).float(),
                                 v.detach().transpose(1, 2).float(), causal=True, key_padding_mask=mask, return_lse=True)
    ro, rl = ro.transpose(1, 2), rl.transpose(1, 2)
    valid = mask[:, None, :, None]
    assert ((o.float() - ro) * valid).abs().max().item() < 2e-2
    assert ((lse - rl) * mask[:, None, :]).nan_to_num(0, 0, 0).abs().max().item() < 1e-3
    o.backward(torch.randn(B, HQ, S, D, device=dev(), generator=g).bfloat16() * valid)
    assert torch.isfinite(q.grad).all() and torch.isfinite(k.grad).all() and k.grad[1, :, 150:].abs().max().item() == 0
    # prefix-shared single-head form of the reference: q [bs, G, Lq, D], k/v [bs, Lkv, D]
    qs = torch.randn(2, 4, 3, D, device=dev(), generator=g).bfloat16()
    ks = torch.randn(2, 50, D, device=dev(), generator=g).bfloat16()
    vs = torch.randn(2, 50, D, device=dev(), generator=g).bfloat16()
    got = PrefixSharedAttentionOp()(qs, ks, vs)
    s = torch.einsum("bgqd,bkd->bgqk", qs.float(), ks.float()) / math.sqrt(D)
    want = torch.einsum("bgqk,bkd->bgqd", torch.softmax(s, -1), vs.float())
    assert (got.float() - want).abs().max().item() < 2e-2


def test_elementwise_and_gather_ops_under_reference_names():
    from rl_engine.backends.cuda.activation import SwiGLUCudaOp
    from rl_engine.backends.cuda.embedding import SM90EmbeddingOp
    from rl_engine.backends.cuda.norm import RMSNormCudaOp

    g = _g(4)
    gate = torch.randn(33, 1024, device=dev(), generator=g).bfloat16()
    up = torch.randn(33, 1024, device=dev(), generator=g).bfloat16()
    sw = SwiGLUCudaOp()
    want = torch.nn.functional.silu(gate.float()) * up.float()
    assert (sw(gate, up).float() - want).abs().max().item() < 0.05 and (sw.forward_fp32(gate, up) - want).abs().max().item() < 1e-4
    x = torch.randn(33, 4096, device=dev(), generator=g).bfloat16().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(4096, device=dev(), generator=g)).bfloat16().requires_grad_(True)
    rn = RMSNormCudaOp()
    y = rn(x, w, eps=1e-6)
    assert (y.float() - rn.forward_fp32(x.detach(), w.detach(), eps=1e-6)).abs().max().item() < 0.05
    y.sum().backward()
    contrib = rn.parameter_vjp_contributions_fp32(x=x.detach(), weight=w.detach(), grad_output=torch.ones_like(y))["weight"]
    assert (w.grad.float() - contrib.sum(0)).abs().max().item() < 0.5
    emb = SM90EmbeddingOp()
    table = torch.randn(1000, 256, device=dev(), generator=g).bfloat16().requires_grad_(True)
    ids = torch.randint(0, 1000, (4, 19), device=dev(), generator=g)
    e = emb(ids, table)
    assert torch.equal(e, table.detach()[ids])
    e.backward(torch.ones_like(e))
    cnt = torch.bincount(ids.reshape(-1), minlength=1000).float()
    assert torch.equal(table.grad.float()[:, 0], cnt)
    sync_and_check()
