"""Attention kernels on a B200: accuracy, decode == training bits, deterministic backward."""
import math

import pytest
import torch

from tests.gpu_util import dev, sync_and_check

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
HQ, HKV, D = 8, 2, 128
G = HQ // HKV
SCALE = 1.0 / math.sqrt(D)


def _inputs(B, S, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    T = B * S
    q = torch.randn(T, HQ * D, device=dev(), generator=g).to(BF)
    k = torch.randn(T, HKV * D, device=dev(), generator=g).to(BF)
    v = torch.randn(T, HKV * D, device=dev(), generator=g).to(BF)
    return q, k, v


def _gold(q, k, v, B, S):
    qf = q.float().view(B, S, HQ, D).transpose(1, 2)
    kf = k.float().view(B, S, HKV, D).transpose(1, 2).repeat_interleave(G, 1)
    vf = v.float().view(B, S, HKV, D).transpose(1, 2).repeat_interleave(G, 1)
    sc = (qf @ kf.transpose(-1, -2) * SCALE).masked_fill(
        ~torch.ones(S, S, device=q.device, dtype=torch.bool).tril(), float("-inf"))
    return sc, vf


@pytest.mark.parametrize("S", [128, 320, 1000])
def test_forward_and_decode_equivalence(S):
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.models.qwen3.engine import train_tiles

    B, T = 2, 2 * S
    q, k, v = _inputs(B, S)
    o = torch.zeros_like(q)
    lse = torch.zeros(T, HQ, device=dev())
    tiles, _ = train_tiles(B, S, HQ, HKV, D, dev())
    nv.attn_fwd(q, [k], [v], o, lse, tiles, SCALE)
    sync_and_check()
    sc, vf = _gold(q, k, v, B, S)
    ref = (sc.softmax(-1) @ vf).transpose(1, 2).reshape(T, HQ * D)
    assert (o.float() - ref).abs().max().item() < 0.03
    assert (lse - sc.logsumexp(-1).transpose(1, 2).reshape(T, HQ)).abs().max().item() < 1e-3
    # single-token decode of selected positions must reproduce the training rows bit for bit
    pos = [p for p in (0, 1, 127, 128, 129, S // 2, S - 1) if p < S]
    n = len(pos)
    qd = torch.zeros(n * HQ + 128, D, device=dev(), dtype=BF)
    qd[: n * HQ] = torch.stack([q.view(B, S, HQ, D)[1, p] for p in pos]).reshape(n * HQ, D)
    t2 = [[i * HQ + hk * G, 0, G, S, hk * D, p, 0, S, i * HQ + hk * G, 1, 0, 0] for i, p in enumerate(pos) for hk in range(HKV)]
    want_o = torch.stack([o.view(B, S, HQ, D)[1, p] for p in pos])
    want_l = torch.stack([lse.view(B, S, HQ)[1, p] for p in pos])
    for decode in (False, True):
        od, ld = torch.zeros_like(qd), torch.zeros(n * HQ + 128, device=dev())
        nv.attn_fwd(qd, [k], [v], od, ld, torch.tensor(t2, dtype=torch.int32, device=dev()), SCALE, decode=decode)
        sync_and_check()
        assert torch.equal(od[: n * HQ].view(n, HQ, D), want_o)
        assert torch.equal(ld[: n * HQ].view(n, HQ), want_l)


@pytest.mark.parametrize("S", [128, 320, 1000])
def test_backward(S):
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.models.qwen3.engine import train_tiles

    B, T = 2, 2 * S
    q, k, v = _inputs(B, S, 1)
    o, lse = torch.zeros_like(q), torch.zeros(T, HQ, device=dev())
    tiles, kvt = train_tiles(B, S, HQ, HKV, D, dev())
    nv.attn_fwd(q, [k], [v], o, lse, tiles, SCALE)
    do = torch.randn(T, HQ * D, device=dev()).to(BF)
    delta = torch.empty(T, HQ, device=dev())
    grads = []
    for _ in range(2):
        dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
        nv.attn_bwd_delta(o, do, delta, T, HQ)
        nv.attn_bwd_dq(q, do, k, v, lse, delta, dq, tiles, SCALE)
        nv.attn_bwd_dkv(q, do, k, v, lse, delta, dk, dv, kvt, SCALE)
        sync_and_check()
        grads.append((dq, dk, dv))
    for a, b in zip(*grads):
        assert torch.equal(a, b), "backward is not run-to-run deterministic"
    qf = q.float().view(B, S, HQ, D).transpose(1, 2).requires_grad_(True)
    k0 = k.float().view(B, S, HKV, D).transpose(1, 2).requires_grad_(True)
    v0 = v.float().view(B, S, HKV, D).transpose(1, 2).requires_grad_(True)
    sc = (qf @ k0.repeat_interleave(G, 1).transpose(-1, -2) * SCALE).masked_fill(
        ~torch.ones(S, S, device=dev(), dtype=torch.bool).tril(), float("-inf"))
    (sc.softmax(-1) @ v0.repeat_interleave(G, 1)).backward(do.float().view(B, S, HQ, D).transpose(1, 2))
    for got, want in zip(grads[0], (qf.grad, k0.grad, v0.grad)):
        w = want.transpose(1, 2).reshape(got.shape)
        assert (got.float() - w).abs().max().item() < 0.02 * w.abs().max().item() + 0.02


def test_paged_attention_equals_contiguous_bitwise():
    """Decode and chunked prefill through a fragmented page pool give the bits of contiguous KV."""
    from rl_kernel_b200.ops.attention import PagedKVCache, causal_attention, paged_attention

    hq, hkv, d = 8, 2, 128
    lens = [300, 129, 517]
    cache = PagedKVCache(16, hkv, d, dev())
    cache.free = torch.randperm(16, generator=torch.Generator().manual_seed(1)).tolist()   # scrambled pool
    ks, vs, qs = [], [], []
    g = torch.Generator(device="cuda").manual_seed(5)
    for s, n in enumerate(lens):
        ks.append(torch.randn(n, hkv, d, device=dev(), generator=g).to(BF))
        vs.append(torch.randn(n, hkv, d, device=dev(), generator=g).to(BF))
        qs.append(torch.randn(n, hq, d, device=dev(), generator=g).to(BF))
    # interleave the allocations so that every sequence's pages are scattered over the pool
    for upto in (100, 260, 600):
        for s, n in enumerate(lens):
            m = min(n, upto)
            old = cache.lengths.get(s, 0)
            if m > old:
                cache.reserve(s, m)
                cache.write(s, torch.arange(old, m), ks[s][old:m].reshape(m - old, -1), vs[s][old:m].reshape(m - old, -1))
    assert cache.tables[2] != sorted(cache.tables[2]), "the test wants out-of-order pages"
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    ref, ref_lse = causal_attention(torch.cat(qs), torch.cat(ks), torch.cat(vs), cu, return_lse=True)
    # decode: the last token of every sequence
    q_last = torch.stack([q[-1] for q in qs])
    out = paged_attention(q_last, cache, [0, 1, 2], [torch.tensor([n - 1]) for n in lens])
    sync_and_check()
    for s in range(3):
        assert torch.equal(out[s], ref[cu[s + 1] - 1])
    # chunked prefill: the second half of every sequence as one query chunk each
    halves = [n // 2 for n in lens]
    q_chunk = torch.cat([q[h:] for q, h in zip(qs, halves)])
    out2, lse2 = paged_attention(q_chunk, cache, [0, 1, 2], [torch.arange(h, n) for h, n in zip(halves, lens)],
                                 return_lse=True)
    sync_and_check()
    t0 = 0
    for s, (h, n) in enumerate(zip(halves, lens)):
        assert torch.equal(out2[t0:t0 + n - h], ref[cu[s] + h:cu[s + 1]])
        assert torch.equal(lse2[t0:t0 + n - h], ref_lse[cu[s] + h:cu[s + 1]])
        t0 += n - h


def test_prefix_shared_attention_matches_per_sample_attention():
    from rl_kernel_b200.ops.attention import prefix_shared_attention

    bs, G, Lq, hq, hkv, d, Lkv = 2, 8, 24, 8, 2, 128, 300
    g = torch.Generator(device="cuda").manual_seed(8)
    q = torch.randn(bs, G, Lq, hq, d, device=dev(), generator=g).to(BF)
    k = torch.randn(bs, Lkv, hkv, d, device=dev(), generator=g).to(BF)
    v = torch.randn(bs, Lkv, hkv, d, device=dev(), generator=g).to(BF)
    out, lse = prefix_shared_attention(q, k, v, return_lse=True)
    sync_and_check()
    ref, rl = prefix_shared_attention(q.cpu(), k.cpu(), v.cpu(), return_lse=True)
    assert (out.float().cpu() - ref.float()).abs().max().item() < 0.02
    assert (lse.cpu() - rl).abs().max().item() < 1e-2
    # packing the samples into shared tiles does not change a row: one sample alone gives the same bits
    one = prefix_shared_attention(q[:, 3:4].contiguous(), k, v)
    sync_and_check()
    assert torch.equal(one[:, 0], out[:, 3])


@pytest.mark.parametrize("cp,layout", [(4, "zigzag"), (8, "zigzag"), (4, "contiguous")])
def test_context_parallel_kernels_with_emulated_ranks(cp, layout):
    """The CP kernels never wait on a peer inside a launch, so the ranks of a CP group can be run one
    after the other on a single GPU with every rank's buffers resident: forward, dQ and dK/dV of all
    4 or 8 ranks -- with the remote blocks staged by the kernels -- must reproduce the single-GPU
    tensors bit for bit."""
    import math

    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.distributed.cp_attention import cp_positions, cp_tiles
    from rl_kernel_b200.models.qwen3.engine import train_tiles

    hq, hkv, d, B, S = 8, 2, 128, 2, 2048
    g = torch.Generator(device="cuda").manual_seed(13)
    mk = lambda h: torch.randn(B, S, h * d, device=dev(), generator=g).to(BF)  # noqa: E731
    q, k, v, do = mk(hq), mk(hkv), mk(hkv), mk(hq)
    sc = 1 / math.sqrt(d)
    T = B * S
    o1, l1, dl1 = torch.empty(T, hq * d, device=dev(), dtype=BF), torch.empty(T, hq, device=dev()), torch.empty(T, hq, device=dev())
    tiles, kvt = train_tiles(B, S, hq, hkv, d, dev())
    q2, k2, v2, do2 = (t.view(T, -1) for t in (q, k, v, do))
    nv.attn_fwd(q2, [k2], [v2], o1, l1, tiles, sc)
    nv.attn_bwd_delta(o1, do2, dl1, T, hq)
    dq1, dk1, dv1 = torch.empty_like(q2), torch.empty_like(k2), torch.empty_like(v2)
    nv.attn_bwd_dq(q2, do2, k2, v2, l1, dl1, dq1, tiles, sc)
    nv.attn_bwd_dkv(q2, do2, k2, v2, l1, dl1, dk1, dv1, kvt, sc)
    # every rank's local tensors (what its peers would have mapped)
    pos = [cp_positions(S, cp, r, layout).to(dev()) for r in range(cp)]
    sel = lambda t, r: t[:, pos[r]].reshape(B * pos[r].numel(), -1).contiguous()  # noqa: E731
    ql, kl, vl, dol = ([sel(t, r) for r in range(cp)] for t in (q, k, v, do))
    Tl = ql[0].shape[0]
    zz = layout == "zigzag"
    outs, lses, deltas = [], [], []
    st = lambda cols: torch.zeros(cp * Tl, cols, device=dev(), dtype=BF)  # noqa: E731
    for r in range(cp):
        fw, _, bpc = cp_tiles(cp, r, layout, B, S, hq, hkv, d, dev())
        o, l = torch.empty_like(ql[r]), torch.empty(Tl, hq, device=dev())
        flags = torch.zeros(cp * (Tl // 128) * 2 + 1, dtype=torch.int32, device=dev())
        nv.attn_fwd(ql[r], kl, vl, o, l, fw, sc, cp_blocks_per_chunk=bpc, cp_zigzag=zz,
                    stage=(st(hkv * d), st(hkv * d), flags, Tl, r))
        dl = torch.empty(Tl, hq, device=dev())
        nv.attn_bwd_delta(o, dol[r], dl, Tl, hq)
        outs.append(o); lses.append(l); deltas.append(dl)
        assert torch.equal(o, sel(o1.view(B, S, -1), r)) and torch.equal(l, sel(l1.view(B, S, -1), r))
    for r in range(cp):
        fw, kvl, bpc = cp_tiles(cp, r, layout, B, S, hq, hkv, d, dev())
        dq, dk, dv = torch.empty_like(ql[r]), torch.empty_like(kl[r]), torch.empty_like(vl[r])
        f1 = torch.zeros(cp * (Tl // 128) * 2 + 1, dtype=torch.int32, device=dev())
        f2 = torch.zeros_like(f1)
        nv.attn_bwd_dq(ql[r], dol[r], kl, vl, lses[r], deltas[r], dq, fw, sc, cp_blocks_per_chunk=bpc, cp_zigzag=zz,
                       stage=(st(hkv * d), st(hkv * d), f1, Tl, r))
        nv.attn_bwd_dkv(ql, dol, kl[r], vl[r], lses, deltas, dk, dv, kvl, sc, cp_blocks_per_chunk=bpc, cp_zigzag=zz,
                        stage=(st(hq * d), st(hq * d), f2, Tl, r))
        sync_and_check()
        assert torch.equal(dq, sel(dq1.view(B, S, -1), r)), ("dq", r)
        assert torch.equal(dk, sel(dk1.view(B, S, -1), r)), ("dk", r)
        assert torch.equal(dv, sel(dv1.view(B, S, -1), r)), ("dv", r)
