"""Row-wise and element-wise sm_100a kernels against fp32 PyTorch references."""
import pytest
import torch

from tests.gpu_util import dev, sync_and_check

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _rms(x, w, eps=1e-6):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def test_rmsnorm_forward_backward():
    from rl_kernel_b200.backends import native as nv

    rows, H = 300, 4096
    x = torch.randn(rows, H, device=dev()).to(BF)
    w = (1 + 0.1 * torch.randn(H, device=dev())).to(BF)
    res = torch.randn(rows, H, device=dev()).to(BF)
    y = torch.empty_like(x)
    nv.rmsnorm_fwd(x, w, y, 1e-6)
    sync_and_check()
    assert (y.float() - _rms(x.float(), w.float())).abs().max().item() < 0.03
    y1 = torch.empty(7, H, device=dev(), dtype=BF)
    nv.rmsnorm_fwd(x[:7].contiguous(), w, y1, 1e-6)
    assert torch.equal(y1, y[:7]), "rmsnorm must be batch-invariant"
    y2, ro = torch.empty_like(x), torch.empty_like(x)
    nv.rmsnorm_fwd(x, w, y2, 1e-6, res=res, res_out=ro)
    s = (x.float() + res.float()).to(BF)
    assert torch.equal(ro, s)
    assert (y2.float() - _rms(s.float(), w.float())).abs().max().item() < 0.03
    for Hh in (256, 1024, 16384):   # few and many chunks per thread
        xx = torch.randn(5, Hh, device=dev()).to(BF)
        ww = torch.ones(Hh, device=dev(), dtype=BF)
        yy = torch.empty_like(xx)
        nv.rmsnorm_fwd(xx, ww, yy, 1e-6)
        assert (yy.float() - _rms(xx.float(), ww.float())).abs().max().item() < 0.03
    dy = torch.randn(rows, H, device=dev()).to(BF)
    dres = torch.randn(rows, H, device=dev()).to(BF)
    dx, dw = torch.empty_like(x), torch.zeros(H, device=dev(), dtype=BF)
    scratch = torch.empty(nv.rmsnorm_bwd_scratch_elems(rows, H), device=dev())
    nv.rmsnorm_bwd(x, w, dy, dx, scratch, 1e-6, dres=dres, dw_bf16=dw)
    sync_and_check()
    xf, wf = x.float().requires_grad_(True), w.float().requires_grad_(True)
    _rms(xf, wf).backward(dy.float())
    assert (dx.float() - (xf.grad + dres.float())).abs().max().item() < 0.05
    assert (dw.float() - wf.grad).abs().max().item() < 0.01 * wf.grad.abs().max().item() + 0.05


def _tables(D=128, theta=1e6, n=4096):
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, device=dev()).double() / D))
    ang = torch.arange(n, device=dev()).double()[:, None] * inv[None]
    return ang.cos().float().contiguous(), ang.sin().float().contiguous()


def test_qk_norm_rope_forward_backward():
    from rl_kernel_b200.backends import native as nv

    T, Hq, Hkv, D = 200, 8, 2, 128
    G = Hq // Hkv
    W = (Hq + 2 * Hkv) * D
    qkv = torch.randn(T, W, device=dev()).to(BF)
    qw = (1 + 0.1 * torch.randn(D, device=dev())).to(BF)
    kw = (1 + 0.1 * torch.randn(D, device=dev())).to(BF)
    pos = (torch.arange(T, device=dev(), dtype=torch.int32) * 3) % 77
    cos, sin = _tables()
    qo = torch.empty(T, Hq * D, device=dev(), dtype=BF)
    ko = torch.empty(T, Hkv * D, device=dev(), dtype=BF)
    vo = torch.empty(T, Hkv * D, device=dev(), dtype=BF)
    nv.qk_norm_rope_fwd(qkv, qw, kw, cos, sin, pos, qo, ko, vo, Hq=Hq, Hkv=Hkv, eps=1e-6)
    sync_and_check()
    # the activation is GQA-group-major: [G q heads | k | v] per KV head
    grp = qkv.view(T, Hkv, G + 2, D)
    qf, kf, vf = grp[:, :, :G].reshape(T, Hq, D).float(), grp[:, :, G].float(), grp[:, :, G + 1]

    def ref(x, w):
        n = _rms(x, w)
        c, s = cos[pos.long()][:, None], sin[pos.long()][:, None]
        a, b = n[..., :64], n[..., 64:]
        return torch.cat([a * c - b * s, b * c + a * s], -1)

    assert (qo.float().view(T, Hq, D) - ref(qf, qw.float())).abs().max().item() < 0.03
    assert (ko.float().view(T, Hkv, D) - ref(kf, kw.float())).abs().max().item() < 0.03
    assert torch.equal(vo.view(T, Hkv, D), vf)
    dq = torch.randn(T, Hq * D, device=dev()).to(BF)
    dk = torch.randn(T, Hkv * D, device=dev()).to(BF)
    dv = torch.randn(T, Hkv * D, device=dev()).to(BF)
    dqkv = torch.empty_like(qkv)
    dqw, dkw = torch.zeros(D, device=dev(), dtype=BF), torch.zeros(D, device=dev(), dtype=BF)
    scr = torch.empty(nv.qk_norm_rope_bwd_scratch_elems(T), device=dev())
    nv.qk_norm_rope_bwd(qkv, qw, kw, cos, sin, pos, dq, dk, dv, dqkv, scr, dqw, dkw, Hq=Hq, Hkv=Hkv, eps=1e-6,
                        accumulate_dw=False)
    sync_and_check()
    q2, k2 = qf.clone().requires_grad_(True), kf.clone().requires_grad_(True)
    qwf, kwf = qw.float().requires_grad_(True), kw.float().requires_grad_(True)
    (ref(q2, qwf) * dq.float().view(T, Hq, D)).sum().backward()
    (ref(k2, kwf) * dk.float().view(T, Hkv, D)).sum().backward()
    dg = dqkv.view(T, Hkv, G + 2, D)
    assert (dg[:, :, :G].reshape(T, Hq, D).float() - q2.grad).abs().max().item() < 0.05
    assert (dg[:, :, G].float() - k2.grad).abs().max().item() < 0.05
    assert torch.equal(dg[:, :, G + 1].reshape(T, Hkv * D), dv)
    assert (dqw.float() - qwf.grad).abs().max().item() < 0.01 * qwf.grad.abs().max().item() + 0.05
    assert (dkw.float() - kwf.grad).abs().max().item() < 0.01 * kwf.grad.abs().max().item() + 0.05


@pytest.mark.parametrize("rows,I,blk", [(100, 1536, None), (100, 1536, 192), (37, 4096, 512), (101, 256, None),
                                        (300, 12288, 1536), (5, 40, 8)])
def test_swiglu(rows, I, blk):
    """Row widths on both sides of the 256-piece boundary of the launch grid, rows that do not fill a block."""
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.reference.activation.swiglu import swiglu_packed_reference

    gu = torch.randn(rows, 2 * I, device=dev()).to(BF)
    out = torch.empty(rows, I, device=dev(), dtype=BF)
    nv.swiglu_fwd(gu, out, I, blk)
    sync_and_check()
    assert (out.float() - swiglu_packed_reference(gu.float(), blk)).abs().max().item() < 0.05
    dout = torch.randn(rows, I, device=dev()).to(BF)
    dgu = torch.empty_like(gu)
    nv.swiglu_bwd(gu, dout, dgu, I, blk)
    sync_and_check()
    g = gu.float().requires_grad_(True)
    swiglu_packed_reference(g, blk).backward(dout.float())
    assert (dgu.float() - g.grad).abs().max().item() < 0.05


@pytest.mark.parametrize("heads,D,dtype", [(32, 128, BF), (8, 128, BF), (1, 128, BF), (3, 64, torch.float32),
                                           (2, 20, BF), (5, 24, torch.float32), (40, 128, BF)])
def test_rope_standalone_matches_fp32_expression_bitwise(heads, D, dtype):
    """Vector path (half head a multiple of 16 bytes) and scalar path, in place and out of place, strided rows,
    forward and inverse: the bits of a*c - b*s / b*c + a*s in fp32 with one rounding."""
    from rl_kernel_b200.backends import native as nv

    g = torch.Generator(device="cuda").manual_seed(heads * 1000 + D)
    rows, max_pos, half = 333, 700, D // 2
    ang = torch.rand(max_pos, half, device=dev(), generator=g) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    pos = torch.randint(0, max_pos, (rows,), device=dev(), generator=g).to(torch.int32)
    wide = torch.randn(rows, heads * D + 16, device=dev(), generator=g).to(dtype)
    x = wide[:, :heads * D]                                   # row stride larger than the row
    xf = x.float().view(rows, heads, D)
    c, s_ = cos[pos.long()][:, None, :], sin[pos.long()][:, None, :]
    a, b = xf[..., :half], xf[..., half:]
    for inverse in (False, True):
        sg = -s_ if inverse else s_
        want = torch.cat([a * c - b * sg, b * c + a * sg], dim=-1).reshape(rows, heads * D).to(dtype)
        out = torch.empty(rows, heads * D, device=dev(), dtype=dtype)
        nv.rope(x, pos, cos, sin, out, heads=heads, head_dim=D, inverse=inverse)
        sync_and_check()
        assert torch.equal(out, want)
        inplace = wide.clone()[:, :heads * D]
        nv.rope(inplace, pos, cos, sin, inplace, heads=heads, head_dim=D, inverse=inverse)
        sync_and_check()
        assert torch.equal(inplace, want)


def test_rope_op_head_major_view_is_rotated_without_a_copy_and_split_swiglu_matches_packed():
    from rl_kernel_b200.ops.activation import swiglu, swiglu_packed
    from rl_kernel_b200.ops.rope import rope

    g = torch.Generator(device="cuda").manual_seed(11)
    S, H, D = 77, 6, 128
    store = torch.randn(2, S, H, D, device=dev(), generator=g).to(BF)
    pos = torch.stack([torch.arange(S), torch.arange(9, 9 + S)]).to(dev())
    for xs, ps in ((store[0], pos[0]), (store, pos), (store, pos[1])):
        xv = xs.transpose(-3, -2).requires_grad_(True)                    # [.., H, S, D] over token-major storage
        y = rope(xv, ps, max_position=4096)
        sync_and_check()
        xc = xs.transpose(-3, -2).contiguous().requires_grad_(True)
        yc = rope(xc, ps)
        assert y.shape == xv.shape and y.stride() == xv.stride() and torch.equal(y, yc)
        gy = torch.randn(y.shape, device=dev(), generator=g).to(BF)
        y.backward(gy)
        yc.backward(gy)
        assert torch.equal(xv.grad, xc.grad)
    rows, I = 130, 1024
    wide = torch.randn(rows, 2 * I + 8, device=dev(), generator=g).to(BF)
    gate, up = wide[:, :I].detach().requires_grad_(True), wide[:, I:2 * I].detach().requires_grad_(True)   # strided rows
    out = swiglu(gate, up)
    sync_and_check()
    gu = torch.cat([gate.detach(), up.detach()], -1).requires_grad_(True)
    want = swiglu_packed(gu)
    assert torch.equal(out, want)
    go = torch.randn(rows, I, device=dev(), generator=g).to(BF)
    out.backward(go)
    want.backward(go)
    assert torch.equal(gate.grad, gu.grad[:, :I]) and torch.equal(up.grad, gu.grad[:, I:])
    assert torch.equal(swiglu(gate.detach().view(10, 13, I), up.detach().view(10, 13, I)), want.detach().view(10, 13, I))


def test_embedding():
    from rl_kernel_b200.backends import native as nv

    V, H, T = 1000, 256, 500
    ids = torch.randint(0, V, (T,), device=dev())
    w = torch.randn(V, H, device=dev()).to(BF)
    out = torch.empty(T, H, device=dev(), dtype=BF)
    nv.embedding_fwd(ids, w, out)
    assert torch.equal(out, w[ids])
    half = torch.empty_like(out)
    nv.embedding_fwd(ids, w[500:].contiguous(), half, vocab_start=500)   # vocab-parallel shard
    assert torch.equal(half, w[ids] * (ids >= 500)[:, None])
    dy = torch.randn(T, H, device=dev()).to(BF)
    runs = []
    for _ in range(2):
        dw = torch.zeros(V, H, device=dev(), dtype=BF)
        sid, order = torch.sort(ids, stable=True)
        nv.embedding_bwd(sid, order, dy, dw)
        sync_and_check()
        runs.append(dw)
    assert torch.equal(runs[0], runs[1])
    ref = torch.zeros(V, H, device=dev()).index_add_(0, ids, dy.float())
    assert (runs[0].float() - ref).abs().max().item() < 0.05


@pytest.mark.parametrize("temp", [1.0, 0.7])
def test_logp_fused_equals_from_logits_and_vocab_parallel(temp):
    from rl_kernel_b200.backends import native as nv

    T, H, V = 333, 512, 5000
    h = torch.randn(T, H, device=dev()).to(BF)
    w = (torch.randn(V, H, device=dev()) * 0.05).to(BF)
    tg = torch.randint(0, V, (T,), device=dev())
    nt = (V + 127) // 128

    def fused(hh, tt, shards):
        n = hh.shape[0]
        stats = torch.zeros(n, nt, 2, device=dev())
        tl = torch.zeros(n, device=dev())
        for start, ws in shards:
            nv.lmhead_logp_stats(hh, ws, tt, stats, tl, vocab_start=start, inv_temp=1 / temp)
        lp, lse = torch.empty(n, device=dev()), torch.empty(n, device=dev())
        nv.logp_merge(stats, tl, lp, lse)
        sync_and_check()
        return lp, lse

    lp, lse = fused(h, tg, [(0, w)])
    logits = torch.empty(T, V, device=dev(), dtype=BF)
    nv.det_gemm(h, w, logits, M=T, N=V, K=H)
    stats2, tl2 = torch.zeros(T, nt, 2, device=dev()), torch.zeros(T, device=dev())
    nv.logits_tile_stats(logits, tg, stats2, tl2, vocab_start=0, inv_temp=1 / temp)
    lp2, lse2 = torch.empty(T, device=dev()), torch.empty(T, device=dev())
    nv.logp_merge(stats2, tl2, lp2, lse2)
    sync_and_check()
    assert torch.equal(lp, lp2) and torch.equal(lse, lse2), "fused LM head and from-logits paths differ"
    ref = torch.log_softmax(logits.float() / temp, -1).gather(1, tg[:, None])[:, 0]
    assert (lp - ref).abs().max().item() < 1e-4
    assert torch.equal(fused(h[:3].contiguous(), tg[:3].contiguous(), [(0, w)])[0], lp[:3])
    assert torch.equal(fused(h, tg, [(0, w[:2560].contiguous()), (2560, w[2560:].contiguous())])[0], lp)
    # gradient of the logits
    g = torch.randn(T, device=dev())
    lc = logits.clone()
    nv.dlogits_(lc, tg, lse2, g, vocab_start=0, inv_temp=1 / temp)
    sync_and_check()
    z = (logits.float() / temp).requires_grad_(True)
    (torch.log_softmax(z, -1).gather(1, tg[:, None])[:, 0] * g).sum().backward()
    assert (lc.float() - z.grad / temp).abs().max().item() < 0.02


def test_logp_from_logits_wide_vocabulary_strided_rows_and_row_subsets():
    """More than 128 vocabulary tiles (several tile groups per row), a ragged last tile, a row pitch wider than
    the vocabulary: matches log_softmax and does not depend on which rows share the launch."""
    from rl_kernel_b200.ops.logprob import logp_from_logits, logp_from_logits_indexed

    g = torch.Generator(device="cuda").manual_seed(5)
    T, V = 37, 20008
    wide = (torch.randn(T, V + 24, device=dev(), generator=g) * 3).to(BF)
    logits = wide[:, :V]
    tg = torch.randint(0, V, (T,), device=dev(), generator=g)
    tg[0], tg[1] = V - 1, 0
    lp = logp_from_logits(logits, tg, 0.7)
    sync_and_check()
    ref = torch.log_softmax(logits.float() / 0.7, -1).gather(1, tg[:, None])[:, 0]
    assert (lp - ref).abs().max().item() < 2e-4
    assert torch.equal(logp_from_logits(logits[5:6], tg[5:6], 0.7), lp[5:6])
    assert torch.equal(logp_from_logits(logits.contiguous(), tg, 0.7), lp)
    idx = torch.tensor([36, 0, 17], device=dev())
    assert torch.equal(logp_from_logits_indexed(logits.contiguous(), tg[idx], idx, temperature=0.7), lp[idx])


def test_grpo_loss_and_advantages():
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.reference.loss import grpo_loss_from_logps

    B, L = 16, 100
    lp = -torch.rand(B, L, device=dev())
    old = lp + 0.3 * torch.randn(B, L, device=dev())
    refl = lp + 0.1 * torch.randn(B, L, device=dev())
    adv = torch.randn(B, device=dev())
    mask = torch.rand(B, L, device=dev()) > 0.3
    cnt = int(mask.sum())
    r = nv.grpo_loss(lp, old, refl, adv, mask.to(torch.uint8), clip_lo=0.2, clip_hi=0.2, beta=0.01, inv_norm=1.0 / cnt)
    sync_and_check()
    lpr = lp.clone().requires_grad_(True)
    loss, pol, kl = grpo_loss_from_logps(lpr, old, refl, adv, mask, clip_eps=0.2, beta=0.01)
    loss.backward()
    assert abs(r["totals"][4].item() - loss.item()) < 1e-5
    assert (r["dlogp"] - lpr.grad).abs().max().item() < 1e-6
    rw = torch.rand(4, 8, device=dev())
    a = nv.group_advantages(rw.view(-1).contiguous(), 4, 8, 1e-6).view(4, 8)
    assert (a - (rw - rw.mean(1, keepdim=True)) / rw.std(1, unbiased=False, keepdim=True)).abs().max().item() < 1e-5


def test_sampling():
    from rl_kernel_b200.backends import native as nv

    rows, V = 64, 151936
    lg = (torch.randn(rows, V, device=dev()) * 2).to(BF)
    ids, val = torch.empty(rows, device=dev(), dtype=torch.int64), torch.empty(rows, device=dev())
    nv.sample_gumbel(lg, ids, val, vocab_start=0, inv_temp=1.0, seed=1, step=0, greedy=True)
    sync_and_check()
    assert torch.equal(ids, lg.float().argmax(-1))
    # the draw does not depend on how the vocabulary is sharded
    ia, va = torch.empty_like(ids), torch.empty_like(val)
    nv.sample_gumbel(lg, ia, va, vocab_start=0, inv_temp=1.0, seed=5, step=9)
    hv = V // 2
    i1, v1, i2, v2 = torch.empty_like(ids), torch.empty_like(val), torch.empty_like(ids), torch.empty_like(val)
    nv.sample_gumbel(lg[:, :hv], i1, v1, vocab_start=0, inv_temp=1.0, seed=5, step=9)
    nv.sample_gumbel(lg[:, hv:], i2, v2, vocab_start=hv, inv_temp=1.0, seed=5, step=9)
    sync_and_check()
    assert torch.equal(torch.where(v1 >= v2, i1, i2), ia)
    small = torch.tensor([[2.0, 1.0, 0.0, -1.0, -2, -3, -4, -5]], device=dev()).to(BF).repeat(8192, 1).contiguous()
    oi = torch.empty(8192, device=dev(), dtype=torch.int64)
    nv.sample_gumbel(small, oi, None, vocab_start=0, inv_temp=1.0, seed=7, step=3)
    sync_and_check()
    freq = torch.bincount(oi, minlength=8).float() / 8192
    assert (freq - torch.softmax(small[0].float(), -1)).abs().max().item() < 0.03


def test_adamw_and_exact_sumsq():
    from rl_kernel_b200.backends import native as nv

    n = 100003
    master = torch.randn(n, device=dev())
    m, v = torch.zeros(n, device=dev()), torch.zeros(n, device=dev())
    g = torch.randn(n, device=dev()).to(BF)
    pb = master.to(BF)
    pr = torch.nn.Parameter(master.clone())
    opt = torch.optim.AdamW([pr], lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for st in (1, 2):
        nv.adamw(master, m, v, g, pb, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=st)
        pr.grad = g.float()
        opt.step()
    sync_and_check()
    assert (master - pr.data).abs().max().item() < 1e-5
    assert torch.equal(pb, master.to(BF))
    e = torch.arange(256, device=dev()).clamp(min=1).double()
    wts = torch.pow(2.0, 2 * (e - 134))
    wts[255] = 0

    def ss(parts):
        bins = torch.zeros(256, device=dev(), dtype=torch.int64)
        for p in parts:
            nv.sumsq_bins(p, bins)
        sync_and_check()
        return (bins.double() * wts).sum().item()

    whole = ss([g])
    assert whole == ss([g[:1000], g[1000:50000], g[50000:]]), "sum of squares must not depend on the partition"
    assert whole == ss([g[:1001], g[1001:50003], g[50003:]]), "nor on the alignment of the pieces"
    assert abs(whole - g.double().pow(2).sum().item()) < 1e-6 * whole


def test_top_k_top_p_threshold_matches_sorted_policy():
    """The histogram threshold keeps the ids of the sort-based policy (value groups are kept whole);
    ids whose preceding mass is within 1e-5 of top_p may fall on either side."""
    from rl_kernel_b200.backends import native as nv

    rows, V = 12, 20000
    logits = (torch.randn(rows, V, device=dev()) * 3).to(BF)
    for temperature, top_k, top_p in ((1.0, 50, 1.0), (0.7, 0, 0.9), (1.3, 200, 0.95), (1.0, 1, 0.5)):
        thr = torch.empty(rows, device=dev())
        nv.sample_keep_threshold(logits, thr, inv_temp=1.0 / temperature, top_k=top_k, top_p=top_p)
        sync_and_check()
        z32 = logits.float() * (1.0 / temperature)
        mine = z32 >= thr[:, None]
        z = z32.double()
        keep = torch.ones_like(mine)
        fuzzy = torch.zeros_like(mine)
        if top_k:
            kth = torch.topk(z, top_k, dim=-1).values[:, -1:]
            keep &= z >= kth
        if top_p < 1.0:
            p = torch.softmax(z, -1)
            # mass strictly above each id's value
            zs, idx = torch.sort(z, dim=-1, descending=True)
            ps = torch.gather(p, 1, idx)
            cum_before = ps.cumsum(-1) - ps
            first = torch.ones_like(zs, dtype=torch.bool)
            first[:, 1:] = zs[:, 1:] != zs[:, :-1]
            grp_before = torch.where(first, cum_before, torch.zeros_like(cum_before)).cummax(-1).values
            above = torch.zeros_like(p).scatter(1, idx, grp_before)
            keep &= (above < top_p) | (above == 0)
            fuzzy |= (above - top_p).abs() < 1e-5
        assert torch.all((mine == keep) | fuzzy), (temperature, top_k, top_p)
        assert torch.all(mine.any(-1))


def test_indexed_logp_and_lse_gradient():
    from rl_kernel_b200.ops.logprob import logp_from_logits, logp_from_logits_indexed

    R, V = 40, 4096
    logits = torch.randn(R, V, device=dev()).to(BF).requires_grad_(True)
    idx = torch.tensor([3, 17, 17, 39, 0], device=dev())
    tgt = torch.randint(0, V, (5,), device=dev())
    lp, lse = logp_from_logits_indexed(logits, tgt, idx, temperature=0.8, return_lse=True)
    full = logp_from_logits(logits.detach(), torch.zeros(R, dtype=torch.long, device=dev()), 0.8)
    dense = logp_from_logits(logits.detach()[idx], tgt, 0.8)
    assert torch.equal(lp.detach(), dense), "indexed scoring must equal scoring the gathered rows"
    assert full.shape == (R,)
    g1, g2 = torch.randn(5, device=dev()), torch.randn(5, device=dev())
    (lp * g1).sum().add((lse * g2).sum()).backward()
    ref = logits.detach().float().requires_grad_(True)
    z = ref[idx] / 0.8
    rl = torch.log_softmax(z, -1).gather(1, tgt[:, None])[:, 0]
    ((rl * g1).sum() + (torch.logsumexp(z, -1) * g2).sum()).backward()
    sync_and_check()
    assert (lse.detach() - torch.logsumexp(z, -1).detach()).abs().max().item() < 1e-3
    assert (logits.grad.float() - ref.grad).abs().max().item() < 0.02


def test_exact_fp32_sum_of_squares_matches_cpu_bins():
    from rl_kernel_b200.ops.norm.reproducible import norm_from_bins_f32, sumsq_bins_f32

    x = torch.randn(300001, device=dev()) * 5
    x[7], x[8] = 1e-41, 0.0
    gpu = sumsq_bins_f32([x[:1000], x[1000:170001], x[170001:]])
    sync_and_check()
    cpu = sumsq_bins_f32([x.cpu()])
    assert torch.equal(gpu.cpu(), cpu), "integer bins must be exact and independent of the partition"
    ref = x.double().pow(2).sum().sqrt().item()
    assert abs(norm_from_bins_f32(gpu).item() - ref) <= 1e-12 * ref


@pytest.mark.parametrize("world", [4, 8])
def test_collective_kernels_for_4_and_8_ranks_emulated_on_one_gpu(world):
    """The 4- and 8-rank instantiations of the collective kernels, run as one cooperative kernel over
    all ranks' windows on a single GPU, against the balanced tree computed with torch."""
    import ctypes

    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.distributed import balanced_tree_sum

    lib = ext.load()
    n = 8 * world * 1031 * 4                       # elements: multiple of 8 * world, not of the slice size
    for dtype, code in ((torch.bfloat16, 0), (torch.float32, 1)):
        parts = [torch.randn(n, device=dev()).to(dtype) for _ in range(world)]
        want = balanced_tree_sum(parts, dtype)
        nbytes = n * parts[0].element_size()
        for mode in (0, 1, 2, 3):
            size = {0: n, 1: n, 2: n // world, 3: n * world}[mode]
            outs = [torch.zeros(size, device=dev(), dtype=dtype) for _ in range(world)]
            srcs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in parts])
            dsts = (ctypes.c_void_p * world)(*[t.data_ptr() for t in outs])
            ext.check(lib.rlk_symm_emulate(ctypes.c_int(world), ctypes.c_int(mode), ctypes.c_longlong(nbytes),
                                           ctypes.c_int(code), srcs, dsts, ext.stream_ptr(dev())), "symm_emulate")
            sync_and_check()
            for r in range(world):
                if mode in (0, 1):
                    assert torch.equal(outs[r], want), (world, dtype, mode, r)
                elif mode == 2:
                    assert torch.equal(outs[r], want[r * size:(r + 1) * size]), (world, dtype, mode, r)
                else:
                    assert torch.equal(outs[r], torch.cat(parts)), (world, dtype, mode, r)


def test_pack_unpack_kernel_matches_boolean_indexing():
    from rl_kernel_b200.ops.packing import PackOp
    from rl_kernel_b200.reference.packing.pack import NativePackOp

    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.randn(5, 37, 256, device=dev(), generator=g).bfloat16()
    lengths = torch.tensor([37, 0, 5, 36, 1], device=dev())
    mask = torch.arange(37, device=dev())[None, :] < lengths[:, None]
    op, ref = PackOp(), NativePackOp()
    packed, cu = op.pack(x, mask)
    sync_and_check()
    rp, rcu = ref.pack(x, mask)
    assert torch.equal(packed, rp) and torch.equal(cu, rcu)
    back = op.unpack(packed, mask, fill=-1.0)
    sync_and_check()
    assert torch.equal(back, ref.unpack(rp, mask, fill=-1.0))
    # a left-padded mask packs in the same row-major order
    mask2 = mask.flip(1)
    p2, _ = op.pack(x, mask2)
    assert torch.equal(p2, x[mask2])


def test_registry_hands_out_native_ops_for_the_fused_operator_names():
    """On a B200 every operator name that has an sm_100a implementation resolves to it, including
    the multi-GPU ones (cp_attention needs its collective, so without one the reference is built)."""
    from rl_kernel_b200.runtime.registry import OpBackend, kernel_registry

    for name, want in (("ratio_kl", OpBackend.B200_RATIO_KL), ("distributed_grpo_loss", OpBackend.B200_DIST_GRPO_LOSS),
                       ("vocab_parallel_logp", OpBackend.B200_VOCAB_PARALLEL_LOGP), ("pack", OpBackend.B200_PACK),
                       ("cp_attention", OpBackend.B200_CP_ATTENTION)):
        res = kernel_registry.resolve(name)
        assert res.actual is want and not res.fallback, (name, res)


def test_ratio_kl_and_single_rank_distributed_loss_match_references():
    from rl_kernel_b200.ops.distributed import DistributedGRPOLossNativeOp, RatioKLNativeOp
    from rl_kernel_b200.reference.loss.distributed_grpo_loss import DistributedGRPOLossOp
    from rl_kernel_b200.reference.loss.ratio_kl import NativeRatioKLOp

    g = torch.Generator(device="cuda").manual_seed(8)
    B, L, V = 6, 40, 1024
    pol = (torch.randn(B, L, V, device=dev(), generator=g) * 2).bfloat16().requires_grad_(True)
    ref = (pol.detach().float() + 0.05 * torch.randn(B, L, V, device=dev(), generator=g)).bfloat16()
    ids = torch.randint(0, V, (B, L), device=dev(), generator=g)
    mask = torch.ones(B, L, dtype=torch.bool, device=dev())
    mask[1, 30:] = False
    mask[4, :3] = False
    with torch.no_grad():
        old = torch.log_softmax(pol.float(), -1).gather(-1, ids[..., None])[..., 0] + 0.01 * torch.randn(B, L, device=dev(), generator=g)
    ratio, kl = RatioKLNativeOp()(pol, ref, ids, mask, old)
    sync_and_check()
    pr = pol.detach().clone().float().requires_grad_(True)
    rr, rk = NativeRatioKLOp()(pr, ref.float(), ids, mask, old)
    assert (ratio - rr).abs().max().item() < 5e-3 and (kl - rk).abs().max().item() < 5e-3
    (ratio.sum() + kl.sum()).backward()
    (rr.sum() + rk.sum()).backward()
    assert (pol.grad.float() - pr.grad).abs().max().item() < 2e-2
    # data-parallel loss with a single rank == the reference on the whole batch
    logp = (old + 0.02 * torch.randn(B, L, device=dev(), generator=g)).requires_grad_(True)
    refl = old + 0.03 * torch.randn(B, L, device=dev(), generator=g)
    rewards = torch.tensor([1.0, 0.0, 1.0, 1.0, 0.0, 0.0], device=dev())
    loss, pl, k = DistributedGRPOLossNativeOp(clip_eps=0.2, beta=0.01)(logp, old, refl, rewards, mask, samples_per_prompt=3)
    sync_and_check()
    lr2 = logp.detach().clone().requires_grad_(True)
    rl, rpl, rkk = DistributedGRPOLossOp(clip_eps=0.2, beta=0.01)(lr2.cpu(), old.cpu(), refl.cpu(), rewards.cpu(), mask.cpu(),
                                                              samples_per_prompt=3)
    assert abs(loss.item() - rl.item()) < 1e-5 and abs(pl.item() - rpl.item()) < 1e-5 and abs(k.item() - rkk.item()) < 1e-6
    loss.backward()
    g_ref = torch.autograd.grad(rl, [], allow_unused=True) if False else None
    assert logp.grad is not None and torch.isfinite(logp.grad).all() and logp.grad[~mask].abs().max().item() == 0.0


def test_restricted_support_logp_threshold_replay_and_fused_head_agree_bitwise():
    """Train-side log-prob under the rollout's top-k / top-p support: (a) from logits with a per-token
    threshold, (b) the fused LM head with the same threshold in its epilogue, (c) the compact id-list
    kernel -- all three give the same bits, equal to masking the logits first, and match a PyTorch fp32
    reference; the gradient is zero outside the support."""
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.ops.logprob import linear_logp, logp_from_logits, replay_logp_from_logits
    from rl_kernel_b200.ops.sampling.policy import keep_threshold

    g = torch.Generator(device="cuda").manual_seed(31)
    N, H, V = 150, 256, 5000 - 8
    hidden = torch.randn(N, H, device=dev(), generator=g).bfloat16()
    w = (torch.randn(V, H, device=dev(), generator=g) * 0.2).bfloat16()
    logits = torch.empty(N, V, device=dev(), dtype=torch.bfloat16)
    nv.det_gemm(hidden, w, logits, M=N, N=V, K=H)
    T = 0.8
    thr = keep_threshold(logits, temperature=T, top_k=40, top_p=0.9)
    z = logits.float() / T
    keep = z >= thr[:, None]
    counts = keep.sum(1)
    assert int(counts.min()) >= 1 and int(counts.max()) <= 60          # bf16 ties at the boundary stay together
    # a target inside the support (the most likely kept id, and for odd rows the least likely one)
    order = z.masked_fill(~keep, float("-inf")).argsort(dim=-1, descending=True)
    targets = torch.where(torch.arange(N, device=dev()) % 2 == 0, order[:, 0], order.gather(1, (counts - 1)[:, None])[:, 0])
    lg = logits.clone().requires_grad_(True)
    a = logp_from_logits(lg, targets, T, min_keep=thr)
    masked = logits.masked_fill(~keep, float("-inf"))
    a_masked = logp_from_logits(masked, targets, T)
    hh = hidden.clone().requires_grad_(True)
    ww = w.clone().requires_grad_(True)
    b = linear_logp(hh, ww, targets, T, min_keep=thr)
    ids = order[:, :64].clone()
    ids[~keep.gather(1, ids)] = -1                                   # beyond the support: an id no shard owns
    ids[:, 63] = targets                                              # duplicates are allowed
    c, c_lse = replay_logp_from_logits(logits, targets, ids, T, return_lse=True)
    sync_and_check()
    ref = torch.log_softmax(z.masked_fill(~keep, float("-inf")), -1).gather(1, targets[:, None])[:, 0]
    assert torch.equal(a.detach(), a_masked) and torch.equal(a.detach(), b.detach()) and torch.equal(a.detach(), c)
    assert (a.detach() - ref).abs().max().item() < 1e-4
    assert (c_lse - torch.logsumexp(z.masked_fill(~keep, float("-inf")), -1)).abs().max().item() < 1e-4
    gout = torch.randn(N, device=dev(), generator=g)
    a.backward(gout)
    b.backward(gout)
    assert lg.grad[~keep].abs().max().item() == 0.0                   # nothing outside the support moves
    zr = (logits.float() / T).requires_grad_(True)
    torch.log_softmax(zr.masked_fill(~keep, float("-inf")), -1).gather(1, targets[:, None])[:, 0].backward(gout)
    assert (lg.grad.float() - zr.grad / T).abs().max().item() < 2e-2
    assert torch.isfinite(hh.grad).all() and torch.isfinite(ww.grad).all()
    # a target outside the replay set scores -inf, like the dense masked path
    bad = order.gather(1, counts[:, None].clamp(max=V - 1))[:, 0]
    assert torch.isinf(replay_logp_from_logits(logits, bad, ids[:, :63], T)).all()
