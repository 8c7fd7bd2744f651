"""CPU checks of the mixture-of-experts contract: router tie-breaking and renormalisation, the
dispatch plan's ordering, and independence of a token's output from the rest of the batch."""
import torch

from rl_kernel_b200.reference.moe import moe_dispatch_plan_reference, moe_ffn_reference, router_topk_reference


def test_router_is_sorted_renormalised_and_breaks_ties_low():
    logits = torch.randn(64, 32)
    logits[0] = 1.0
    idx, w, p = router_topk_reference(logits, 4)
    assert idx[0].tolist() == [0, 1, 2, 3]
    assert torch.all(idx[:, 1:] > idx[:, :-1])
    assert torch.allclose(w.sum(-1), torch.ones(64), atol=1e-6)
    top = torch.topk(p[1:], 4, dim=-1).indices.sort(-1).values
    assert torch.equal(idx[1:], top)


def test_dispatch_plan_orders_rows_by_source_rank_then_token():
    g = torch.Generator().manual_seed(0)
    idx = [torch.stack([torch.randperm(8, generator=g)[:2].sort().values for _ in range(50)]) for _ in range(2)]
    rows, base, total, padded = moe_dispatch_plan_reference(idx, 8)
    assert torch.all(padded % 128 == 0) and torch.all(padded >= total)
    for e in range(8):
        r0 = rows[0][idx[0] == e]
        r1 = rows[1][idx[1] == e]
        got = torch.cat([r0, r1])
        assert torch.equal(got, base[e] + torch.arange(got.numel())), "rank 0's copies first, each in token order"
    # experts of one owner do not overlap
    assert base[1] == padded[0] and base[4] == 0


def test_token_output_does_not_depend_on_the_batch():
    g = torch.Generator().manual_seed(1)
    bf = torch.bfloat16
    T, H, I, E, K = 24, 32, 16, 8, 2
    x = torch.randn(T, H, generator=g).to(bf)
    wr = (torch.randn(E, H, generator=g) * 0.1).to(bf)
    w1 = (torch.randn(E, 2 * I, H, generator=g) * 0.1).to(bf)
    w2 = (torch.randn(E, H, I, generator=g) * 0.1).to(bf)
    full, _, _ = moe_ffn_reference(x, wr, w1, w2, K)
    part, _, _ = moe_ffn_reference(x[5:9], wr, w1, w2, K)
    assert torch.equal(part, full[5:9])
