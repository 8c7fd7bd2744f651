"""CPU restatement of the mixture-of-experts contract implemented by csrc/moe/*.cu.

Router: fp32 softmax over all experts, top-k by probability (ties to the lower expert id), weights
renormalised over the selected experts, a token's experts kept in ascending id.  Experts: SwiGLU
with bf16 materialisation after each GEMM and after the activation.  Combine: per token an fp32
fma chain over its experts in ascending id, starting from ``base`` (the shared-expert output or
zero), rounded to bf16 once.  Dispatch order inside an expert: (source rank, token, k).

The reference project lists MoE as roadmap only (rl_engine/ops/moe/__init__.py is an empty package;
docs/blog/2026-08-09-dsv4-flash-moe-consistency-roadmap.md:120-134).
"""
from __future__ import annotations

import torch

BF16 = torch.bfloat16


def router_topk_reference(logits: torch.Tensor, k: int):
    """logits fp32 [T, E] -> (idx int64 [T, k] ascending, w fp32 [T, k], probs fp32 [T, E])."""
    l32 = logits.float()
    p = torch.exp(l32 - l32.max(dim=-1, keepdim=True).values)
    p = p / p.sum(dim=-1, keepdim=True)
    E = p.shape[-1]
    # stable descending sort: equal probabilities keep ascending expert order
    order = torch.sort(-p, dim=-1, stable=True).indices[:, :k]
    idx = torch.sort(order, dim=-1).values
    sel = torch.gather(p, 1, idx)
    w = sel / sel.sum(dim=-1, keepdim=True)
    assert E >= k
    return idx, w, p


def moe_dispatch_plan_reference(idx_per_rank: list[torch.Tensor], num_experts: int):
    """For every source rank s and routed copy (t, k): the row of the owner's buffer it lands in.
    Returns (rows per rank [list of [T_s, k] tensors], per-expert (base, total, padded) lists per owner)."""
    W = len(idx_per_rank)
    e_loc = num_experts // W
    counts = torch.stack([torch.bincount(i.reshape(-1), minlength=num_experts) for i in idx_per_rank])
    total = counts.sum(0)
    padded = (total + 127) // 128 * 128
    base = torch.zeros(num_experts, dtype=torch.long)
    for e in range(num_experts):
        o = e // e_loc
        base[e] = padded[o * e_loc:e].sum()
    rows = []
    for s, idx in enumerate(idx_per_rank):
        flat = idx.reshape(-1)
        out = torch.empty_like(flat)
        for e in range(num_experts):
            hit = torch.nonzero(flat == e).reshape(-1)
            out[hit] = base[e] + counts[:s, e].sum() + torch.arange(hit.numel())
        rows.append(out.view_as(idx))
    return rows, base, total, padded


def _swiglu(gu: torch.Tensor, inter: int) -> torch.Tensor:
    g, u = gu[:, :inter].float(), gu[:, inter:].float()
    return (g / (1.0 + torch.exp(-g)) * u).to(BF16)


def moe_ffn_reference(x: torch.Tensor, w_router: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, k: int,
                      base: torch.Tensor | None = None):
    """x bf16 [T, H]; w_router bf16 [E, H]; w1 bf16 [E, 2I, H] ([gate | up] rows); w2 bf16 [E, H, I].
    Returns (out bf16 [T, H], idx, w)."""
    T, H = x.shape
    E, two_i, _ = w1.shape
    inter = two_i // 2
    logits = x.float() @ w_router.float().t()
    idx, w, _ = router_topk_reference(logits, k)
    acc = base.float().clone() if base is not None else torch.zeros(T, H)
    y_all = torch.zeros(T, k, H, dtype=BF16)
    for e in range(E):
        hit = torch.nonzero(idx == e)
        if hit.numel() == 0:
            continue
        xe = x[hit[:, 0]].float()
        gu = (xe @ w1[e].float().t()).to(BF16)
        act = _swiglu(gu, inter)
        y_all[hit[:, 0], hit[:, 1]] = (act.float() @ w2[e].float().t()).to(BF16)
    for j in range(k):       # ascending expert id
        acc = torch.addcmul(acc, w[:, j:j + 1], y_all[:, j].float())
    return acc.to(BF16), idx, w
