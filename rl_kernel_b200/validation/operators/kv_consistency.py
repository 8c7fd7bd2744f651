"""Decode-vs-prefill and stateful-KV consistency of an attention candidate (parity: rl_engine/validation/operators/
kv_consistency.py:58-744).

Level A (decode == prefill): the query at position t attended over keys 0..t through the candidate's decode path gives
the bits of row t of its prefill.  Level B (stateful KV): a cache filled step by step -- prefill chunk, then one token
per step, written through the cache object and never concatenated by the caller -- yields for every generated position
the bits of a fresh rescore of the whole sequence.  Selected log-probs downstream (a fixed probe head) are compared
too, under the chain thresholds of the precision profile.  Candidates: ``pytorch`` (block-wise strict core, any
device) and ``b200`` (the sm_100a paged kernels; CUDA)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

import torch

from rl_kernel_b200.contracts.numerical import chain_thresholds
from rl_kernel_b200.reference.attention.blockwise import blockwise_attention_reference
from rl_kernel_b200.reference.attention.stateful_kv import StatefulKVCache


@dataclass(frozen=True)
class DecodePrefillCase:
    name: str
    batch: int
    seq_len: int
    decode_from: int
    q_heads: int = 4
    kv_heads: int = 2
    head_dim: int = 128
    seed: int = 0


@dataclass(frozen=True)
class DecodePrefillCell:
    case: str
    position: int
    out_bitwise: bool
    lse_bitwise: bool
    out_max_abs: float
    dlogp_abs: float


@dataclass
class DecodePrefillReport:
    candidate: str
    device: str
    cells: list[DecodePrefillCell] = field(default_factory=list)
    provenance: dict[str, Any] = field(default_factory=dict)

    @property
    def bitwise(self) -> bool:
        return bool(self.cells) and all(c.out_bitwise and c.lse_bitwise for c in self.cells)

    @property
    def max_abs_dlogp(self) -> float:
        return max((c.dlogp_abs for c in self.cells), default=0.0)

    def passed(self, *, require_bitwise: bool = True) -> bool:
        return self.bitwise if require_bitwise else self.max_abs_dlogp <= chain_thresholds()["max_abs_dlogp"]


@dataclass
class StatefulKVReport:
    candidate: str
    device: str
    generated_positions: int = 0
    mismatched_positions: int = 0
    max_abs_dlogp: float = 0.0
    cache_identity: dict[str, str] = field(default_factory=dict)
    writes: int = 0

    @property
    def bitwise(self) -> bool:
        return self.generated_positions > 0 and self.mismatched_positions == 0


def build_decode_prefill_cases(*, head_dim: int = 128) -> tuple[DecodePrefillCase, ...]:
    """Short, block-boundary and multi-block sequences; decode starts inside, at and after a 128-key boundary."""
    return (DecodePrefillCase("short", 2, 40, 24, head_dim=head_dim), DecodePrefillCase("boundary", 2, 130, 126, head_dim=head_dim, seed=1),
            DecodePrefillCase("multi_block", 1, 300, 250, head_dim=head_dim, seed=2))


def resolve_attention_candidate(candidate: str, device: str) -> str:
    c = candidate.strip().lower()
    if c == "auto":
        return "b200" if device.startswith("cuda") else "pytorch"
    if c not in ("pytorch", "b200"):
        raise ValueError("candidate must be auto, pytorch or b200")
    if c == "b200" and not device.startswith("cuda"):
        raise ValueError("the b200 candidate runs on CUDA")
    return c


def _qkv(case: DecodePrefillCase, device, dtype):
    g = torch.Generator().manual_seed(case.seed)
    mk = lambda h: torch.randn(case.batch, case.seq_len, h, case.head_dim, generator=g).to(dtype).to(device)  # noqa: E731
    return mk(case.q_heads), mk(case.kv_heads), mk(case.kv_heads)


def _probe_head(case: DecodePrefillCase, device, vocab: int = 64):
    g = torch.Generator().manual_seed(case.seed + 77)
    return (torch.randn(vocab, case.q_heads * case.head_dim, generator=g) * 0.05).to(device), torch.randint(0, vocab, (case.batch, case.seq_len), generator=g).to(device)


def _logp(out_row: torch.Tensor, W: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    return torch.log_softmax(out_row.reshape(1, -1).float() @ W.float().t(), -1)[0, target]


class _Runner:
    """prefill(q, k, v) -> (out, lse) for one sequence; decode(q_t, k[:t+1], v[:t+1]) -> (out, lse) for one query."""

    def __init__(self, candidate: str):
        self.candidate = candidate

    def prefill(self, q, k, v):
        S = q.shape[0]
        if self.candidate == "pytorch":
            return blockwise_attention_reference(q.cpu(), k.cpu(), v.cpu(), torch.arange(S), strict=True)
        from rl_kernel_b200.ops.attention.attention import causal_attention

        return causal_attention(q, k, v, [0, S], return_lse=True)

    def decode(self, q_t, k, v):
        n = k.shape[0]
        if self.candidate == "pytorch":
            o, l = blockwise_attention_reference(q_t[None].cpu(), k.cpu(), v.cpu(), torch.tensor([n - 1]), strict=True)
            return o[0], l[0]
        from rl_kernel_b200.ops.attention.paged import PAGE, paged_attention_block_table, write_kv_slots

        hkv, d = k.shape[1], k.shape[2]
        pages = (n + PAGE - 1) // PAGE
        kp = torch.zeros(pages * PAGE, hkv * d, device=k.device, dtype=k.dtype)
        vp = torch.zeros_like(kp)
        write_kv_slots(kp, vp, k.reshape(n, -1), v.reshape(n, -1), torch.arange(n, device=k.device))
        o, l = paged_attention_block_table(q_t[None].contiguous(), kp, vp, torch.arange(pages, dtype=torch.int32, device=k.device)[None],
                                           [n], [0, 1], num_kv_heads=hkv, return_lse=True)
        return o[0], l[0]


def _bits(a: torch.Tensor, b: torch.Tensor) -> bool:
    a, b = a.detach().cpu().contiguous(), b.detach().cpu().contiguous()
    return a.dtype == b.dtype and a.shape == b.shape and bool(torch.equal(a.view(torch.uint8), b.view(torch.uint8)))


def assert_decode_prefill_consistent(candidate: str = "auto", *, device: str = "cpu", dtype: torch.dtype | None = None, cases=None,
                                     require_bitwise: bool = True) -> DecodePrefillReport:
    cand = resolve_attention_candidate(candidate, device)
    dtype = dtype or (torch.bfloat16 if cand == "b200" else torch.float32)
    run = _Runner(cand)
    rep = DecodePrefillReport(cand, device, provenance={"dtype": str(dtype), "level": "A"})
    for case in cases or build_decode_prefill_cases(head_dim=128 if cand == "b200" else 32):
        q, k, v = _qkv(case, device, dtype)
        W, tg = _probe_head(case, device)
        for b in range(case.batch):
            out, lse = run.prefill(q[b], k[b], v[b])
            for t in range(case.decode_from, case.seq_len):
                o, l = run.decode(q[b, t], k[b, : t + 1], v[b, : t + 1])
                rep.cells.append(DecodePrefillCell(case.name, t, _bits(o, out[t]), _bits(l.float(), lse[t].float()),
                                                   float((o.float().cpu() - out[t].float().cpu()).abs().max()),
                                                   float((_logp(o.cpu(), W.cpu(), tg[b, t].cpu()) - _logp(out[t].cpu(), W.cpu(), tg[b, t].cpu())).abs())))
    if not rep.passed(require_bitwise=require_bitwise):
        bad = next(c for c in rep.cells if not (c.out_bitwise and c.lse_bitwise))
        raise AssertionError(f"{cand}: decode differs from prefill at case {bad.case} position {bad.position} "
                             f"(max |d out| {bad.out_max_abs:.3e}, |dlogp| {bad.dlogp_abs:.3e})")
    return rep


def assert_stateful_kv_consistent(candidate: str = "auto", *, device: str = "cpu", dtype: torch.dtype | None = None,
                                  case: DecodePrefillCase | None = None, require_bitwise: bool = True) -> StatefulKVReport:
    """Generate-then-rescore through a stateful cache: prefill chunk written once, then one write per step."""
    cand = resolve_attention_candidate(candidate, device)
    dtype = dtype or (torch.bfloat16 if cand == "b200" else torch.float32)
    case = case or DecodePrefillCase("stateful", 2, 140, 120, head_dim=128 if cand == "b200" else 32, seed=3)
    run = _Runner(cand)
    q, k, v = _qkv(case, device, dtype)
    W, tg = _probe_head(case, device)
    cache = StatefulKVCache.allocate(batch=case.batch, kv_heads=case.kv_heads, max_len=case.seq_len, head_dim=case.head_dim, dtype=dtype,
                                     device=device)
    p = case.decode_from
    cache.write(k[:, :p].permute(0, 2, 1, 3), v[:, :p].permute(0, 2, 1, 3), position=0)
    rep = StatefulKVReport(cand, device)
    rescore = [run.prefill(q[b], k[b], v[b]) for b in range(case.batch)]
    for t in range(p, case.seq_len):
        cache.write(k[:, t:t + 1].permute(0, 2, 1, 3), v[:, t:t + 1].permute(0, 2, 1, 3), position=t)
        kk, vv, n = cache.read()
        for b in range(case.batch):
            o, l = run.decode(q[b, t], kk[b].permute(1, 0, 2).contiguous(), vv[b].permute(1, 0, 2).contiguous())
            rep.generated_positions += 1
            same = _bits(o, rescore[b][0][t]) and _bits(l.float(), rescore[b][1][t].float())
            rep.mismatched_positions += 0 if same else 1
            rep.max_abs_dlogp = max(rep.max_abs_dlogp, float((_logp(o.cpu(), W.cpu(), tg[b, t].cpu()) - _logp(rescore[b][0][t].cpu(), W.cpu(),
                                                                                                             tg[b, t].cpu())).abs()))
    rep.cache_identity, rep.writes = cache.identity(), cache.writes
    ok = rep.bitwise if require_bitwise else rep.max_abs_dlogp <= chain_thresholds()["max_abs_dlogp"]
    if not ok:
        raise AssertionError(f"{cand}: {rep.mismatched_positions}/{rep.generated_positions} generated positions differ from the rescore "
                             f"(max |dlogp| {rep.max_abs_dlogp:.3e})")
    return rep


__all__ = ["DecodePrefillCase", "DecodePrefillCell", "DecodePrefillReport", "StatefulKVReport", "assert_decode_prefill_consistent",
           "assert_stateful_kv_consistent", "build_decode_prefill_cases", "resolve_attention_candidate"]
