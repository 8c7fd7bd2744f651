"""Single-GPU attention attribution harness (parity: rl_engine/validation/common/attention_comparison.py:53-2127).

The same attention problem is materialised along several paths -- whole, query-chunked, KV-paged
with an ordered merge of partial states, RoPE applied before or inside, decode against a paged
cache -- and every path is compared with a reference path: output, log-sum-exp and, when an LM head
and targets are given, the selected log-prob downstream.  Two families:

* tolerance paths (``run_full_attention`` and friends): fp32 PyTorch softmax, whose bits depend on
  the shapes a path happens to use; their drift measures how much a layout may move a result;
* strict paths (``run_strict_shared_core_*``): the block-wise core with a fixed 128-key block order
  and per-row products, whose result for a query row cannot depend on chunking or paging -- the
  drift must be exactly zero.  On a CUDA device ``run_device_attention`` adds the sm_100a kernel,
  which follows the same block order.
"""
from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass
from typing import Any, Literal

import torch

from rl_kernel_b200.contracts.operators.attention import SplitKVSpec
from rl_kernel_b200.reference.attention.blockwise import blockwise_attention_reference, merge_two_states
from rl_kernel_b200.reference.attention.standard_attn import NativeAttentionOp

RoPEState = Literal["pre_rope", "post_rope"]


class TransformerEngineUnavailable(RuntimeError):
    """Transformer Engine's context-parallel merge helpers are not importable in this environment."""


@dataclass(frozen=True)
class AttentionComparisonInputs:
    q: torch.Tensor                                  # [B, S, Hq, D]
    k: torch.Tensor                                  # [B, S, Hkv, D]
    v: torch.Tensor
    causal: bool = True
    scale: float | None = None
    key_padding_mask: torch.Tensor | None = None     # [B, S] bool, True = key takes part
    lm_head_weight: torch.Tensor | None = None       # [V, Hq * D]
    target_ids: torch.Tensor | None = None           # [B, S]
    active_token_mask: torch.Tensor | None = None    # [B, S] bool
    output_dtype: torch.dtype = torch.float32
    rope_positions: torch.Tensor | None = None       # [S] or [B, S]
    rope_theta: float = 1_000_000.0
    rope_rotary_dim: int | None = None
    rope_cast_at: str = "after_rope"                 # after_rope | after_attention
    rope_output_dtype: torch.dtype | None = None


@dataclass(frozen=True)
class DecodeKVCacheMetadata:
    """Logical identity and physical layout of a decode-stage cache.  ``block_table`` [B, max_blocks] maps a request's
    logical KV blocks to cache pages (-1 = none); ``cache_position`` [num_pages, page_size] holds the logical position
    stored in every slot (-1 = unused).  Keeping both explicit separates a layout change from a change of the
    logical sequence."""
    cache_position: torch.Tensor
    kv_seq_lens: torch.Tensor                        # [B]
    block_table: torch.Tensor
    global_token_positions: torch.Tensor             # [B] position of the decode query
    query_position_ids: torch.Tensor                 # [B] RoPE position of the query
    key_position_ids: torch.Tensor                   # [B, max_len] RoPE position of every cached key
    page_size: int
    prefix_cache_key: str | None = None
    prefix_cache_enabled: bool = False
    prefix_length: int = 0
    prefix_cache_fingerprint: str | None = None
    q_rope_state: RoPEState = "post_rope"
    k_cache_rope_state: RoPEState = "post_rope"
    cp_block_owners: torch.Tensor | None = None      # [B, max_blocks] owner rank of a block under paged context parallelism
    cp_world_size: int = 1


@dataclass(frozen=True)
class DecodeAttentionInputs:
    q: torch.Tensor                                  # [B, Hq, D]: one query token per request
    k_cache: torch.Tensor                            # [num_pages, page_size, Hkv, D]
    v_cache: torch.Tensor
    metadata: DecodeKVCacheMetadata
    scale: float | None = None
    output_dtype: torch.dtype = torch.float32
    rope_theta: float = 1_000_000.0
    rope_rotary_dim: int | None = None
    rope_cast_at: str = "after_rope"
    q_rope_output_dtype: torch.dtype | None = None
    k_cache_rope_output_dtype: torch.dtype | None = None
    lm_head_weight: torch.Tensor | None = None
    target_ids: torch.Tensor | None = None           # [B]
    active_token_mask: torch.Tensor | None = None    # [B]
    k_new: torch.Tensor | None = None                # [B, Hkv, D]: this step's K/V when not yet in the cache
    v_new: torch.Tensor | None = None
    split_kv: SplitKVSpec | None = None


@dataclass(frozen=True)
class AttentionPathResult:
    name: str
    out: torch.Tensor
    lse: torch.Tensor
    provenance: dict[str, Any]
    post_rope_q: torch.Tensor | None = None
    post_rope_k: torch.Tensor | None = None


@dataclass(frozen=True)
class DriftStats:
    max_abs: float
    mean_abs: float
    p95_abs: float
    p99_abs: float
    active_count: int

    def to_dict(self) -> dict[str, Any]:
        return {"max_abs": self.max_abs, "mean_abs": self.mean_abs, "p95_abs": self.p95_abs, "p99_abs": self.p99_abs,
                "active_count": self.active_count}

    @property
    def bitwise_zero(self) -> bool:
        return self.active_count > 0 and self.max_abs == 0.0


@dataclass(frozen=True)
class AttentionPathDrift:
    candidate_name: str
    out: DriftStats
    lse: DriftStats
    dlogp: DriftStats | None
    provenance: dict[str, Any]
    post_rope_q: DriftStats | None = None
    post_rope_k: DriftStats | None = None

    def to_dict(self) -> dict[str, Any]:
        opt = lambda s: None if s is None else s.to_dict()  # noqa: E731
        return {"candidate_name": self.candidate_name, "out": self.out.to_dict(), "lse": self.lse.to_dict(), "dlogp": opt(self.dlogp),
                "post_rope_q": opt(self.post_rope_q), "post_rope_k": opt(self.post_rope_k), "provenance": self.provenance}


@dataclass(frozen=True)
class AttentionComparisonReport:
    reference_name: str
    drifts: tuple[AttentionPathDrift, ...]
    unavailable: tuple[str, ...] = ()

    def to_dict(self) -> dict[str, Any]:
        return {"reference_name": self.reference_name, "drifts": [d.to_dict() for d in self.drifts],
                "unavailable": list(self.unavailable)}

    @property
    def bitwise(self) -> bool:
        return all(d.out.bitwise_zero and d.lse.bitwise_zero for d in self.drifts)


# ------------------------------------------------------------------------------------------------ helpers
def _positive(value, name: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ValueError(f"{name} must be a positive integer")
    return value


def _bounds(length: int, size: int) -> list[tuple[int, int]]:
    return [(a, min(length, a + size)) for a in range(0, length, size)]


def _scale(inputs) -> float:
    return inputs.scale if inputs.scale is not None else 1.0 / math.sqrt(inputs.q.shape[-1])


def _validate(inputs: AttentionComparisonInputs) -> None:
    q, k, v = inputs.q, inputs.k, inputs.v
    if q.dim() != 4 or k.dim() != 4 or v.shape != k.shape:
        raise ValueError("q, k, v must be [B, S, H, D] with k and v of one shape")
    if q.shape[0] != k.shape[0] or q.shape[3] != k.shape[3] or q.shape[2] % k.shape[2]:
        raise ValueError("batch and head_dim must agree and the query heads must be a multiple of the KV heads")
    if inputs.causal and q.shape[1] != k.shape[1]:
        raise ValueError("causal comparison paths take self-attention inputs (as many queries as keys)")
    if inputs.key_padding_mask is not None and inputs.key_padding_mask.shape != k.shape[:2]:
        raise ValueError("key_padding_mask must be [B, S]")
    if (inputs.lm_head_weight is None) != (inputs.target_ids is None):
        raise ValueError("lm_head_weight and target_ids come together")
    if inputs.lm_head_weight is not None and inputs.lm_head_weight.shape[1] != q.shape[2] * q.shape[3]:
        raise ValueError("lm_head_weight must be [V, Hq * D]")
    if inputs.rope_cast_at not in ("after_rope", "after_attention"):
        raise ValueError("rope_cast_at must be after_rope or after_attention")


def _drift(c: torch.Tensor, r: torch.Tensor, mask: torch.Tensor | None = None) -> DriftStats:
    d = (c.double() - r.double()).abs()
    d = torch.nan_to_num(d, nan=0.0) if bool(torch.isinf(c).any() or torch.isinf(r).any()) else d   # -inf lse on both sides
    if mask is not None:
        while mask.dim() < d.dim():
            mask = mask.unsqueeze(-1)
        d = d[mask.expand_as(d)]
    vals = d.reshape(-1)
    if vals.numel() == 0:
        return DriftStats(0.0, 0.0, 0.0, 0.0, 0)
    s = vals.sort().values
    pick = lambda qq: float(s[min(s.numel() - 1, int(round(qq * (s.numel() - 1))))])  # noqa: E731
    return DriftStats(float(s[-1]), float(vals.mean()), pick(0.95), pick(0.99), int(vals.numel()))


def _selected_logps(out: torch.Tensor, inputs) -> torch.Tensor | None:
    if inputs.lm_head_weight is None:
        return None
    lead = out.shape[:-2]
    logits = out.reshape(*lead, -1).float() @ inputs.lm_head_weight.float().t()
    return torch.log_softmax(logits, -1).gather(-1, inputs.target_ids.unsqueeze(-1)).squeeze(-1)


def _compare_path(cand: AttentionPathResult, ref: AttentionPathResult, inputs) -> AttentionPathDrift:
    mask = inputs.active_token_mask
    dl = None
    if inputs.lm_head_weight is not None:
        dl = _drift(_selected_logps(cand.out, inputs), _selected_logps(ref.out, inputs), mask)
    rq = rk = None
    if cand.post_rope_q is not None and ref.post_rope_q is not None:
        rq, rk = _drift(cand.post_rope_q, ref.post_rope_q), _drift(cand.post_rope_k, ref.post_rope_k)
    return AttentionPathDrift(cand.name, _drift(cand.out, ref.out, mask), _drift(cand.lse, ref.lse, mask), dl,
                              {"candidate": cand.provenance, "reference": ref.provenance}, rq, rk)


def _attn(q, k, v, inputs, q_pos0: int, kmask=None):
    """fp32 softmax attention of a [B, n, Hq, D] query block at positions q_pos0.. over keys [B, m, Hkv, D]
    (key j at position j of the given slice offset 0) -> (out fp32, lse [B, n, Hq])."""
    o, lse = NativeAttentionOp()(q.float(), k.float(), v.float(), causal=inputs.causal, key_padding_mask=kmask, scale=_scale(inputs),
                                 q_pos0=q_pos0, return_lse=True)
    return o, lse


def _merge(states: list[tuple[torch.Tensor, torch.Tensor]]):
    """Ordered merge of (out, lse) partial states, ascending block order."""
    o, l = states[0]
    for o2, l2 in states[1:]:
        o, l = merge_two_states(o, l, o2, l2)
    return o, l


# ------------------------------------------------------------------------------------------------ tolerance paths
def run_full_attention(inputs: AttentionComparisonInputs) -> AttentionPathResult:
    _validate(inputs)
    o, lse = _attn(inputs.q, inputs.k, inputs.v, inputs, 0, inputs.key_padding_mask)
    return AttentionPathResult("full_attention", o.to(inputs.output_dtype), lse, {"path": "full", "softmax": "fp32"})


def run_chunked_query_attention(inputs: AttentionComparisonInputs, *, query_chunk_size: int | None = None) -> AttentionPathResult:
    _validate(inputs)
    size = _positive(query_chunk_size or max(1, inputs.q.shape[1] // 2), "query_chunk_size")
    outs, lses = [], []
    for a, b in _bounds(inputs.q.shape[1], size):
        # a chunk sees the keys up to its own last position: what a chunked prefill has in its cache
        kv_end = b if inputs.causal else inputs.k.shape[1]
        km = None if inputs.key_padding_mask is None else inputs.key_padding_mask[:, :kv_end]
        o, l = _attn(inputs.q[:, a:b], inputs.k[:, :kv_end], inputs.v[:, :kv_end], inputs, a, km)
        outs.append(o)
        lses.append(l)
    return AttentionPathResult("chunked_query_attention", torch.cat(outs, 1).to(inputs.output_dtype), torch.cat(lses, 1),
                               {"path": "chunked_query", "query_chunk_size": size})


def transformer_engine_context_parallel_available() -> bool:
    try:
        _load_te()
    except TransformerEngineUnavailable:
        return False
    return True


def _load_te():
    try:
        import transformer_engine.pytorch.attention as te_attn  # noqa: F401
    except Exception as exc:  # noqa: BLE001 - any import problem means the backend is not there
        raise TransformerEngineUnavailable(f"transformer_engine is not importable: {type(exc).__name__}: {exc}") from exc
    return te_attn


def run_paged_kv_attention(inputs: AttentionComparisonInputs, *, kv_page_size: int | None = None,
                           merge_backend: str = "rl_kernel") -> AttentionPathResult:
    """Keys split into pages; every page yields a partial state for all queries and the states merge in page order."""
    _validate(inputs)
    if merge_backend == "transformer_engine":
        _load_te()
        raise TransformerEngineUnavailable("the Transformer Engine merge is not wired on this platform")
    if merge_backend != "rl_kernel":
        raise ValueError("merge_backend must be rl_kernel or transformer_engine")
    size = _positive(kv_page_size or max(1, inputs.k.shape[1] // 2), "kv_page_size")
    B, S = inputs.q.shape[:2]
    states = []
    for a, b in _bounds(inputs.k.shape[1], size):
        km = torch.ones(B, b - a, dtype=torch.bool, device=inputs.q.device) if inputs.key_padding_mask is None \
            else inputs.key_padding_mask[:, a:b]
        # causal against a page: query i sees key j of the page iff a + j <= i, i.e. positions shift by -a
        o, l = NativeAttentionOp()(inputs.q.float(), inputs.k[:, a:b].float(), inputs.v[:, a:b].float(), causal=inputs.causal,
                                   key_padding_mask=km, scale=_scale(inputs), q_pos0=-a, return_lse=True)
        states.append((o, l))
    o, l = _merge(states)
    return AttentionPathResult("paged_kv_attention", o.to(inputs.output_dtype), l,
                               {"path": "paged_kv", "kv_page_size": size, "merge_backend": merge_backend, "merge_order": "ascending"})


# ------------------------------------------------------------------------------------------------ strict paths
def _strict(q, k, v, q_pos, inputs):
    """Block-wise core on one sequence, fp32 in and out."""
    o, lse = blockwise_attention_reference(q.float().cpu(), k.float().cpu(), v.float().cpu(), q_pos.cpu(), scale=_scale(inputs),
                                           strict=True)
    return o.to(q.device), lse.to(q.device)


def _need_strict(inputs):
    _validate(inputs)
    if not inputs.causal or inputs.key_padding_mask is not None:
        raise ValueError("the strict shared core covers causal attention without a padding mask")


def run_strict_shared_core_attention(inputs: AttentionComparisonInputs) -> AttentionPathResult:
    _need_strict(inputs)
    S = inputs.q.shape[1]
    res = [_strict(inputs.q[b], inputs.k[b], inputs.v[b], torch.arange(S), inputs) for b in range(inputs.q.shape[0])]
    return AttentionPathResult("strict_shared_core", torch.stack([r[0] for r in res]).to(inputs.output_dtype),
                               torch.stack([r[1] for r in res]), {"path": "strict_full", "kv_block": 128, "products": "per-row"})


def run_strict_shared_core_chunked_attention(inputs: AttentionComparisonInputs, *, query_chunk_size: int | None = None
                                             ) -> AttentionPathResult:
    _need_strict(inputs)
    S = inputs.q.shape[1]
    size = _positive(query_chunk_size or max(1, S // 2), "query_chunk_size")
    outs, lses = [], []
    for b in range(inputs.q.shape[0]):
        parts = [_strict(inputs.q[b, a:e], inputs.k[b, :e], inputs.v[b, :e], torch.arange(a, e), inputs) for a, e in _bounds(S, size)]
        outs.append(torch.cat([p[0] for p in parts]))
        lses.append(torch.cat([p[1] for p in parts]))
    return AttentionPathResult("strict_shared_core_chunked", torch.stack(outs).to(inputs.output_dtype), torch.stack(lses),
                               {"path": "strict_chunked", "query_chunk_size": size})


def run_strict_shared_core_paged_layout_attention(inputs: AttentionComparisonInputs, *, kv_page_size: int | None = None
                                                  ) -> AttentionPathResult:
    """K/V live in a page pool in scrambled page order; a block table restores the logical order before the core runs."""
    _need_strict(inputs)
    B, S, Hkv, D = inputs.k.shape
    size = _positive(kv_page_size or 16, "kv_page_size")
    nblk = (S + size - 1) // size
    perm = torch.randperm(B * nblk, generator=torch.Generator().manual_seed(B * 7919 + S))
    table = perm.view(B, nblk)
    kp = torch.zeros(B * nblk, size, Hkv, D, dtype=inputs.k.dtype, device=inputs.k.device)
    vp = torch.zeros_like(kp)
    for b in range(B):
        for i, (a, e) in enumerate(_bounds(S, size)):
            kp[table[b, i], : e - a], vp[table[b, i], : e - a] = inputs.k[b, a:e], inputs.v[b, a:e]
    outs, lses = [], []
    for b in range(B):
        kk = kp[table[b]].reshape(-1, Hkv, D)[:S]
        vv = vp[table[b]].reshape(-1, Hkv, D)[:S]
        o, l = _strict(inputs.q[b], kk, vv, torch.arange(S), inputs)
        outs.append(o)
        lses.append(l)
    return AttentionPathResult("strict_shared_core_paged_layout", torch.stack(outs).to(inputs.output_dtype), torch.stack(lses),
                               {"path": "strict_paged_layout", "kv_page_size": size, "pages": int(B * nblk)})


def run_device_attention(inputs: AttentionComparisonInputs) -> AttentionPathResult:
    """The sm_100a attention kernel on CUDA bf16 inputs with head_dim 128 (block order of the strict core)."""
    _need_strict(inputs)
    if not inputs.q.is_cuda:
        raise ValueError("run_device_attention takes CUDA tensors")
    from rl_kernel_b200.ops.attention.attention import causal_attention

    B, S, Hq, D = inputs.q.shape
    cu = [i * S for i in range(B + 1)]
    o, lse = causal_attention(inputs.q.reshape(B * S, Hq, D).bfloat16(), inputs.k.reshape(B * S, -1, D).bfloat16(),
                              inputs.v.reshape(B * S, -1, D).bfloat16(), cu, scale=_scale(inputs), return_lse=True)
    return AttentionPathResult("sm100_attention", o.view(B, S, Hq, D).to(inputs.output_dtype), lse.view(B, S, Hq),
                               {"path": "device", "kernel": "tcgen05 flash attention", "kv_block": 128})


def compare_single_gpu_attention(inputs: AttentionComparisonInputs, *, query_chunk_size: int | None = None,
                                 kv_page_size: int | None = None, include_transformer_engine: bool = False,
                                 strict_bitwise: bool = False, include_device: bool = False) -> AttentionComparisonReport:
    """Whole attention against its chunked and paged materialisations.  With an LM head and targets the report also
    carries the drift of the selected log-prob (candidate minus reference) over the active tokens."""
    _validate(inputs)
    unavailable: list[str] = []
    if strict_bitwise:
        ref = run_strict_shared_core_attention(inputs)
        cands = [run_strict_shared_core_chunked_attention(inputs, query_chunk_size=query_chunk_size),
                 run_strict_shared_core_paged_layout_attention(inputs, kv_page_size=kv_page_size)]
    else:
        ref = run_full_attention(inputs)
        cands = [run_chunked_query_attention(inputs, query_chunk_size=query_chunk_size),
                 run_paged_kv_attention(inputs, kv_page_size=kv_page_size)]
    if include_device:
        cands.append(run_device_attention(inputs))
    if include_transformer_engine:
        try:
            cands.append(run_paged_kv_attention(inputs, kv_page_size=kv_page_size, merge_backend="transformer_engine"))
        except TransformerEngineUnavailable as exc:
            unavailable.append(f"transformer_engine_paged_kv: {exc}")
    return AttentionComparisonReport(ref.name, tuple(_compare_path(c, ref, inputs) for c in cands), tuple(unavailable))


# ------------------------------------------------------------------------------------------------ RoPE placement
def _rope_tables(inputs, device):
    D = inputs.q.shape[-1]
    rd = inputs.rope_rotary_dim or D
    if rd % 2 or rd > D:
        raise ValueError("rope_rotary_dim must be even and at most head_dim")
    pos = inputs.rope_positions
    if pos is None:
        pos = torch.arange(inputs.q.shape[1], device=device)
    inv = 1.0 / (inputs.rope_theta ** (torch.arange(0, rd, 2, dtype=torch.float64, device=device) / rd))
    ang = pos.to(device).double().unsqueeze(-1) * inv              # [S, rd/2] or [B, S, rd/2]
    if ang.dim() == 2:
        ang = ang.unsqueeze(0)
    return ang.cos().float().unsqueeze(2), ang.sin().float().unsqueeze(2), rd


def _apply_rope(x: torch.Tensor, cos, sin, rd: int) -> torch.Tensor:
    xf = x.float()
    a, b = xf[..., : rd // 2], xf[..., rd // 2: rd]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, xf[..., rd:]], -1)


def run_unfused_rope_attention(inputs: AttentionComparisonInputs) -> AttentionPathResult:
    """RoPE as its own operator: q and k are rotated, rounded to the RoPE output dtype, then attended."""
    _validate(inputs)
    cos, sin, rd = _rope_tables(inputs, inputs.q.device)
    dt = inputs.rope_output_dtype or inputs.q.dtype
    q, k = _apply_rope(inputs.q, cos, sin, rd).to(dt), _apply_rope(inputs.k, cos, sin, rd).to(dt)
    o, lse = _attn(q, k, inputs.v, inputs, 0, inputs.key_padding_mask)
    return AttentionPathResult("unfused_rope_attention", o.to(inputs.output_dtype), lse,
                               {"path": "rope_then_attention", "rope_output_dtype": str(dt), "rotary_dim": rd}, q, k)


def run_fused_like_rope_attention(inputs: AttentionComparisonInputs) -> AttentionPathResult:
    """RoPE inside the attention prologue: with ``rope_cast_at='after_attention'`` the rotated q, k stay fp32."""
    _validate(inputs)
    cos, sin, rd = _rope_tables(inputs, inputs.q.device)
    q, k = _apply_rope(inputs.q, cos, sin, rd), _apply_rope(inputs.k, cos, sin, rd)
    if inputs.rope_cast_at == "after_rope":
        dt = inputs.rope_output_dtype or inputs.q.dtype
        q, k = q.to(dt), k.to(dt)
    o, lse = _attn(q, k, inputs.v, inputs, 0, inputs.key_padding_mask)
    return AttentionPathResult("fused_like_rope_attention", o.to(inputs.output_dtype), lse,
                               {"path": "rope_in_prologue", "rope_cast_at": inputs.rope_cast_at, "rotary_dim": rd}, q, k)


def compare_single_gpu_rope_attention(inputs: AttentionComparisonInputs) -> AttentionComparisonReport:
    ref = run_unfused_rope_attention(inputs)
    return AttentionComparisonReport(ref.name, (_compare_path(run_fused_like_rope_attention(inputs), ref, inputs),))


# ------------------------------------------------------------------------------------------------ decode against a paged cache
def _validate_decode(inputs: DecodeAttentionInputs) -> None:
    md = inputs.metadata
    q, kc = inputs.q, inputs.k_cache
    if q.dim() != 3 or kc.dim() != 4 or inputs.v_cache.shape != kc.shape:
        raise ValueError("q must be [B, Hq, D] and the caches [num_pages, page_size, Hkv, D]")
    B = q.shape[0]
    _positive(md.page_size, "page_size")
    if kc.shape[1] != md.page_size or md.cache_position.shape != kc.shape[:2]:
        raise ValueError("cache_position must be [num_pages, page_size] with the caches' page size")
    if md.block_table.dim() != 2 or md.block_table.shape[0] != B or md.kv_seq_lens.shape != (B,):
        raise ValueError("block_table must be [B, max_blocks] and kv_seq_lens [B]")
    if md.cp_world_size > 1 and (md.cp_block_owners is None or md.cp_block_owners.shape != md.block_table.shape):
        raise ValueError("cp_world_size > 1 needs cp_block_owners with the block table's shape")
    if (inputs.k_new is None) != (inputs.v_new is None):
        raise ValueError("k_new and v_new come together")
    for b in range(B):
        n = int(md.kv_seq_lens[b])
        need = (n + md.page_size - 1) // md.page_size
        pages = md.block_table[b, :need]
        if bool((pages < 0).any()) or bool((pages >= kc.shape[0]).any()):
            raise ValueError(f"request {b}: block table does not cover {n} cached tokens")
        stored = md.cache_position[pages.long()].reshape(-1)[:n]
        if not torch.equal(stored.cpu(), torch.arange(n)):
            raise ValueError(f"request {b}: cache_position of its pages is not 0..{n - 1} in logical order")
        if int(md.global_token_positions[b]) < n - 1:
            raise ValueError(f"request {b}: the query at position {int(md.global_token_positions[b])} lies before cached keys")
    if md.prefix_cache_enabled and not 0 <= md.prefix_length <= int(md.kv_seq_lens.min()):
        raise ValueError("prefix_length must lie inside every request's cached length")


def _logical_kv(inputs: DecodeAttentionInputs, b: int):
    md = inputs.metadata
    n = int(md.kv_seq_lens[b])
    pages = md.block_table[b, : (n + md.page_size - 1) // md.page_size].long()
    k = inputs.k_cache[pages].reshape(-1, *inputs.k_cache.shape[2:])[:n]
    v = inputs.v_cache[pages].reshape(-1, *inputs.v_cache.shape[2:])[:n]
    if inputs.k_new is not None:
        k, v = torch.cat([k, inputs.k_new[b][None]]), torch.cat([v, inputs.v_new[b][None]])
    if md.k_cache_rope_state == "pre_rope":
        k = _rope_rows(k, md.key_position_ids[b, : k.shape[0]], inputs, inputs.k_cache_rope_output_dtype or inputs.k_cache.dtype)
    return k, v


def _rope_rows(x: torch.Tensor, pos: torch.Tensor, inputs: DecodeAttentionInputs, dt: torch.dtype) -> torch.Tensor:
    D = x.shape[-1]
    rd = inputs.rope_rotary_dim or D
    inv = 1.0 / (inputs.rope_theta ** (torch.arange(0, rd, 2, dtype=torch.float64, device=x.device) / rd))
    ang = pos.to(x.device).double().reshape(-1, 1) * inv
    y = _apply_rope(x, ang.cos().float().unsqueeze(1), ang.sin().float().unsqueeze(1), rd)
    return y.to(dt) if inputs.rope_cast_at == "after_rope" else y


def _decode_q(inputs: DecodeAttentionInputs, b: int) -> torch.Tensor:
    q = inputs.q[b][None]                                        # [1, Hq, D]
    if inputs.metadata.q_rope_state == "pre_rope":
        q = _rope_rows(q, inputs.metadata.query_position_ids[b: b + 1], inputs, inputs.q_rope_output_dtype or inputs.q.dtype)
    return q


def _decode_result(name, outs, lses, inputs, prov):
    return AttentionPathResult(name, torch.stack(outs).to(inputs.output_dtype), torch.stack(lses), prov)


def run_decode_full_prefill_reference(inputs: DecodeAttentionInputs) -> AttentionPathResult:
    """The decode query attended over its request's logical K/V in one softmax: what a full prefill computes for it."""
    _validate_decode(inputs)
    outs, lses = [], []
    for b in range(inputs.q.shape[0]):
        k, v = _logical_kv(inputs, b)
        o, l = NativeAttentionOp()(_decode_q(inputs, b)[None].float(), k[None].float(), v[None].float(), causal=False,
                                   scale=_scale(inputs), return_lse=True)
        outs.append(o[0, 0])
        lses.append(l[0, 0])
    return _decode_result("decode_full_prefill_reference", outs, lses, inputs, {"path": "decode_full_softmax"})


def _split_bounds(n: int, inputs: DecodeAttentionInputs) -> list[tuple[int, int]]:
    size = inputs.metadata.page_size
    if inputs.split_kv is not None and inputs.split_kv.fixed_split_size:
        size = int(inputs.split_kv.fixed_split_size)
    return _bounds(n, size)


def run_decode_kv_replay(inputs: DecodeAttentionInputs) -> AttentionPathResult:
    """Walk the block table page by page (or split by split), one partial state each, merged in logical order.  Under
    paged context parallelism the blocks of one owner merge first, then the owners in rank order."""
    _validate_decode(inputs)
    md = inputs.metadata
    outs, lses = [], []
    for b in range(inputs.q.shape[0]):
        k, v = _logical_kv(inputs, b)
        q = _decode_q(inputs, b)[None].float()
        parts = []
        for a, e in _split_bounds(k.shape[0], inputs):
            o, l = NativeAttentionOp()(q, k[None, a:e].float(), v[None, a:e].float(), causal=False, scale=_scale(inputs),
                                       return_lse=True)
            owner = 0 if md.cp_world_size == 1 else int(md.cp_block_owners[b, min(a // md.page_size, md.block_table.shape[1] - 1)])
            parts.append((owner, (o[0, 0], l[0, 0])))
        by_owner = [_merge([s for w, s in parts if w == r]) for r in sorted({w for w, _ in parts})]
        o, l = _merge(by_owner)
        outs.append(o)
        lses.append(l)
    return _decode_result("decode_kv_replay", outs, lses, inputs,
                          {"path": "decode_paged_replay", "page_size": md.page_size, "cp_world_size": md.cp_world_size})


def run_decode_strict_shared_core(inputs: DecodeAttentionInputs) -> AttentionPathResult:
    """The block-wise core on the logical K/V: bit-equal to a strict prefill row at the same position."""
    _validate_decode(inputs)
    outs, lses = [], []
    for b in range(inputs.q.shape[0]):
        k, v = _logical_kv(inputs, b)
        o, l = blockwise_attention_reference(_decode_q(inputs, b).float().cpu(), k.float().cpu(), v.float().cpu(),
                                             torch.tensor([k.shape[0] - 1]), scale=_scale(inputs), strict=True)
        outs.append(o[0].to(inputs.q.device))
        lses.append(l[0].to(inputs.q.device))
    return _decode_result("decode_strict_shared_core", outs, lses, inputs, {"path": "decode_strict", "kv_block": 128})


def compare_decode_kv_replay(inputs: DecodeAttentionInputs, *, strict_bitwise: bool = False) -> AttentionComparisonReport:
    ref = run_decode_full_prefill_reference(inputs)
    cands = [run_decode_kv_replay(inputs)] + ([run_decode_strict_shared_core(inputs)] if strict_bitwise else [])
    return AttentionComparisonReport(ref.name, tuple(_compare_path(c, ref, inputs) for c in cands))


# ------------------------------------------------------------------------------------------------ fingerprints
def _hash_tensor(h, t: torch.Tensor) -> None:
    t = t.detach().contiguous().cpu().reshape(-1) if t.dim() == 0 else t.detach().contiguous().cpu()
    h.update(str(t.dtype).encode())
    h.update(str(tuple(t.shape)).encode())
    h.update(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


def decode_prefix_cache_fingerprint(inputs: DecodeAttentionInputs, *, prefix_length: int | None = None) -> str:
    """sha256 of the first ``prefix_length`` LOGICAL cached tokens (K, V and their positions) of every request: equal
    for two caches that hold the same prefix whatever pages it sits in."""
    md = inputs.metadata
    n = md.prefix_length if prefix_length is None else prefix_length
    h = hashlib.sha256(f"prefix:{n}:{md.k_cache_rope_state}".encode())
    for b in range(inputs.q.shape[0]):
        pages = md.block_table[b, : (n + md.page_size - 1) // md.page_size].long()
        _hash_tensor(h, inputs.k_cache[pages].reshape(-1, *inputs.k_cache.shape[2:])[:n])
        _hash_tensor(h, inputs.v_cache[pages].reshape(-1, *inputs.v_cache.shape[2:])[:n])
        _hash_tensor(h, md.key_position_ids[b, :n])
    return h.hexdigest()


def decode_kv_cache_fingerprint(inputs: DecodeAttentionInputs) -> str:
    """sha256 of every request's whole logical cache; independent of the physical page assignment."""
    md = inputs.metadata
    h = hashlib.sha256(f"kv:{md.k_cache_rope_state}:{md.page_size}".encode())
    for b in range(inputs.q.shape[0]):
        n = int(md.kv_seq_lens[b])
        pages = md.block_table[b, : (n + md.page_size - 1) // md.page_size].long()
        _hash_tensor(h, inputs.k_cache[pages].reshape(-1, *inputs.k_cache.shape[2:])[:n])
        _hash_tensor(h, inputs.v_cache[pages].reshape(-1, *inputs.v_cache.shape[2:])[:n])
        _hash_tensor(h, md.kv_seq_lens[b])
    return h.hexdigest()


def decode_rope_identity_fingerprint(inputs: DecodeAttentionInputs) -> str:
    """sha256 of everything that fixes the rotation of q and the cached k: positions, states, theta, rotary dim, dtypes."""
    md = inputs.metadata
    h = hashlib.sha256()
    h.update(repr((md.q_rope_state, md.k_cache_rope_state, float(inputs.rope_theta), inputs.rope_rotary_dim or inputs.q.shape[-1],
                   inputs.rope_cast_at, str(inputs.q_rope_output_dtype), str(inputs.k_cache_rope_output_dtype))).encode())
    _hash_tensor(h, md.query_position_ids)
    for b in range(inputs.q.shape[0]):
        _hash_tensor(h, md.key_position_ids[b, : int(md.kv_seq_lens[b])])
    return h.hexdigest()


__all__ = ["AttentionComparisonInputs", "AttentionComparisonReport", "AttentionPathDrift", "AttentionPathResult", "DecodeAttentionInputs",
           "DecodeKVCacheMetadata", "DriftStats", "TransformerEngineUnavailable", "compare_decode_kv_replay",
           "compare_single_gpu_attention", "compare_single_gpu_rope_attention", "decode_kv_cache_fingerprint",
           "decode_prefix_cache_fingerprint", "decode_rope_identity_fingerprint", "run_chunked_query_attention",
           "run_decode_full_prefill_reference", "run_decode_kv_replay", "run_decode_strict_shared_core", "run_device_attention",
           "run_full_attention", "run_fused_like_rope_attention", "run_paged_kv_attention", "run_strict_shared_core_attention",
           "run_strict_shared_core_chunked_attention", "run_strict_shared_core_paged_layout_attention",
           "run_unfused_rope_attention", "transformer_engine_context_parallel_available"]
