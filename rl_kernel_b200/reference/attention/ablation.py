"""Executable attention ablations (parity: AttentionAblationOp, rl_engine/reference/attention/ablation.py:46-738, and
the replay matrix of rl_engine/contracts/diagnostics/attention_matrix.py).

``AttentionAblationOp`` runs the attention block of one layer -- q/k RMSNorm, RoPE, causal GQA attention -- on the
block-wise reference core under explicit settings (positions, theta, norm, scale placement, masks, dtypes, split / merge
policy, page order) and returns a standard result with provenance.  ``run_attention_debug_matrix`` replays a fixed
input through the eleven rows of the matrix: the strict baseline A0, one representative perturbation per root-cause
axis (the topology row is a comparability gate and is rejected, not measured) and three invariant controls whose
drift must be exactly zero.
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import dataclass, field, replace
from types import MappingProxyType
from typing import Any, Mapping

import torch
from torch import Tensor

from rl_kernel_b200.contracts.diagnostics.attention_axes import attention_debug_probe_metadata
from rl_kernel_b200.contracts.diagnostics.attention_matrix import ATTENTION_DEBUG_MATRIX, attention_debug_matrix
from rl_kernel_b200.contracts.operators.attention import AttentionContractError
from rl_kernel_b200.reference.attention.blockwise import blockwise_attention_reference, merge_two_states

BACKEND_ID = "rlkernel.attention.deterministic.v1"
REFERENCE_BACKEND_ID = "rlkernel.attention.reference.v1"
STRICT_ATTENTION_CORE_ID = "rlkernel.attention.blockwise128.v1"
STRICT_ATTENTION_SCHEDULE_ID = "ascending_global_block_index"


@dataclass(frozen=True)
class AttentionAblationConfig:
    backend: str = "auto"
    deterministic: bool = True
    communication_backend: str = "none"
    return_lse: bool = True
    return_gradients: bool = False
    strict_core_id: str = STRICT_ATTENTION_CORE_ID
    strict_schedule: str = STRICT_ATTENTION_SCHEDULE_ID
    validate: bool = True

    def __post_init__(self) -> None:
        for name in ("backend", "communication_backend", "strict_core_id", "strict_schedule"):
            v = getattr(self, name)
            if not isinstance(v, str) or not v.strip():
                raise AttentionContractError(f"{name} must be a non-empty string")
        for name in ("deterministic", "return_lse", "return_gradients", "validate"):
            if not isinstance(getattr(self, name), bool):
                raise AttentionContractError(f"{name} must be a bool")
        object.__setattr__(self, "backend", self.backend.strip().lower())


@dataclass(frozen=True)
class AttentionAblationResult:
    out: Tensor
    lse: Tensor | None
    dq: Tensor | None = None
    dk: Tensor | None = None
    dv: Tensor | None = None
    backend_id: str = BACKEND_ID
    deterministic: bool = True
    provenance: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self) -> None:
        if not isinstance(self.out, Tensor):
            raise TypeError("out must be a tensor")
        object.__setattr__(self, "provenance", MappingProxyType(dict(self.provenance)))

    @property
    def out_lse(self) -> tuple[Tensor, Tensor | None]:
        return self.out, self.lse

    def readback(self) -> dict[str, Any]:
        name = lambda t: None if t is None else str(t.dtype).removeprefix("torch.")  # noqa: E731
        return {"backend_id": self.backend_id, "deterministic": self.deterministic, "out_shape": list(self.out.shape),
                "out_dtype": name(self.out), "lse_shape": None if self.lse is None else list(self.lse.shape), "lse_dtype": name(self.lse),
                "gradients": {k: getattr(self, k) is not None for k in ("dq", "dk", "dv")}, "provenance": dict(self.provenance)}


@dataclass(frozen=True)
class AttentionSettings:
    """Everything the block's result depends on beyond the tensors themselves."""
    position_shift: tuple[int, ...] = ()           # per-sequence shift of position ids (empty: none)
    position_offset: int = 0                        # one offset for all positions
    rope_theta: float = 1_000_000.0
    qk_norm: bool = True
    qk_norm_eps: float = 1e-6
    qk_norm_unit_weight: bool = False
    scale_factor: float = 1.0                       # multiplies 1/sqrt(D)
    scale_on_q: bool = False                        # fold the scale into q (rounded to the execution dtype) before QK^T
    causal: bool = True
    masked_tail_keys: int = 0                       # keys at the end of sequence 0 hidden by a padding mask
    p_dtype: torch.dtype | None = None              # probabilities rounded before P.V (bf16 tensor-core operand)
    execution_dtype: torch.dtype = torch.float32    # dtype q/k/v are rounded to before the core
    final_write_dtype: torch.dtype = torch.float32
    early_downcast: bool = False                    # partial outputs rounded to the write dtype before they merge
    split_kv: int = 0                               # keys per split (0: one pass)
    merge_reversed: bool = False
    cp_degree: int = 1                              # >1: contiguous query/key shards, per-shard softmax, arrival-order merge
    page_swap: tuple[int, int] | None = None        # two 16-token K/V pages of sequence 0 exchanged
    k_noise: float = 0.0                            # added to one cached key

    def fingerprint(self) -> str:
        d = {k: (str(v) if isinstance(v, torch.dtype) else v) for k, v in self.__dict__.items()}
        return hashlib.sha256(json.dumps(d, sort_keys=True, default=str).encode()).hexdigest()[:16]


def _rms(x: Tensor, w: Tensor, eps: float) -> Tensor:
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def _rope(x: Tensor, pos: Tensor, theta: float) -> Tensor:
    D = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    ang = pos.double().unsqueeze(-1) * inv
    c, s = ang.cos().float().unsqueeze(-2), ang.sin().float().unsqueeze(-2)
    a, b = x[..., : D // 2], x[..., D // 2:]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


class AttentionAblationOp:
    """``op(q, k, v, q_gain, k_gain, settings=...)`` with q [B, S, Hq, D], k / v [B, S, Hkv, D] (pre-norm, pre-RoPE)."""

    backend_id = REFERENCE_BACKEND_ID

    def __init__(self, config: AttentionAblationConfig | None = None):
        self.config = config or AttentionAblationConfig()

    # -- stages
    def preprocess(self, q, k, q_gain, k_gain, st: AttentionSettings):
        B, S = q.shape[:2]
        pos = torch.arange(S).repeat(B, 1) + st.position_offset
        for b, sh in enumerate(st.position_shift):
            pos[b] += sh
        if st.qk_norm:
            one = torch.ones_like(q_gain)
            q, k = _rms(q, one if st.qk_norm_unit_weight else q_gain, st.qk_norm_eps), _rms(k, one if st.qk_norm_unit_weight else k_gain,
                                                                                            st.qk_norm_eps)
        q, k = _rope(q.float(), pos, st.rope_theta), _rope(k.float(), pos, st.rope_theta)
        return q.to(st.execution_dtype), k.to(st.execution_dtype)

    def _core(self, q, k, v, q_pos, scale, st: AttentionSettings, kmask=None):
        """One sequence.  q [n, Hq, D] at key positions q_pos, keys [m, Hkv, D]; -> (out fp32, lse)."""
        if not st.causal:
            q_pos = torch.full_like(q_pos, k.shape[0] - 1)
        if kmask is not None:                              # masked keys: drop them and let positions refer to the kept prefix
            keep = int(kmask.sum())
            k, v, q_pos = k[:keep], v[:keep], q_pos.clamp(max=keep - 1)
        bounds = [(0, k.shape[0])] if not st.split_kv else [(a, min(k.shape[0], a + st.split_kv)) for a in range(0, k.shape[0], st.split_kv)]
        parts = []
        for a, e in bounds:
            o, l = blockwise_attention_reference(q.float(), k[a:e].float(), v[a:e].float(), q_pos - a, scale=scale, p_dtype=st.p_dtype,
                                                 strict=True)
            dead = (q_pos - a) < 0                         # queries that see nothing of this split
            o, l = o.float().masked_fill(dead[:, None, None], 0.0), l.masked_fill(dead[:, None], float("-inf"))
            if st.early_downcast:
                o = o.to(st.final_write_dtype).float()
            parts.append((o, l))
        if st.merge_reversed:
            parts = parts[::-1]
        o, l = parts[0]
        for o2, l2 in parts[1:]:
            o, l = merge_two_states(o, l, o2, l2)
        return o, l

    def __call__(self, q, k, v, q_gain, k_gain, *, settings: AttentionSettings | None = None) -> AttentionAblationResult:
        st = settings or AttentionSettings()
        if self.config.validate:
            if q.dim() != 4 or k.shape != v.shape or q.shape[:2] != k.shape[:2] or q.shape[2] % k.shape[2]:
                raise AttentionContractError("q [B, S, Hq, D] and k, v [B, S, Hkv, D] with Hq a multiple of Hkv")
        B, S, Hq, D = q.shape
        qq, kk = self.preprocess(q, k, q_gain, k_gain, st)
        vv = v.to(st.execution_dtype)
        scale = st.scale_factor / math.sqrt(D)
        if st.scale_on_q:
            qq, scale = (qq.float() * scale).to(st.execution_dtype), 1.0
        outs, lses = [], []
        for b in range(B):
            kb, vb = kk[b].clone(), vv[b].clone()
            if b == 0 and st.k_noise:
                kb[S // 2, 0, 0] += st.k_noise
            if b == 0 and st.page_swap is not None:
                i, j = st.page_swap
                for t in (kb, vb):
                    pi, pj = t[i * 16:(i + 1) * 16].clone(), t[j * 16:(j + 1) * 16].clone()
                    t[i * 16:(i + 1) * 16], t[j * 16:(j + 1) * 16] = pj, pi
            kmask = None
            if b == 0 and st.masked_tail_keys:
                kmask = torch.ones(S, dtype=torch.bool)
                kmask[S - st.masked_tail_keys:] = False
            if st.cp_degree > 1:
                o, l = self._cp(qq[b], kb, vb, scale, st)
            else:
                o, l = self._core(qq[b], kb, vb, torch.arange(S), scale, st, kmask)
            outs.append(o)
            lses.append(l)
        out = torch.stack(outs).to(st.final_write_dtype)
        prov = {"core": self.config.strict_core_id, "schedule": "arrival" if (st.merge_reversed or st.cp_degree > 1) else self.config.strict_schedule,
                "settings": st.fingerprint(), "split_kv": st.split_kv, "cp_degree": st.cp_degree,
                "communication_backend": self.config.communication_backend}
        return AttentionAblationResult(out, torch.stack(lses) if self.config.return_lse else None, backend_id=self.backend_id,
                                       deterministic=self.config.deterministic and not st.merge_reversed and st.cp_degree == 1,
                                       provenance=prov)

    def _cp(self, q, k, v, scale, st):
        """Non-strict context parallelism: contiguous shards; every query shard merges the key shards in the order a
        ring delivers them (own shard first, then the earlier ones walking backwards), not by global block index."""
        S = q.shape[0]
        n = st.cp_degree
        edges = [S * i // n for i in range(n + 1)]
        outs, lses = [], []
        for r in range(n):
            qs = slice(edges[r], edges[r + 1])
            state = None
            for step in range(r + 1):
                src = r - step
                ks = slice(edges[src], edges[src + 1])
                o, l = blockwise_attention_reference(q[qs].float(), k[ks].float(), v[ks].float(), torch.arange(qs.start, qs.stop) - ks.start,
                                                     scale=scale, p_dtype=st.p_dtype, strict=True)
                state = (o.float(), l) if state is None else merge_two_states(*state, o.float(), l)
            outs.append(state[0])
            lses.append(state[1])
        return torch.cat(outs), torch.cat(lses)


# ------------------------------------------------------------------------------------------------ the replay matrix
BASELINE = AttentionSettings(p_dtype=torch.bfloat16, execution_dtype=torch.bfloat16, final_write_dtype=torch.bfloat16)

PROBES: dict[str, Any] = {
    "position_ids": lambda s: replace(s, position_shift=(1,)),
    "rope_theta": lambda s: replace(s, rope_theta=10_000.0),
    "position_offsets": lambda s: replace(s, position_offset=64),
    "decode_cache_position": lambda s: replace(s, position_shift=(0, 1)),
    "qk_norm_eps": lambda s: replace(s, qk_norm_eps=1e-5),
    "qk_norm_disabled": lambda s: replace(s, qk_norm=False),
    "qk_norm_weight": lambda s: replace(s, qk_norm_unit_weight=True),
    "attention_scale": lambda s: replace(s, scale_factor=1.01),
    "scale_placement": lambda s: replace(s, scale_on_q=True),
    "causal_mask": lambda s: replace(s, causal=False),
    "key_padding_mask": lambda s: replace(s, masked_tail_keys=3),
    "kv_page_order": lambda s: replace(s, page_swap=(0, 1)),
    "kv_cache_content": lambda s: replace(s, k_noise=0.25),
    "accum_dtype": lambda s: replace(s, p_dtype=None),
    "execution_dtype": lambda s: replace(s, execution_dtype=torch.float32),
    "final_write_dtype": lambda s: replace(s, final_write_dtype=torch.float32),
    "early_downcast": lambda s: replace(s, early_downcast=True, split_kv=128),
    "nonstrict_cp_degree": lambda s: replace(s, cp_degree=2),
    "split_kv": lambda s: replace(s, split_kv=96),
    "merge_order": lambda s: replace(s, split_kv=128, merge_reversed=True),
}


def make_debug_inputs(*, batch: int = 2, seq: int = 320, q_heads: int = 4, kv_heads: int = 2, head_dim: int = 32, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(batch, seq, q_heads, head_dim, generator=g).bfloat16()
    k = torch.randn(batch, seq, kv_heads, head_dim, generator=g).bfloat16()
    v = torch.randn(batch, seq, kv_heads, head_dim, generator=g).bfloat16()
    return q, k, v, (1 + 0.2 * torch.randn(head_dim, generator=g)), (1 + 0.2 * torch.randn(head_dim, generator=g))


def _max_abs(a: Tensor, b: Tensor) -> float:
    d = (a.double() - b.double()).abs()
    return float(torch.nan_to_num(d, nan=0.0).max())


def _controls(op: AttentionAblationOp, inputs, base: AttentionAblationResult) -> dict[str, float]:
    q, k, v, gq, gk = inputs
    hq, hkv = q.shape[2], k.shape[2]
    g = hq // hkv
    halves = [op(q[:, :, i * g * (hkv // 2):(i + 1) * g * (hkv // 2)], k[:, :, i * (hkv // 2):(i + 1) * (hkv // 2)],
                 v[:, :, i * (hkv // 2):(i + 1) * (hkv // 2)], gq, gk, settings=BASELINE) for i in range(2)]
    tp = max(_max_abs(torch.cat([h.out for h in halves], 2), base.out), _max_abs(torch.cat([h.lse for h in halves], 2), base.lse))
    alone = op(q[1:2], k[1:2], v[1:2], gq, gk, settings=BASELINE)
    bc = max(_max_abs(alone.out[0], base.out[1]), _max_abs(alone.lse[0], base.lse[1]))
    # decode tail: the last query against the cached keys is the last row of the prefill
    qq, kk = op.preprocess(q[:1], k[:1], gq, gk, BASELINE)
    S = q.shape[1]
    o, l = op._core(qq[0, S - 1:], kk[0], v[0].to(BASELINE.execution_dtype), torch.tensor([S - 1]), 1.0 / math.sqrt(q.shape[-1]), BASELINE)
    tail = max(_max_abs(o[0].to(BASELINE.final_write_dtype), base.out[0, S - 1]), _max_abs(l[0], base.lse[0, S - 1]))
    return {"tp_partition_control": tp, "batch_composition_control": bc, "prefill_decode_tail_control": tail}


def run_attention_debug_matrix(inputs=None, *, op: AttentionAblationOp | None = None) -> dict[str, Any]:
    """Replay ``inputs`` through every row.  Diagnostic rows report their drift against A0; the gate row is rejected with
    its reason; the controls must read exactly zero (``passed`` says whether they all do)."""
    op = op or AttentionAblationOp()
    inputs = inputs or make_debug_inputs()
    base = op(*inputs, settings=BASELINE)
    controls = _controls(op, inputs, base)
    rows = []
    for row in ATTENTION_DEBUG_MATRIX:
        rec = row.to_dict()
        if row.category == "baseline":
            rec.update(status="baseline", readback=base.readback())
        elif row.category == "comparability_gate":
            rec.update(status="rejected", reason="head ownership differs between the two sides: their per-head results are not "
                                                 "the same quantities, so no drift is computed")
        elif row.category == "invariant_control":
            rec.update(status="pass" if controls[row.probe] == 0.0 else "fail", out_max_abs=controls[row.probe])
        else:
            res = op(*inputs, settings=PROBES[row.probe](BASELINE))
            rec.update(status="measured", out_max_abs=_max_abs(res.out, base.out), lse_max_abs=_max_abs(res.lse, base.lse),
                       deterministic=res.deterministic,
                       **{k: v for k, v in attention_debug_probe_metadata(row.probe).items() if k != "category"})
        rows.append(rec)
    return {**{k: v for k, v in attention_debug_matrix().items() if k != "rows"}, "rows": rows,
            "passed": all(r["status"] != "fail" for r in rows)}


def run_attention_subprobe(probe: str, inputs=None, *, op: AttentionAblationOp | None = None) -> dict[str, Any]:
    """One sub-probe (not only the representatives) against the baseline."""
    meta = attention_debug_probe_metadata(probe)
    if probe not in PROBES:
        raise AttentionContractError(f"probe {probe!r} is a gate or a control and has no perturbation")
    op = op or AttentionAblationOp()
    inputs = inputs or make_debug_inputs()
    base, res = op(*inputs, settings=BASELINE), op(*inputs, settings=PROBES[probe](BASELINE))
    return {"probe": probe, **meta, "out_max_abs": _max_abs(res.out, base.out), "lse_max_abs": _max_abs(res.lse, base.lse)}


__all__ = ["AttentionAblationConfig", "AttentionAblationOp", "AttentionAblationResult", "AttentionSettings", "BACKEND_ID", "BASELINE",
           "PROBES", "REFERENCE_BACKEND_ID", "STRICT_ATTENTION_CORE_ID", "STRICT_ATTENTION_SCHEDULE_ID", "make_debug_inputs",
           "run_attention_debug_matrix", "run_attention_subprobe"]
