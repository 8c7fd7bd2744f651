"""Paged-KV decode / prefill attention behind the FlashInfer-shaped operator surface (parity:
FlashInferQwen3PagedAttentionOp, rl_engine/backends/cuda/attention/flashinfer_paged_attention.py:66-2196).

The reference drives FlashInfer's ``BatchPrefillWithPagedKVCacheWrapper`` and reads its split-KV plan back.  Here the
same inputs (``DecodeAttentionInputs``: queries, a page pool, block table, positions) run on this framework's own sm_100a
paged attention kernel, whose schedule is fixed -- 128-key blocks in ascending logical order, no split-KV -- so the
"actual plan" it reports is that schedule.  The plan builder produces the CSR page metadata (indptr / indices /
last_page_len) a FlashInfer-style runtime consumes, for callers that hand it to another engine.  On CPU tensors the
strict block-wise core computes the same result.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass, field
from typing import Any

import torch

from rl_kernel_b200.validation.common.attention_comparison import (DecodeAttentionInputs, _decode_q, _logical_kv, _scale,
                                                                   _validate_decode, run_decode_strict_shared_core)

BACKEND_ID = "rlkernel.b200.paged_attention.v1"


class FlashInferUnavailable(RuntimeError):
    """The requested FlashInfer runtime path cannot run here (no CUDA device, or a geometry the kernels do not cover)."""


@dataclass(frozen=True)
class FlashInferRoPEFusionConfig:
    enabled: bool = False
    rotary_dim: int | None = None
    theta: float = 1_000_000.0
    interleave: bool = False

    def validate(self, head_dim: int) -> None:
        rd = self.rotary_dim or head_dim
        if rd % 2 or rd > head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        if self.interleave:
            raise ValueError("Qwen3 uses the NeoX (half-split) rotation, not the interleaved one")

    def provenance(self, head_dim: int) -> dict[str, Any]:
        return {"fused_rope": self.enabled, "rotary_dim": self.rotary_dim or head_dim, "theta": self.theta, "style": "neox"}


@dataclass(frozen=True)
class FlashInferPagedAttentionConfig:
    causal: bool = True
    backend: str = "auto"                     # auto | native | reference
    strict: bool = True                       # fixed schedule, no split-KV
    return_lse: bool = True
    rope: FlashInferRoPEFusionConfig = field(default_factory=FlashInferRoPEFusionConfig)
    kv_layout: str = "NHD"

    def validate(self, *, head_dim: int, query_len: int) -> None:
        if self.backend not in ("auto", "native", "reference"):
            raise ValueError("backend must be auto, native or reference")
        if self.kv_layout != "NHD":
            raise ValueError("the page pool is [page, token, head, dim] (NHD)")
        if query_len < 1:
            raise ValueError("query_len must be positive")
        self.rope.validate(head_dim)


@dataclass(frozen=True)
class FlashInferPagedKVPlan:
    """CSR description of every request's pages, the form FlashInfer-style runtimes plan with."""
    kv_indptr: torch.Tensor            # [B + 1]
    kv_indices: torch.Tensor           # [sum pages]
    kv_last_page_len: torch.Tensor     # [B]
    qo_indptr: torch.Tensor            # [B + 1]
    page_size: int
    kv_seq_lens: tuple[int, ...]

    def provenance(self) -> dict[str, Any]:
        return {"page_size": self.page_size, "requests": len(self.kv_seq_lens), "pages": int(self.kv_indices.numel()),
                "kv_seq_lens": list(self.kv_seq_lens), "layout_sha256": hashlib.sha256(
                    self.kv_indices.cpu().numpy().tobytes() + self.kv_indptr.cpu().numpy().tobytes()).hexdigest()[:16]}


@dataclass(frozen=True)
class FlashInferAttentionResult:
    out: torch.Tensor
    lse: torch.Tensor | None
    provenance: dict[str, Any]


def build_flashinfer_paged_kv_plan(inputs: DecodeAttentionInputs, *, query_len: int = 1) -> FlashInferPagedKVPlan:
    _validate_decode(inputs)
    md = inputs.metadata
    lens = [int(x) for x in md.kv_seq_lens]
    indptr, indices, last = [0], [], []
    for b, n in enumerate(lens):
        need = (n + md.page_size - 1) // md.page_size
        indices += [int(p) for p in md.block_table[b, :need]]
        indptr.append(len(indices))
        last.append(n - (need - 1) * md.page_size)
    dev = inputs.q.device
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)  # noqa: E731
    return FlashInferPagedKVPlan(mk(indptr), mk(indices), mk(last), mk([i * query_len for i in range(len(lens) + 1)]), md.page_size,
                                 tuple(lens))


def materialize_flashinfer_paged_kv_cache(inputs: DecodeAttentionInputs) -> torch.Tensor:
    """The combined cache [num_pages, 2, page_size, Hkv, D] FlashInfer-style runtimes take."""
    return torch.stack([inputs.k_cache, inputs.v_cache], 1).contiguous()


def flashinfer_qwen3_paged_attention_available() -> bool:
    """True when the native paged path can run: a CUDA device with the library loaded."""
    if not torch.cuda.is_available():
        return False
    try:
        from rl_kernel_b200.backends import extension as ext

        ext.load()
    except Exception:  # noqa: BLE001 - any load problem means "not available"
        return False
    return True


def flashinfer_prefix_cache_fingerprint(inputs: DecodeAttentionInputs, *, prefix_length: int | None = None) -> str:
    from rl_kernel_b200.validation.common.attention_comparison import decode_prefix_cache_fingerprint

    return decode_prefix_cache_fingerprint(inputs, prefix_length=prefix_length)


class FlashInferQwen3PagedAttentionOp:
    """``op(inputs, config) -> FlashInferAttentionResult``: one decode query per request over its paged cache."""

    backend_id = BACKEND_ID

    def __call__(self, inputs: DecodeAttentionInputs, config: FlashInferPagedAttentionConfig | None = None) -> FlashInferAttentionResult:
        return self.forward(inputs, config)

    def forward(self, inputs: DecodeAttentionInputs, config: FlashInferPagedAttentionConfig | None = None) -> FlashInferAttentionResult:
        cfg = config or FlashInferPagedAttentionConfig()
        _validate_decode(inputs)
        cfg.validate(head_dim=inputs.q.shape[-1], query_len=1)
        plan = build_flashinfer_paged_kv_plan(inputs)
        md = inputs.metadata
        native_ok = (inputs.q.is_cuda and md.page_size == 128 and inputs.q.shape[-1] == 128 and inputs.q.dtype == torch.bfloat16
                     and md.q_rope_state == "post_rope" and md.k_cache_rope_state == "post_rope" and inputs.k_new is None)
        if cfg.backend == "native" and not native_ok:
            raise FlashInferUnavailable("the native paged kernel takes CUDA bf16 tensors, 128-token pages, head_dim 128 and "
                                        "post-RoPE operands already in the cache")
        if cfg.backend == "reference" or not native_ok:
            r = run_decode_strict_shared_core(inputs)
            return FlashInferAttentionResult(r.out, r.lse if cfg.return_lse else None,
                                             {"backend_id": "rlkernel.attention.reference.v1", "plan": plan.provenance(),
                                              "actual_split_kv": self.actual_split_kv_plan(plan), **cfg.rope.provenance(inputs.q.shape[-1])})
        from rl_kernel_b200.ops.attention.paged import paged_attention_block_table

        B, Hq, D = inputs.q.shape
        Hkv = inputs.k_cache.shape[2]
        kp, vp = inputs.k_cache.reshape(-1, Hkv * D), inputs.v_cache.reshape(-1, Hkv * D)
        o, lse = paged_attention_block_table(inputs.q.contiguous(), kp, vp, md.block_table.to(torch.int32), list(plan.kv_seq_lens),
                                             list(range(B + 1)), num_kv_heads=Hkv, scale=_scale(inputs), return_lse=True)
        return FlashInferAttentionResult(o.to(inputs.output_dtype), lse if cfg.return_lse else None,
                                         {"backend_id": BACKEND_ID, "plan": plan.provenance(), "actual_split_kv": self.actual_split_kv_plan(plan),
                                          "arithmetic": {"qk": "bf16 x bf16 -> fp32 (tcgen05)", "softmax": "fp32 online, 128-key blocks ascending",
                                                         "pv": "bf16 P x bf16 V -> fp32"}, **cfg.rope.provenance(D)})

    @staticmethod
    def actual_split_kv_plan(plan: FlashInferPagedKVPlan) -> list[dict[str, Any]]:
        """What the kernel really does with every request's keys: one pass, blocks of 128 in ascending order."""
        return [{"request": i, "kv_len": n, "splits": 1, "split_bounds": [[0, n]], "block": 128, "order": "ascending"}
                for i, n in enumerate(plan.kv_seq_lens)]


__all__ = ["BACKEND_ID", "FlashInferAttentionResult", "FlashInferPagedAttentionConfig", "FlashInferPagedKVPlan",
           "FlashInferQwen3PagedAttentionOp", "FlashInferRoPEFusionConfig", "FlashInferUnavailable", "build_flashinfer_paged_kv_plan",
           "flashinfer_prefix_cache_fingerprint", "flashinfer_qwen3_paged_attention_available", "materialize_flashinfer_paged_kv_cache"]
