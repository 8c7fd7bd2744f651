"""Attention provider (parity: rl_engine/integrations/orchestrators/vime/providers/attention.py:55-477).

The request carries this rank's packed ``q`` [T, Hq_local, D], ``k`` / ``v`` [T, Hkv_local, D] after q/k norm and RoPE, the
sequence boundaries ``cu_seqlens`` and ``metadata`` (global head counts, global sequence length under CP).  One rank of
context: the sm_100a causal attention (CUDA bf16, head_dim 128) or the block-wise reference.  Under context parallelism the
request must name the communication object (``cp_attention``: a ``CPAttentionOp`` built by the worker, since peer memory is
set up once per process); requests that ask for materialisations this runtime does not have -- sliding windows, soft caps,
attention bias, dropout -- are refused instead of approximated."""
from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any

import torch

from rl_kernel_b200.contracts.operators.attention import AttentionContract, AttentionMode, AttentionRole
from rl_kernel_b200.integrations.orchestrators.vime.providers._request import cp_coordinates, metadata, positive_int, request_tensor, tp_coordinates


class AttentionProviderUnavailable(RuntimeError):
    attention_provider_unavailable = True


@dataclass(frozen=True)
class AttentionProviderResult:
    out: torch.Tensor                 # [T, Hq_local, D]
    lse: torch.Tensor | None          # [T, Hq_local] fp32
    backend_id: str
    contract_id: str
    provenance: Mapping[str, Any]


_UNSUPPORTED = ("sliding_window", "softcap", "attention_bias", "alibi_slopes", "dropout_p")


def _reject_unsupported(request: Any, md: Mapping[str, Any]) -> None:
    for name in _UNSUPPORTED:
        v = getattr(request, name, md.get(name))
        if v not in (None, 0, 0.0, False, (-1, -1)):
            raise AttentionProviderUnavailable(f"{name}={v!r}: this runtime computes plain causal GQA attention only")
    if getattr(request, "causal", True) is not True:
        raise AttentionProviderUnavailable("non-causal attention is outside the post-training chain")


def _contract_for_request(request: Any, q: torch.Tensor, k: torch.Tensor) -> AttentionContract:
    U = AttentionProviderUnavailable
    md = metadata(request)
    tp_rank, tp_world = tp_coordinates(getattr(request, "tensor_parallel_group", None))
    cp_rank, cp_world, layout = cp_coordinates(request, U)
    hq = positive_int(md.get("num_q_heads", q.shape[1] * tp_world), "num_q_heads", U)
    hkv = positive_int(md.get("num_kv_heads", k.shape[1] * tp_world), "num_kv_heads", U)
    if hq != q.shape[1] * tp_world or hkv != k.shape[1] * tp_world:
        raise U(f"local heads ({q.shape[1]}, {k.shape[1]}) x TP {tp_world} do not give the global ({hq}, {hkv})")
    seq = positive_int(md.get("global_sequence_length"), "global_sequence_length", U)
    nseq = positive_int(md.get("num_sequences", 1), "num_sequences", U)
    try:
        return AttentionContract.for_layout(hq, hkv, head_dim=q.shape[2], seq_len=seq, batch_size=nseq, tp_rank=tp_rank, tp_world_size=tp_world,
                                            cp_rank=cp_rank, cp_world_size=cp_world, layout="none" if cp_world == 1 else
                                            ("zigzag" if layout == "zigzag" else "contiguous"), role=AttentionRole.TRAIN,
                                            mode=AttentionMode.PREFILL)
    except ValueError as exc:
        raise U(f"the request does not form a valid attention contract: {exc}") from exc


def attention_provider(request: Any) -> AttentionProviderResult:
    U = AttentionProviderUnavailable
    q, k, v = (request_tensor(request, n, U) for n in ("q", "k", "v"))
    if q.ndim != 3 or k.ndim != 3 or v.shape != k.shape or q.shape[0] != k.shape[0] or q.shape[2] != k.shape[2] or q.shape[1] % k.shape[1]:
        raise U("request must contain packed q [T, Hq, D] and k, v [T, Hkv, D]")
    md = metadata(request)
    _reject_unsupported(request, md)
    contract = _contract_for_request(request, q, k)
    cp_world = contract.sharding.cp_world_size
    scale = getattr(request, "softmax_scale", None)
    if cp_world > 1:
        cp_op = getattr(request, "cp_attention", None)
        if cp_op is None:
            raise U("context parallelism needs the worker's CPAttentionOp (request.cp_attention): peer memory is set up once per process")
        out, lse = cp_op(q.reshape(q.shape[0], -1), k.reshape(k.shape[0], -1), v.reshape(v.shape[0], -1), nseq=contract.batch_size,
                         seq_len=contract.sharding.global_sequence_length)
        out, backend = out.view_as(q), getattr(cp_op, "backend_id", "b200-cp-attention")
    else:
        from rl_kernel_b200.ops.attention.attention import causal_attention

        cu = getattr(request, "cu_seqlens", None)
        if cu is None:
            n = contract.sharding.global_sequence_length
            cu = [i * n for i in range(q.shape[0] // n + 1)]
        out, lse = causal_attention(q, k, v, cu, scale=scale, return_lse=True)
        backend = "b200-tcgen05" if q.is_cuda else "reference"
    prov = {"actual_backend": backend, "fallback": False,
            "request": {"q_shape": list(q.shape), "k_shape": list(k.shape), "dtype": str(q.dtype).removeprefix("torch."),
                        "tp_world_size": contract.sharding.tp_world_size, "cp_world_size": cp_world},
            "execution": {"role": "vime_training_attention", "strict_backend": True, "kv_block": 128, "order": "ascending global block index"},
            "cp_row_ownership": {"cp_rank": contract.sharding.cp_rank, "cp_world_size": cp_world,
                                 "layout": getattr(getattr(request, "context_parallel", None), "layout", "single")}}
    return AttentionProviderResult(out, lse if getattr(request, "return_lse", True) else None, backend, contract.cross_rank_fingerprint(), prov)


provider = attention_provider

__all__ = ["AttentionProviderResult", "AttentionProviderUnavailable", "attention_provider", "provider"]
