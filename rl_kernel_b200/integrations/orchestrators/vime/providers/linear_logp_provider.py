"""Fused linear + selected-log-prob provider (parity: rl_engine/integrations/orchestrators/vime/providers/
linear_logp_provider.py:33-576).

The request carries the final hidden rows ``hidden`` [T, H], this rank's LM-head shard ``weight`` [V_local, H] and
``target_ids`` [T]; the [T, V] logits are never materialised.  CUDA bf16 operands run the tcgen05 LM-head GEMM whose epilogue
produces the 128-id tile statistics (vocabulary-parallel over the TP group through the deterministic collective); anything
else runs the PyTorch tile reference.  ``temperature`` divides the logits inside the epilogue.  A sampler's support arrives as
``log_prob_min_keep`` [T] (the per-token threshold on the scaled logit that the rollout recorded)."""
from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any

import torch

from rl_kernel_b200.integrations.orchestrators.vime.providers._request import (cp_coordinates, metadata, positive_int, request_tensor,
                                                                               tp_coordinates)


class LinearLogpProviderUnavailable(RuntimeError):
    linear_logp_provider_unavailable = True


@dataclass(frozen=True)
class LinearLogpResult:
    selected_logprobs: torch.Tensor           # [T, 1]
    entropy: torch.Tensor | None
    backend_id: str
    contract_id: str
    provenance: Mapping[str, Any]


def _temperature(request: Any) -> float:
    t = getattr(request, "temperature", None)
    if t is None:
        return 1.0
    if isinstance(t, torch.Tensor):
        if t.numel() != 1:
            raise LinearLogpProviderUnavailable("a per-token temperature is not supported; pass one scalar")
        t = float(t)
    if not t > 0:
        raise LinearLogpProviderUnavailable("temperature must be positive")
    return float(t)


def provider(request: Any, *, linear_logp: Any = None) -> LinearLogpResult:
    U = LinearLogpProviderUnavailable
    hidden, weight, targets = (request_tensor(request, n, U) for n in ("hidden", "weight", "target_ids"))
    md = metadata(request)
    if hidden.ndim != 2 or weight.ndim != 2 or hidden.shape[1] != weight.shape[1] or targets.shape != (hidden.shape[0],):
        raise U("request must contain hidden [T, H], weight [V_local, H] and target_ids [T]")
    cp_rank, cp_world, layout = cp_coordinates(request, U)
    tp_group = getattr(request, "tensor_parallel_group", None)
    tp_rank, tp_world = tp_coordinates(tp_group)
    real = positive_int(md.get("real_vocab_size"), "real_vocab_size", U)
    padded = positive_int(md.get("padded_vocab_size"), "padded_vocab_size", U)
    if weight.shape[0] * tp_world != padded:
        raise U(f"weight shard rows and TP group do not cover padded_vocab_size: {weight.shape[0]} * {tp_world} != {padded}")
    temperature = _temperature(request)
    min_keep = getattr(request, "log_prob_min_keep", None)
    if getattr(request, "log_prob_keep_mask", None) is not None:
        raise U("the fused provider replays a sampling support from its per-token threshold (log_prob_min_keep), not from a [T, V] mask")
    if linear_logp is None:
        from rl_kernel_b200.integrations.common.linear_logp import LinearLogpWrapper

        linear_logp = LinearLogpWrapper(temperature, real, tp_group, tp_rank * weight.shape[0], padded)
    lp = linear_logp(hidden, weight, targets, **({"min_keep": min_keep} if min_keep is not None else {}))
    entropy = None
    if getattr(request, "with_entropy", False):
        with torch.no_grad():                                   # a metric: chunked, without a gradient
            ent = []
            for a in range(0, hidden.shape[0], 1024):
                z = (hidden[a:a + 1024].float() @ weight.float().t()) / temperature
                if tp_world > 1:
                    raise U("the entropy metric over a sharded vocabulary needs the logits provider")
                p = torch.softmax(z[:, :real], -1)
                ent.append(-(p * torch.log(p.clamp_min(1e-30))).sum(-1))
            entropy = torch.cat(ent)
    backend = getattr(linear_logp, "backend_id", type(linear_logp).__name__) if hidden.is_cuda else "reference"
    prov = {"actual_backend": backend, "fallback": False,
            "request": {"hidden_shape": list(hidden.shape), "weight_shape": list(weight.shape), "dtype": str(hidden.dtype).removeprefix("torch."),
                        "real_vocab_size": real, "padded_vocab_size": padded, "tp_rank": tp_rank, "tp_world_size": tp_world,
                        "cp_rank": cp_rank, "cp_world_size": cp_world, "temperature": temperature},
            "execution": {"role": "vime_training_fused_linear_logprob", "strict_backend": True, "logits_materialized": False,
                          "top_p_replay": min_keep is not None},
            "cp_row_ownership": {"cp_rank": cp_rank, "cp_world_size": cp_world, "layout": layout, "local_token_rows": int(hidden.shape[0]),
                                 "cp_is_merge_axis": False}}
    import hashlib
    import json

    cid = hashlib.sha256(json.dumps({k: prov["request"][k] for k in ("real_vocab_size", "padded_vocab_size", "tp_world_size", "temperature",
                                                                    "dtype")}, sort_keys=True).encode()).hexdigest()
    return LinearLogpResult(lp.reshape(-1, 1), entropy, backend, cid, prov)


__all__ = ["LinearLogpProviderUnavailable", "LinearLogpResult", "provider"]
