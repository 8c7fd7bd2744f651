"""Selected-log-prob provider for the orchestrator's Megatron backend (parity: rl_engine/integrations/orchestrators/vime/
providers/logp.py:34-261).

The request carries this rank's ``logits`` [T, V_local] (its CP token rows, its TP vocabulary columns), ``target_ids`` [T],
the TP group and ``metadata`` (real / padded vocabulary size).  The provider owns the vocabulary reduction only: 128-id
tiles merged in ascending order over the TP group, on the sm_100a tile-statistics kernels for CUDA bf16 logits and on the
PyTorch reference otherwise.  CP rank and layout are row-ownership facts that are validated and recorded, never a merge
axis.  A sampler's top-p / top-k support arrives as ``log_prob_keep_mask`` [T, V_local]: ids outside it count as -inf,
which the tile contract handles exactly (a masked id adds +0 to its tile's sum)."""
from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any

import torch

from rl_kernel_b200.contracts.operators.logprob import LogprobContract, LogprobDType, LogprobRole, MaskSpec, ReductionSpec, ShardingSpec
from rl_kernel_b200.integrations.orchestrators.vime.providers._request import (cp_coordinates, metadata, positive_int, request_tensor,
                                                                               tp_coordinates)

_DTYPES = {torch.bfloat16: LogprobDType.BF16, torch.float16: LogprobDType.FP16, torch.float32: LogprobDType.FP32}


class SelectedLogprobProviderUnavailable(RuntimeError):
    """Asks the orchestrator for its own provider in ``auto`` mode.  The orchestrator recognises the marker attribute; it
    does not import this class."""
    selected_logprob_provider_unavailable = True


@dataclass(frozen=True)
class ProviderResult:
    selected_logprobs: torch.Tensor           # [T, 1]
    entropy: torch.Tensor | None
    backend_id: str
    contract_id: str
    provenance: Mapping[str, Any]


def _contract_for_request(request: Any) -> LogprobContract:
    U = SelectedLogprobProviderUnavailable
    logits, targets = request_tensor(request, "logits", U), request_tensor(request, "target_ids", U)
    md = metadata(request)
    if logits.ndim != 2 or targets.shape != (logits.shape[0],):
        raise U("request must contain local [T, V] logits and aligned [T] targets")
    if logits.dtype not in _DTYPES:
        raise U(f"unsupported logit dtype {logits.dtype}")
    if targets.device != logits.device:
        raise U("target_ids must share the local logits' device")
    cp_rank, cp_world, _ = cp_coordinates(request, U)
    tp_rank, tp_world = tp_coordinates(getattr(request, "tensor_parallel_group", None))
    for key, got in (("tp_rank", tp_rank), ("tp_world_size", tp_world)):
        if md.get(key) is not None and md[key] != got:
            raise U(f"metadata {key}={md[key]} disagrees with the TP group ({got})")
    real = positive_int(md.get("real_vocab_size"), "real_vocab_size", U)
    padded = positive_int(md.get("padded_vocab_size"), "padded_vocab_size", U)
    if logits.shape[1] * tp_world != padded:
        raise U(f"local vocabulary width and TP group do not cover padded_vocab_size: {logits.shape[1]} * {tp_world} != {padded}")
    if real > padded:
        raise U("real_vocab_size must not exceed padded_vocab_size")
    V = logits.shape[1]
    return LogprobContract(role=LogprobRole.TRAIN, dtype=_DTYPES[logits.dtype], mask=MaskSpec.all_active(logits.shape[0]),
                           sharding=ShardingSpec(tp_rank=tp_rank, tp_world_size=tp_world,
                                                 vocab_shard_bounds=tuple((r * V, (r + 1) * V) for r in range(tp_world)),
                                                 real_vocab_size=real, padded_vocab_size=padded, cp_rank=cp_rank, cp_world_size=cp_world),
                           reduction=ReductionSpec())


def provider(request: Any) -> ProviderResult:
    contract = _contract_for_request(request)
    logits = request.logits
    keep = getattr(request, "log_prob_keep_mask", None)
    if keep is not None:
        if keep.shape != logits.shape or keep.dtype != torch.bool:
            raise SelectedLogprobProviderUnavailable("log_prob_keep_mask must be a bool mask of the local logits' shape")
        logits = logits.masked_fill(~keep, float("-inf"))
    if logits.is_cuda:
        from rl_kernel_b200.backends.cuda.logprob.vocab_parallel_logp import CudaVocabParallelLogprobOp as Op
    else:
        from rl_kernel_b200.reference.logprob.vocab_parallel_logp import VocabParallelLogprobOp as Op
    op = Op()
    tp_group = getattr(request, "tensor_parallel_group", None)
    tiles = metadata(request).get("num_vocab_tiles")
    if getattr(request, "with_entropy", False):
        lp, _lse, entropy = op.apply_with_entropy(logits, request.target_ids, contract=contract, tp_group=tp_group, num_vocab_tiles=tiles,
                                                  with_entropy_grad=bool(getattr(request, "with_entropy_grad", False)))
    else:
        lp, _lse = op.apply(logits, request.target_ids, contract=contract, tp_group=tp_group, num_vocab_tiles=tiles)
        entropy = None
    sh = contract.sharding
    prov = {"actual_backend": getattr(op, "backend_id", type(op).__name__), "route": getattr(op, "last_route", "pytorch"), "fallback": False,
            "request": {"logits_shape": list(request.logits.shape), "logits_dtype": str(request.logits.dtype).removeprefix("torch."),
                        "real_vocab_size": sh.real_vocab_size, "padded_vocab_size": sh.padded_vocab_size, "tp_rank": sh.tp_rank,
                        "tp_world_size": sh.tp_world_size, "cp_rank": sh.cp_rank, "cp_world_size": sh.cp_world_size},
            "execution": {"role": "vime_training_selected_logprob", "strict_backend": True, "top_p_replay": keep is not None},
            "cp_row_ownership": {"cp_rank": sh.cp_rank, "cp_world_size": sh.cp_world_size,
                                 "layout": getattr(getattr(request, "context_parallel", None), "layout", "single"),
                                 "local_token_rows": int(request.logits.shape[0]), "cp_is_merge_axis": False}}
    return ProviderResult(lp.unsqueeze(-1), entropy, prov["actual_backend"], contract.cross_rank_fingerprint(), prov)


__all__ = ["ProviderResult", "SelectedLogprobProviderUnavailable", "provider"]
