"""Shared machinery of contract dataclasses: canonical JSON and SHA-256 fingerprints."""
from __future__ import annotations

import dataclasses
import enum
import hashlib
import json


def _plain(v):
    if dataclasses.is_dataclass(v):
        return {f.name: _plain(getattr(v, f.name)) for f in dataclasses.fields(v)}
    if isinstance(v, enum.Enum):
        return v.value
    if isinstance(v, (list, tuple)):
        return [_plain(x) for x in v]
    if isinstance(v, dict):
        return {str(k): _plain(x) for k, x in sorted(v.items())}
    return v


class ContractBase:
    def to_dict(self) -> dict:
        return _plain(self)

    def canonical_json(self) -> str:
        return json.dumps(self.to_dict(), sort_keys=True, separators=(",", ":"))

    def fingerprint(self) -> str:
        return hashlib.sha256(self.canonical_json().encode()).hexdigest()


def assert_same_across_ranks(fingerprint: str, group=None, what: str = "contract") -> None:
    """Preflight run before the first collective of an operator: all ranks must hold the same
    contract (parity: vocab_parallel_logp.py:165-191, distributed_grpo_loss.py:133-175)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    got = [None] * dist.get_world_size(group)
    dist.all_gather_object(got, fingerprint, group=group)
    if any(g != got[0] for g in got):
        raise RuntimeError(f"{what} fingerprint differs across ranks: {got}")
