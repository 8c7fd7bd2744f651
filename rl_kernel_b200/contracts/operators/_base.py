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


# ---------------------------------------------------------------------------------- field validation
def is_plain_int(value) -> bool:
    return isinstance(value, int) and not isinstance(value, bool)


def make_validators(error_type: type):
    """The integer / enum checks every contract module needs, raising that module's error type."""

    def enum_value(enum_type, value, field: str):
        try:
            return enum_type(value)
        except ValueError as exc:
            allowed = ", ".join(str(m.value) for m in enum_type)
            raise error_type(f"{field} must be one of: {allowed}; got {value!r}") from exc

    def positive_int(value, field: str) -> int:
        if not is_plain_int(value) or value <= 0:
            raise error_type(f"{field} must be a positive integer; got {value!r}")
        return value

    def non_negative_int(value, field: str) -> int:
        if not is_plain_int(value) or value < 0:
            raise error_type(f"{field} must be a non-negative integer; got {value!r}")
        return value

    def plain_int(value, field: str) -> int:
        if not is_plain_int(value):
            raise error_type(f"{field} must be an integer; got {value!r}")
        return value

    def integer_tuple(values, field: str) -> tuple:
        try:
            out = tuple(values)
        except TypeError as exc:
            raise error_type(f"{field} must be an iterable of integers") from exc
        for v in out:
            if not is_plain_int(v):
                raise error_type(f"{field} must contain integers only; got {v!r}")
        return out

    def coerce_enums(obj, **fields) -> None:
        """``coerce_enums(self, merge=LogprobMerge, ...)``: replace each field by its enum member."""
        for name, enum_type in fields.items():
            object.__setattr__(obj, name, enum_value(enum_type, getattr(obj, name), name))

    def world_sizes(values, field: str):
        if values is None:
            return None
        try:
            sizes = tuple(values)
        except TypeError as exc:
            raise error_type(f"{field} must be an iterable of integers") from exc
        if not sizes:
            raise error_type(f"{field} must not be empty; use None for unrestricted")
        for v in sizes:
            if not is_plain_int(v) or v <= 0:
                raise error_type(f"{field} must contain positive values; got {v!r}")
        if len(set(sizes)) != len(sizes):
            raise error_type(f"{field} must not contain duplicates")
        return sizes

    return enum_value, positive_int, non_negative_int, plain_int, integer_tuple, coerce_enums, world_sizes


def stable_hash(payload) -> str:
    return hashlib.sha256(json.dumps(payload, sort_keys=True, separators=(",", ":")).encode("utf-8")).hexdigest()
