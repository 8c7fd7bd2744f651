"""Reading the structural request objects the orchestrator hands to a provider.  Nothing of the orchestrator is
imported: a request is anything with the named attributes."""
from __future__ import annotations

from collections.abc import Mapping
from typing import Any

import torch


def metadata(request: Any) -> Mapping[str, Any]:
    md = getattr(request, "metadata", None)
    if md is None:
        return {}
    if not isinstance(md, Mapping):
        raise TypeError("request.metadata must be a mapping")
    return md


def request_tensor(request: Any, name: str, unavailable: type[Exception]) -> torch.Tensor:
    t = getattr(request, name, None)
    if not isinstance(t, torch.Tensor):
        raise unavailable(f"request.{name} must be a tensor")
    return t


def positive_int(value: Any, name: str, unavailable: type[Exception]) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise unavailable(f"{name} must be a positive integer; got {value!r}")
    return value


def tp_coordinates(tp_group: Any) -> tuple[int, int]:
    """(rank, world) of a tensor-parallel group: None = one rank; a process group; or an object with rank / world."""
    if tp_group is None:
        return 0, 1
    if hasattr(tp_group, "rank") and hasattr(tp_group, "world") and not callable(getattr(tp_group, "rank")):
        return int(tp_group.rank), int(tp_group.world)
    import torch.distributed as dist

    return dist.get_rank(group=tp_group), dist.get_world_size(group=tp_group)


def cp_coordinates(request: Any, unavailable: type[Exception]) -> tuple[int, int, str]:
    cp = getattr(request, "context_parallel", None)
    if cp is None:
        return 0, 1, "single"
    world = positive_int(getattr(cp, "world_size", None), "context_parallel.world_size", unavailable)
    rank = getattr(cp, "rank", None)
    if isinstance(rank, bool) or not isinstance(rank, int) or not 0 <= rank < world:
        raise unavailable(f"context_parallel.rank={rank!r} is invalid for CP={world}")
    layout = getattr(cp, "layout", None)
    if layout not in ({"single"} if world == 1 else {"zigzag", "allgather", "contiguous"}):
        raise unavailable("context_parallel layout does not describe local CP token ownership")
    return rank, world, layout
