"""Fixed-order (deterministic) collectives.

Contract shared by every implementation: a sum over ``world`` ranks is the balanced binary tree
``((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7))`` evaluated in fp32 with a rounding to the tensor's dtype at
every node — exactly the tree ``det_gemm`` builds over canonical K chunks, so a row-parallel GEMM
followed by this all-reduce gives the same bits for TP = 1, 2, 4, 8
(reference: fixed_tree_reduce, csrc/cuda/collectives/deterministic_collective.cu:661-695).
All-gather / all-gather-many / broadcast move bits unchanged in rank order.

``TorchDistributedDeterministicCollective`` uses torch.distributed all-gather as the transport and
reduces locally; it runs on Gloo (CPU) and NCCL and is the executable definition the symmetric
memory kernels are tested against (reference: rl_engine/distributed/transports/rccl.py:25-47).
``SymmetricMemoryCollective`` (rl_kernel_b200/distributed/transports/symm.py) is the NVLink path.
"""
from __future__ import annotations

import threading
from typing import Sequence

import torch


class CollectiveTimeout(RuntimeError):
    """A peer did not arrive within the bounded wait; the context stays usable."""


class CollectiveMismatchError(ValueError):
    """The ranks of a group presented different operations, shapes or dtypes for the same collective call.
    Raised on every rank by the host-side check, before anything is launched."""


def balanced_tree_sum(parts: Sequence[torch.Tensor], dtype: torch.dtype | None = None) -> torch.Tensor:
    """Balanced binary tree over a power-of-two number of equally shaped tensors."""
    n = len(parts)
    if n == 0 or n & (n - 1):
        raise ValueError(f"balanced_tree_sum needs a power-of-two number of parts, got {n}")
    dtype = dtype or parts[0].dtype
    level = list(parts)
    while len(level) > 1:
        if dtype.is_floating_point:
            level = [(level[i].float() + level[i + 1].float()).to(dtype) for i in range(0, len(level), 2)]
        else:
            level = [level[i] + level[i + 1] for i in range(0, len(level), 2)]
    return level[0]


def _signature(t: torch.Tensor) -> tuple:
    return (tuple(t.shape), str(t.dtype))


class TorchDistributedDeterministicCollective:
    """all-gather transport + local balanced tree. Works for any backend torch.distributed offers."""

    def __init__(self, group=None, check_signatures: bool = True):
        import torch.distributed as dist

        self._dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world & (self.world - 1):
            raise ValueError(f"world size must be a power of two (1, 2, 4, 8), got {self.world}")
        self._checked: set[tuple] = set()
        self._check = check_signatures
        self._lock = threading.Lock()

    # -- first-use preflight: every rank must present the same (shape, dtype) for an op
    def _preflight(self, op: str, t: torch.Tensor) -> None:
        key = (op,) + _signature(t)
        if not self._check or key in self._checked or self.world == 1:
            return
        sigs = [None] * self.world
        self._dist.all_gather_object(sigs, key, group=self.group)
        if any(s != sigs[0] for s in sigs):
            raise CollectiveMismatchError(f"collective signature mismatch across ranks for {op}: {sigs}")
        self._checked.add(key)

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[...] -> [world, ...] in rank order."""
        if self.world == 1:
            return t.unsqueeze(0)
        with self._lock:
            self._preflight("all_gather", t)
            t = t.contiguous()
            out = torch.empty((self.world,) + tuple(t.shape), dtype=t.dtype, device=t.device)
            self._dist.all_gather_into_tensor(out, t, group=self.group) if t.is_cuda else \
                self._dist.all_gather(list(out.unbind(0)), t, group=self.group)
            return out

    def all_gather_many(self, tensors: Sequence[torch.Tensor]) -> list[torch.Tensor]:
        return [self.all_gather(t) for t in tensors]

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        parts = self.all_gather(t)
        t.copy_(balanced_tree_sum(list(parts.unbind(0)), t.dtype))
        return t

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        return self.all_reduce_(t.clone())

    def all_reduce_int_(self, t: torch.Tensor) -> torch.Tensor:
        """Integer sum: associative, so any order is exact."""
        if self.world > 1:
            self._dist.all_reduce(t, group=self.group)
        return t

    def reduce_scatter(self, t: torch.Tensor) -> torch.Tensor:
        """t [world * n, ...] -> this rank's [n, ...] slice of the tree-reduced tensor."""
        if self.world == 1:
            return t
        n = t.shape[0] // self.world
        full = self.all_reduce(t)
        return full[self.rank * n:(self.rank + 1) * n].contiguous()

    def broadcast_(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        if self.world > 1:
            self._dist.broadcast(t, src=self._dist.get_global_rank(self.group, src) if self.group is not None else src,
                                 group=self.group)
        return t

    def barrier(self) -> None:
        if self.world > 1:
            self._dist.barrier(group=self.group)

    def close(self) -> None:
        pass


_CACHE: dict[tuple, object] = {}
_CACHE_LOCK = threading.Lock()


def create_deterministic_collective(group=None, device: torch.device | str | None = None, *,
                                    prefer_symmetric_memory: bool = True, **kwargs):
    """Pick the implementation for ``group``: symmetric-memory kernels for a CUDA group on one
    node, the torch.distributed transport otherwise (CPU/Gloo, or when peer access is missing)."""
    dev = torch.device(device) if device is not None else None
    if prefer_symmetric_memory and dev is not None and dev.type == "cuda":
        from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

        return SymmetricMemoryCollective(group, dev, **kwargs)
    return TorchDistributedDeterministicCollective(group)


def collective_for_group(group=None, device: torch.device | str | None = None, **kwargs):
    """Process-local cache keyed by (group, device) (reference: collectives.py:785-828)."""
    import torch.distributed as dist

    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    key = (id(group), rank, world, str(device))
    with _CACHE_LOCK:
        if key not in _CACHE:
            _CACHE[key] = create_deterministic_collective(group, device, **kwargs)
        return _CACHE[key]
