"""Deterministic inputs of the operator validation harness (parity: rl_engine/validation/operators/
operator_inputs.py:27-880).

Every input value belongs to a *logical token* ``(sample_id, position)`` and is a pure function of
(seed, sample_id, position, column): the same token carries the same numbers whatever batch, order,
chunk or padding it is placed in.  Values are drawn on the CPU (one generator per sample, seeded
from a stable hash of the sample id) and moved to the target device, so CPU and CUDA runs see the
same bits.  Padding slots get a *filler* row of large, distinctive values: an operator that lets
padding leak into real tokens fails invariance loudly instead of by a rounding error.
"""
from __future__ import annotations

import hashlib

import torch

from rl_kernel_b200.config.workload import LogicalBatch

DEFAULT_RMS_EPS = 1e-6
DEFAULT_ROPE_THETA = 1_000_000.0
Key = tuple[str, int]


def stable_seed(*parts) -> int:
    """31-bit seed from arbitrary printable parts; independent of PYTHONHASHSEED."""
    h = hashlib.sha256("\x1f".join(str(p) for p in parts).encode()).digest()
    return int.from_bytes(h[:4], "little") & 0x7FFFFFFF


def randn(shape, device, dtype, seed: int, scale: float = 1.0) -> torch.Tensor:
    g = torch.Generator().manual_seed(int(seed) & 0x7FFFFFFF)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(device)


def token_table(batch: LogicalBatch, width: int, device, dtype, seed: int, scale: float = 1.0) -> dict[Key, torch.Tensor]:
    """One [width] row per logical token of ``batch``.  A sample's rows come from a generator seeded by
    (seed, sample_id, width) and are drawn position by position, so a sample's values do not depend on
    which other samples are in the batch."""
    table: dict[Key, torch.Tensor] = {}
    for s in batch.samples:
        rows = randn((s.seq_len, width), device, dtype, stable_seed("tok", seed, s.sample_id, width), scale)
        for p in range(s.seq_len):
            table[(s.sample_id, p)] = rows[p]
    return table


def filler_row(width: int, device, dtype, seed: int) -> torch.Tensor:
    """Row stored in padding slots: finite but far outside the data's range."""
    return (randn((width,), device, torch.float32, stable_seed("pad", seed, width)) * 37.0 + 11.0).to(dtype)


def shared_weight(spec, device, dtype, seed: int) -> torch.Tensor | None:
    """The parameter an operator shares between tokens: a gain for norms, a [N, K] matrix for GEMM-shaped operators."""
    p = spec.params
    if spec.name in ("rms_norm", "qk_norm"):
        return (1.0 + 0.1 * randn((p["width"],), device, torch.float32, stable_seed("gain", seed, spec.name))).to(dtype)
    if "out_features" in p:
        return randn((p["out_features"], p["width"]), device, dtype, stable_seed("w", seed, spec.name), p["width"] ** -0.5)
    return None


def grad_rows(keys, out: torch.Tensor, seed: int, batch: LogicalBatch) -> torch.Tensor:
    """Upstream gradient for ``out`` [rows, ...]: a per-token value for real rows, exact zero for padding rows."""
    flat = out.reshape(out.shape[0], -1)
    table = _grad_table(batch, flat.shape[1], str(out.device), out.dtype, seed)
    zero = torch.zeros(flat.shape[1], device=out.device, dtype=out.dtype)
    return torch.stack([table[k] if k is not None else zero for k in keys]).view_as(out)


_GRAD_TABLES: dict = {}


def _grad_table(batch, width, device, dtype, seed):
    key = (batch.workload_id, batch.seed, tuple(s.sample_id for s in sorted(batch.samples, key=lambda s: s.sample_id)), width,
           device, dtype, seed)
    if key not in _GRAD_TABLES:
        if len(_GRAD_TABLES) > 64:
            _GRAD_TABLES.clear()
        _GRAD_TABLES[key] = token_table(batch, width, device, dtype, stable_seed("gout", seed))
    return _GRAD_TABLES[key]


def logical_stack(table: dict[Key, torch.Tensor], keys) -> torch.Tensor:
    return torch.stack([table[k] for k in keys])


__all__ = ["DEFAULT_RMS_EPS", "DEFAULT_ROPE_THETA", "filler_row", "grad_rows", "logical_stack", "randn", "shared_weight",
           "stable_seed", "token_table"]
