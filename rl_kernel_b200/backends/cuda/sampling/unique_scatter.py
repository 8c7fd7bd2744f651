"""Copy-only scatters for indices that are unique by construction
(parity: rl_engine/backends/cuda/sampling/unique_scatter.py:49-67; the reference uses two Triton kernels).

``copy_unique_rows_`` runs the row gather/scatter kernel of csrc/packing/pack.cu when rows are a multiple of 16
bytes; ``scatter_permuted_columns`` inverts a complete per-row argsort permutation -- every output element is written
exactly once, so torch's scatter is already deterministic and no collision sort is needed.  The sm_100a sampler
never sorts (it works from a keep threshold), so these exist for callers that bring a sorted layout with them."""
from __future__ import annotations

import torch


def scatter_permuted_columns(values: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    if values.ndim != 2 or values.shape != indices.shape:
        raise ValueError("values and indices must be 2-D with equal shapes")
    out = torch.empty_like(values)
    out.scatter_(1, indices.long(), values)
    return out


def copy_unique_rows_(output: torch.Tensor, indices: torch.Tensor, values: torch.Tensor) -> torch.Tensor:
    if values.ndim != 2 or output.ndim != 2 or values.shape != (indices.numel(), output.size(1)):
        raise ValueError("values must be [len(indices), output columns]")
    row_bytes = output.size(1) * output.element_size()
    if output.is_cuda and row_bytes % 16 == 0 and values.stride(1) == 1 and output.stride(1) == 1 and values.numel():
        from rl_kernel_b200.ops.packing import _move as _move_rows

        _move_rows(values, indices.reshape(-1).long().contiguous(), output, True)
    elif values.numel():
        output[indices.reshape(-1).long()] = values
    return output
