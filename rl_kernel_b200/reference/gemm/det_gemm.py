"""Reference for the batch-invariant GEMM contract (csrc/gemm/det_gemm_sm100.cu).

``out = x @ w^T`` where every output ROW is computed by its own matrix-vector product, so a row's
bits cannot depend on how many other rows are in the call, and optional canonical K chunks are
combined by a balanced binary tree with a rounding to the compute dtype at the leaves and at
every node — the same tree the fixed-order collectives continue across tensor-parallel ranks.
(Parity: NativeGemmOp / det_gemm tree of csrc/cuda/gemm/det_gemm_kernel.cu:74-85.)
"""
from __future__ import annotations

import torch


def _rows_matvec(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    # one mv per row: identical call shape for every row -> batch-invariant by construction
    xf, wf = x.float(), w.float()
    if xf.shape[0] == 0:
        return xf.new_zeros(0, wf.shape[0])
    return torch.stack([torch.mv(wf, xf[i]) for i in range(xf.shape[0])])


def tree_reduce(parts: list[torch.Tensor], round_dtype: torch.dtype | None) -> torch.Tensor:
    """Balanced binary tree over ``parts`` (power-of-two count): node = round(a + b)."""
    n = len(parts)
    if n & (n - 1):
        raise ValueError("tree_reduce needs a power-of-two number of parts")
    level = list(parts)
    while len(level) > 1:
        nxt = []
        for i in range(0, len(level), 2):
            s = level[i].float() + level[i + 1].float()
            nxt.append(s.to(round_dtype) if round_dtype is not None else s)
        level = nxt
    return level[0]


def det_gemm_reference(x: torch.Tensor, w: torch.Tensor, *, nchunks: int = 1,
                       out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [M,K] @ w[N,K]^T with ``nchunks`` canonical K chunks (1, 2, 4, 8)."""
    out_dtype = out_dtype or x.dtype
    K = x.shape[1]
    if nchunks == 1:
        return _rows_matvec(x, w).to(out_dtype)
    if K % nchunks:
        raise ValueError("K must be divisible by nchunks")
    kc = K // nchunks
    leaves = [_rows_matvec(x[:, i * kc:(i + 1) * kc], w[:, i * kc:(i + 1) * kc]).to(out_dtype)
              for i in range(nchunks)]
    return tree_reduce(leaves, out_dtype)


class NativeGemmOp:
    """Callable reference op (registry name ``det_gemm``): ``op(a, b)`` = a [M,K] @ b [K,N]."""
    backend_id = "reference"

    def __call__(self, a, b, nchunks: int = 1):
        return det_gemm_reference(a, b.t(), nchunks=nchunks)

    forward = __call__

    def forward_rhs_transposed(self, a, b_t, nchunks: int = 1):
        return det_gemm_reference(a, b_t, nchunks=nchunks)

    def forward_fp32(self, a, b, nchunks: int = 1):
        return det_gemm_reference(a, b.t(), nchunks=nchunks, out_dtype=torch.float32)

    def linear(self, x, w, nchunks: int = 1):
        return det_gemm_reference(x.reshape(-1, x.shape[-1]), w, nchunks=nchunks).reshape(*x.shape[:-1], w.shape[0])
