"""Canonical (layout-invariant) parameter gradients under context parallelism
(parity: rl_engine/distributed/algorithms/canonical_cp.py:12-330).

Context parallelism gives every rank a different subset of each sequence's tokens, so a weight
gradient summed first over a rank's tokens and then over ranks rounds differently from the
single-GPU sum over tokens in logical order.  The cure is the same as the reference's: bring the
per-token operands (x, dy) of every parameter use into LOGICAL TOKEN ORDER before the reduction.

What differs is who then does the work.  The reference gathers on every CP rank, computes the
complete gradient cp times and lets only rank 0 contribute.  Here the gradient's OUTPUT ROWS are
split over the CP ranks: rank c computes rows [c N / cp, (c+1) N / cp) of dW = dY^T X over ALL
tokens -- 1/cp of the GEMM, no duplicate work -- and leaves the other rows zero, so the
framework's ordinary sum over the CP group (or an all-gather of the slices) assembles the full
matrix with exactly one non-zero contributor per element, which is exact in any order.  Row slices
of a GEMM whose every output element is one ordered fp32 accumulation over K equal the
corresponding rows of the unsliced GEMM bit for bit.

Pieces:

``packed_gather_indices`` / ``uniform_gather_indices``   rank-major gathered rows -> logical order
``CPLayout``                                            the order tensor + groups; ``gather_many``
``weight_gradient``                                     row-sliced canonical dW (optionally in K-chunks)
``row_parameter_gradient``                              gains / embeddings: one owner rank computes
``CPRowLinear`` / ``CPRMSNorm`` / ``CPEmbedding``       autograd functions for framework bindings
``CanonicalLossGradient``                               removes a framework's CP loss multiplier
``install``                                             binds the above to Megatron-style classes
"""
from __future__ import annotations

from contextvars import ContextVar
from dataclasses import dataclass
from functools import wraps
from typing import Any, Sequence

import torch

_ACTIVE: ContextVar = ContextVar("rl_kernel_cp_gradient_layout", default=None)


def current_layout():
    return _ACTIVE.get()


def bind_layout(function, layout):
    """Keep the forward's token layout during activation recomputation (checkpointed backward)."""

    @wraps(function)
    def wrapped(*args, **kwargs):
        token = _ACTIVE.set(layout)
        try:
            return function(*args, **kwargs)
        finally:
            _ACTIVE.reset(token)

    return wrapped


def zigzag_owner(pos: int, length: int, cp_world: int) -> tuple[int, int, int]:
    """(rank, index inside the rank's shard of this sequence, shard width) of token ``pos`` of a sequence of
    ``length`` tokens cut into 2 cp blocks of equal width (the last may be short): rank r holds blocks r and 2cp-1-r."""
    width = (length + 2 * cp_world - 1) // (2 * cp_world)
    block, within = divmod(pos, width)
    rank = block if block < cp_world else 2 * cp_world - 1 - block
    return rank, within + (width if block >= cp_world else 0), width


def packed_gather_indices(lengths: Sequence[int], local_rows: int, cp_world: int) -> list[int]:
    """For a packed batch (sequences back to back, each zigzag-split and padded to 2 cp equal blocks): the row of
    the rank-major gathered tensor [cp * local_rows, ...] that holds each real token, in sample / position order."""
    out: list[int] = []
    offset = 0
    for length in lengths:
        if cp_world == 1:
            out.extend(range(offset, offset + length))
            offset += length
            continue
        width = 0
        for pos in range(length):
            rank, local, width = zigzag_owner(pos, length, cp_world)
            out.append(rank * local_rows + offset + local)
        offset += 2 * width
    if offset > local_rows:
        raise ValueError("canonical CP layout exceeds packed token rows")
    return out


def uniform_gather_indices(nseq: int, seq_len: int, cp_world: int, layout: str = "zigzag") -> torch.Tensor:
    """The same for ``nseq`` sequences of equal length whose shards are stored sequence-major ([nseq, S / cp] rows per
    rank, positions ascending inside a rank): index [nseq * seq_len] into the gathered [cp * nseq * S / cp] rows."""
    if cp_world == 1:
        return torch.arange(nseq * seq_len)
    if layout == "zigzag":
        if seq_len % (2 * cp_world):
            raise ValueError("zigzag needs a sequence length divisible by 2 * cp")
        chunk = seq_len // (2 * cp_world)
        pos = torch.arange(seq_len)
        block = pos // chunk
        rank = torch.where(block < cp_world, block, 2 * cp_world - 1 - block)
        local = pos % chunk + torch.where(block >= cp_world, chunk, 0)
    elif layout == "contiguous":
        if seq_len % cp_world:
            raise ValueError("contiguous needs a sequence length divisible by cp")
        per = seq_len // cp_world
        pos = torch.arange(seq_len)
        rank, local = pos // per, pos % per
    else:
        raise ValueError(layout)
    s_local = seq_len // cp_world
    b = torch.arange(nseq)[:, None]
    return (rank[None, :] * (nseq * s_local) + b * s_local + local[None, :]).reshape(-1)


@dataclass
class CPLayout:
    order: torch.Tensor                 # logical token t lives in row order[t] of the rank-major gathered tensor
    local_rows: int
    cp_world: int
    cp_group: Any                       # a torch process group, or a deterministic collective (has all_gather / world)
    tp_world: int = 1
    tp_group: Any = None
    cp_rank: int = 0
    tp_rank: int = 0

    def ordered(self, value: torch.Tensor) -> torch.Tensor:
        return value.index_select(0, self.order)

    def _collective(self):
        if hasattr(self.cp_group, "all_gather") and hasattr(self.cp_group, "world"):
            return self.cp_group
        from rl_kernel_b200.distributed.algorithms.collectives import collective_for_group

        return collective_for_group(self.cp_group)

    def gather_many(self, *values: torch.Tensor) -> tuple[torch.Tensor, ...]:
        """Every tensor [local_rows, ...] -> all ranks' rows in logical token order."""
        values = tuple(v.contiguous() for v in values)
        if any(v.size(0) != self.local_rows for v in values):
            raise ValueError("canonical CP tensors must start with packed token rows")
        if self.cp_world > 1:
            coll = self._collective()
            values = tuple(coll.all_gather(v).reshape(-1, *v.shape[1:]) for v in values)
        return tuple(self.ordered(v) for v in values)

    def row_slice(self, n_rows: int, align: int = 8) -> tuple[int, int]:
        """The output rows of a gradient this rank computes: equal contiguous slices, boundaries on ``align`` rows."""
        per = -(-n_rows // self.cp_world)
        per = -(-per // align) * align
        lo = min(n_rows, self.cp_rank * per)
        return lo, min(n_rows, lo + per)


def replica_parameter_gradient(gradient: torch.Tensor, replicas: int, rank: int) -> torch.Tensor:
    """For frameworks that AVERAGE gradients over the CP group: a complete gradient held by one replica only, scaled so
    that the average gives it back exactly (the others contribute zeros).  The input is never modified."""
    if rank != 0:
        return torch.zeros_like(gradient)
    return gradient if replicas == 1 else gradient * replicas


def sliced_parameter_gradient(gradient_rows: torch.Tensor, n_rows: int, lo: int, hi: int, *, average_over: int = 1
                              ) -> torch.Tensor:
    """This rank's rows placed into a zero matrix of the full shape (times ``average_over`` when the framework
    averages): summing over the CP group assembles the full gradient with one non-zero contributor per element."""
    full = gradient_rows.new_zeros((n_rows,) + tuple(gradient_rows.shape[1:]))
    full[lo:hi] = gradient_rows if average_over == 1 else gradient_rows * average_over
    return full


class CanonicalLossGradient(torch.autograd.Function):
    """Identity on the loss; divides the incoming gradient by ``cp_world`` so that a framework's CP multiplier is
    removed before any low-precision derivative is formed."""

    @staticmethod
    def forward(ctx, loss, cp_world):
        ctx.cp_world = cp_world
        return loss.clone()                       # frameworks rescale this scalar in place afterwards

    @staticmethod
    def backward(ctx, gradient):
        return gradient / ctx.cp_world, None


def _dw(dy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """dW [N, K] = dY [T, N]^T @ X [T, K], tokens reduced in ascending order."""
    from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_db

    return det_gemm_db(dy.contiguous(), x.contiguous())


def weight_gradient(x: torch.Tensor, dy: torch.Tensor, layout: CPLayout | None, chunks: int = 1, column: bool = True,
                    *, framework_averages: bool = False) -> torch.Tensor:
    """Canonical dW [N, K] of y = x W^T from this rank's token rows ``x`` [T_local, K], ``dy`` [T_local, N].

    Without a layout this is the plain deterministic weight gradient.  With one, (x, dy) are gathered into logical
    token order and this rank computes its row slice over all tokens; the result has the full shape with the other
    rows zero (see the module text).  ``chunks`` > 1 evaluates the gradient per canonical TP shard (``column``:
    shards split N, otherwise K) -- the shapes a TP-sharded run would see -- and concatenates."""
    if layout is None or layout.cp_world == 1:
        if layout is not None:
            x, dy = layout.gather_many(x, dy)
        return _chunked_dw(x, dy, chunks, column)
    xg, dyg = layout.gather_many(x, dy)
    n = dyg.shape[1]
    lo, hi = layout.row_slice(n)
    rows = _chunked_dw(xg, dyg[:, lo:hi], 1, column) if hi > lo else dyg.new_zeros(0, xg.shape[1])
    return sliced_parameter_gradient(rows, n, lo, hi, average_over=layout.cp_world if framework_averages else 1)


def _chunked_dw(x, dy, chunks: int, column: bool) -> torch.Tensor:
    if chunks == 1:
        return _dw(dy, x)
    source = dy if column else x
    if source.size(-1) % chunks:
        raise ValueError("canonical parameter shard does not divide TP")
    width = source.size(-1) // chunks
    parts = [_dw(dy.narrow(1, i * width, width) if column else dy, x if column else x.narrow(1, i * width, width))
             for i in range(chunks)]
    return torch.cat(parts, dim=0 if column else 1)


def row_parameter_gradient(fn, layout: CPLayout | None, *operands: torch.Tensor, owner_tp_rank: int | None = None,
                           framework_averages: bool = False) -> torch.Tensor:
    """Gradients that are reductions over token rows but not GEMMs (norm gains, embedding rows): the operands are
    gathered into logical order and ONE owner rank evaluates ``fn(*gathered)``; every other rank returns zeros."""
    if layout is None:
        return fn(*operands)
    gathered = layout.gather_many(*operands)
    owner = layout.cp_rank == 0 and (owner_tp_rank is None or layout.tp_rank == owner_tp_rank)
    value = fn(*gathered)
    if not owner:
        return torch.zeros_like(value)
    return value * layout.cp_world if framework_averages and layout.cp_world > 1 else value


class CPRowLinear(torch.autograd.Function):
    """y = linear(x, W) whose weight gradient is canonical under the active layout."""

    @staticmethod
    def forward(ctx, x, weight, linear, layout):
        ctx.save_for_backward(x, weight)
        ctx.layout = layout
        return linear(x, weight)

    @staticmethod
    def backward(ctx, dy):
        from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_da

        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = det_gemm_da(dy2, w).reshape(x.shape) if ctx.needs_input_grad[0] else None
        dw = weight_gradient(x2, dy2, ctx.layout) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None


def _rms(x, weight, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


class CPRMSNorm(torch.autograd.Function):
    """RMSNorm whose gain gradient is the logical-order row sum.  ``sharded_heads``: the gain is shared by heads that
    are split over TP (Q/K norms); the heads are gathered over TP as well and only TP rank 0 contributes."""

    @staticmethod
    def forward(ctx, x, weight, eps, layout, sharded_heads):
        ctx.save_for_backward(x, weight)
        ctx.eps, ctx.layout, ctx.sharded_heads = eps, layout, sharded_heads
        return _rms(x, weight, eps)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        eps, layout = ctx.eps, ctx.layout
        with torch.enable_grad():
            local = x.detach().requires_grad_(True)
            (dx,) = torch.autograd.grad(_rms(local, weight.detach(), eps), local, dy)

        def gain_grad(full_x, full_dy):
            if ctx.sharded_heads and layout.tp_world > 1:
                import torch.distributed as dist

                parts = []
                for v in (full_x, full_dy):
                    pieces = [torch.empty_like(v) for _ in range(layout.tp_world)]
                    dist.all_gather(pieces, v.contiguous(), group=layout.tp_group)
                    parts.append(torch.cat(pieces, dim=-2))            # heads in TP-rank order
                full_x, full_dy = parts
            xf, gf = full_x.float(), full_dy.float()
            rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
            rows = (gf * xf * rstd).reshape(-1, xf.shape[-1])
            acc = torch.zeros(xf.shape[-1], dtype=torch.float32, device=x.device)
            for r in range(rows.shape[0]):                             # ascending logical row order
                acc = acc + rows[r]
            return acc.to(weight.dtype)

        dw = row_parameter_gradient(gain_grad, layout, x, dy, owner_tp_rank=0 if ctx.sharded_heads else None)
        return dx, dw, None, None, None


def rms_norm(x, weight, eps, sharded_heads: bool = False):
    layout = current_layout()
    if layout is None or not torch.is_grad_enabled():
        return _rms(x, weight, eps)
    return CPRMSNorm.apply(x, weight, eps, layout, sharded_heads)


class CPEmbedding(torch.autograd.Function):
    """Vocabulary-sharded embedding gather whose weight gradient adds the occurrences of every id in logical token
    order."""

    @staticmethod
    def forward(ctx, ids, weight, start, layout):
        ctx.save_for_backward(ids)
        ctx.shape, ctx.dtype, ctx.start, ctx.layout = weight.shape, weight.dtype, start, layout
        local = ids - start
        valid = (local >= 0) & (local < weight.size(0))
        out = torch.nn.functional.embedding(local.masked_fill(~valid, 0), weight)
        return out.masked_fill(~valid.unsqueeze(-1), 0)

    @staticmethod
    def backward(ctx, dy):
        from rl_kernel_b200.reference.embedding.embedding import embedding_grad_weight_reference

        (ids,) = ctx.saved_tensors

        def rows_grad(all_ids, all_dy):
            return embedding_grad_weight_reference(all_ids.flatten() - ctx.start, all_dy.float(), ctx.shape[0]).to(ctx.dtype)

        dw = row_parameter_gradient(rows_grad, ctx.layout, ids.reshape(-1, 1), dy.reshape(-1, dy.size(-1)))
        return None, dw, None, None


def install(*, model_cls=None, embedding_cls=None, checkpoint_function_cls=None, loss_module=None, parallel_state=None,
            lengths_of=None) -> bool:
    """Bind the canonical gradients to a Megatron-style stack.  Every class is passed in (stand-ins work); with no
    arguments the real Megatron / vime classes are imported.

    * ``model_cls.forward`` opens a ``CPLayout`` for the packed batch (sequence lengths from
      ``lengths_of(packed_seq_params)``) for the duration of the call,
    * ``checkpoint_function_cls.forward`` re-binds that layout when a checkpointed function is recomputed,
    * ``embedding_cls.forward`` goes through ``CPEmbedding``,
    * ``loss_module.loss_function`` is wrapped with ``CanonicalLossGradient``.
    """
    if model_cls is None:
        from megatron.core import parallel_state  # type: ignore  # noqa: PLC0415
        from megatron.core.models.gpt.gpt_model import GPTModel as model_cls  # type: ignore  # noqa: PLC0415
        from megatron.core.tensor_parallel.layers import VocabParallelEmbedding as embedding_cls  # type: ignore  # noqa: PLC0415
        from megatron.core.tensor_parallel.random import CheckpointFunction as checkpoint_function_cls  # type: ignore  # noqa: PLC0415
    if getattr(model_cls, "_rlk_cp_parameter_grads", False):
        return False
    mpu = parallel_state
    lengths_of = lengths_of or (lambda packed: getattr(packed, "_rlk_true_lengths", None))
    if loss_module is not None:
        original_loss = loss_module.loss_function

        @wraps(original_loss)
        def loss_function(*args, **kwargs):
            value, normalizer, metrics = original_loss(*args, **kwargs)
            return CanonicalLossGradient.apply(value, mpu.get_context_parallel_world_size()), normalizer, metrics

        loss_module.loss_function = loss_function
    if checkpoint_function_cls is not None:
        checkpoint_forward = checkpoint_function_cls.forward

        @wraps(checkpoint_forward)
        def checkpoint(ctx, function, distribute_saved_activations, *args):
            layout = current_layout()
            if layout is not None:
                function = bind_layout(function, layout)
            return checkpoint_forward(ctx, function, distribute_saved_activations, *args)

        checkpoint_function_cls.forward = staticmethod(checkpoint)
    original_forward = model_cls.forward

    @wraps(original_forward)
    def forward(self, *args, **kwargs):
        packed = kwargs.get("packed_seq_params")
        lengths = lengths_of(packed) if packed is not None else None
        if lengths is None or not torch.is_grad_enabled():
            return original_forward(self, *args, **kwargs)
        ids = kwargs.get("input_ids", args[0] if args else None)
        if ids.size(0) != 1:
            raise ValueError("canonical packed CP backward requires batch dimension one")
        cp = mpu.get_context_parallel_world_size()
        layout = CPLayout(torch.tensor(packed_gather_indices(lengths, ids.size(1), cp), device=ids.device), ids.size(1), cp,
                          mpu.get_context_parallel_group(), mpu.get_tensor_model_parallel_world_size(),
                          mpu.get_tensor_model_parallel_group(), mpu.get_context_parallel_rank(),
                          mpu.get_tensor_model_parallel_rank())
        token = _ACTIVE.set(layout)
        try:
            return original_forward(self, *args, **kwargs)
        finally:
            _ACTIVE.reset(token)

    model_cls.forward = forward
    if embedding_cls is not None:
        original_embedding = embedding_cls.forward

        @wraps(original_embedding)
        def embedding(self, ids):
            layout = current_layout()
            if layout is None:
                return original_embedding(self, ids)
            if getattr(self, "reduce_scatter_embeddings", False):
                raise ValueError("canonical CP embedding does not support sequence parallelism")
            local = CPEmbedding.apply(ids, self.weight, self.vocab_start_index, layout)
            reduce = getattr(self, "_rlk_tp_reduce", None)
            return reduce(local) if reduce is not None else local

        embedding_cls.forward = embedding
    model_cls._rlk_cp_parameter_grads = True
    return True


__all__ = ["CPEmbedding", "CPLayout", "CPRMSNorm", "CPRowLinear", "CanonicalLossGradient", "bind_layout", "current_layout",
           "install", "packed_gather_indices", "replica_parameter_gradient", "rms_norm", "row_parameter_gradient",
           "sliced_parameter_gradient", "uniform_gather_indices", "weight_gradient", "zigzag_owner"]
