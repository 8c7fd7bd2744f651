"""Selected log-prob from logits with output-buffer and row-index variants
(parity: FusedLogpSM90Op / FusedLogpGenericOp / DeterministicLogpCUDAOp,
rl_engine/backends/cuda/logprob/logp.py:58-328).

The reference keeps a fast fused kernel, an "online" two-pass variant and a deterministic one.
The tile contract here is deterministic and single-pass, so every variant name resolves to the
same kernels; ``*_out`` writes into a caller buffer and ``indexed_*`` scores
``logits[row_indices[i]]`` against ``token_ids[i]`` without gathering the logits.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.ops.logprob import logp_from_logits, logp_from_logits_indexed


class FusedLogpGenericOp:
    is_fused_logp = True
    is_batch_invariant = True
    backward_impl = "native"
    backend_id = "b200"

    def __init__(self):
        pass

    @staticmethod
    def _prepare_inputs(logits: torch.Tensor, token_ids: torch.Tensor):
        if logits.shape[:-1] != token_ids.shape:
            raise ValueError(f"logits {tuple(logits.shape)} and token_ids {tuple(token_ids.shape)} do not align")
        return logits.reshape(-1, logits.shape[-1]), token_ids.reshape(-1).to(logits.device), token_ids.shape

    @staticmethod
    def _prepare_output(output: torch.Tensor, orig_shape) -> torch.Tensor:
        if output.dtype != torch.float32 or output.numel() != int(torch.Size(orig_shape).numel()):
            raise ValueError("output must be fp32 with one element per token")
        return output.view(-1)

    @staticmethod
    def _prepare_indices(row_indices: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        return row_indices.reshape(-1).to(device=logits.device, dtype=torch.long).contiguous()

    def apply(self, logits, token_ids):
        """Differentiable in ``logits``."""
        return logp_from_logits(logits, token_ids)

    def apply_fp32(self, logits, token_ids):
        with torch.no_grad():
            return logp_from_logits(logits, token_ids)

    __call__ = apply

    def out(self, logits, token_ids, output):
        lg, ids, shape = self._prepare_inputs(logits, token_ids)
        self._prepare_output(output, shape).copy_(self.apply_fp32(lg, ids))
        return output.view(shape)

    def indexed_fp32(self, logits, token_ids, row_indices):
        lg = logits.reshape(-1, logits.shape[-1])
        idx = self._prepare_indices(row_indices, lg)
        with torch.no_grad():
            return logp_from_logits_indexed(lg, token_ids.reshape(-1).to(lg.device), idx).view(token_ids.shape)

    def indexed_out(self, logits, token_ids, row_indices, output):
        self._prepare_output(output, token_ids.shape).copy_(self.indexed_fp32(logits, token_ids, row_indices).reshape(-1))
        return output.view(token_ids.shape)

    # the "online" names of the reference: same single-pass tile kernels
    def online_out(self, logits, token_ids, output):
        return self.out(logits, token_ids, output)

    def online_fp32(self, logits, token_ids):
        return self.apply_fp32(logits, token_ids)

    def online_indexed_out(self, logits, token_ids, row_indices, output):
        return self.indexed_out(logits, token_ids, row_indices, output)

    def online_indexed_fp32(self, logits, token_ids, row_indices):
        return self.indexed_fp32(logits, token_ids, row_indices)


class FusedLogpSM100Op(FusedLogpGenericOp):
    backend_id = "b200"


class DeterministicLogpCUDAOp(FusedLogpGenericOp):
    """Inference-only spelling of the reference (``__call__`` returns a detached fp32 result)."""

    def __call__(self, logits, token_ids):
        return self.apply_fp32(logits, token_ids)

    def apply(self, logits, token_ids):
        return self.apply_fp32(logits, token_ids)


FusedLogpSM90Op = FusedLogpSM100Op
