"""Kernel registry: operator name -> implementation, with capability checks, strict-mode
fail-closed behaviour and provenance (parity: KernelRegistry, rl_engine/runtime/registry.py:
68-1360; the per-platform priority lists collapse to "b200 kernel, else reference").

``kernel_registry.get_op("det_gemm")`` returns a ready operator object; ``last_resolution`` says
which implementation was chosen and why.  In strict mode (RL_KERNEL_MODE=strict) a reference
fallback on a CUDA machine raises instead of being returned.
"""
from __future__ import annotations

import enum
import importlib
import threading
from dataclasses import dataclass

import torch

from rl_kernel_b200.runtime.policy import RLKernelMode, current_mode, route_report


class OpBackend(str, enum.Enum):
    """Dotted paths of every registered implementation."""
    # --- sm_100a kernels
    B200_DET_GEMM = "rl_kernel_b200.ops.gemm.det_gemm.DetGemmOp"
    B200_RMS_NORM = "rl_kernel_b200.ops.norm.canonical_rmsnorm.RMSNormOp"
    B200_ROPE = "rl_kernel_b200.ops.rope.RoPEOp"
    B200_SWIGLU = "rl_kernel_b200.ops.activation.SwiGLUOp"
    B200_EMBEDDING = "rl_kernel_b200.ops.embedding.canonical_embedding.EmbeddingOp"
    B200_LM_HEAD = "rl_kernel_b200.ops.embedding.canonical_lm_head.LMHeadOp"
    B200_ATTENTION = "rl_kernel_b200.ops.attention.attention.AttentionOp"
    B200_FFN = "rl_kernel_b200.ops.ffn.qwen3.Qwen3FFNOp"
    B200_LOGP = "rl_kernel_b200.ops.logprob.BatchInvariantLogpOp"
    B200_LINEAR_LOGP = "rl_kernel_b200.ops.logprob.LinearLogpOp"
    B200_GRPO_LOSS = "rl_kernel_b200.ops.loss.GRPOLossOp"
    B200_CP_ATTENTION = "rl_kernel_b200.ops.distributed.cp_attention.CPAttentionOp"
    B200_VOCAB_PARALLEL_LOGP = "rl_kernel_b200.ops.distributed.vocab_parallel_logp.VocabParallelLinearLogpOp"
    B200_RATIO_KL = "rl_kernel_b200.ops.distributed.losses.RatioKLNativeOp"
    B200_DIST_GRPO_LOSS = "rl_kernel_b200.ops.distributed.losses.DistributedGRPOLossNativeOp"
    B200_PACK = "rl_kernel_b200.ops.packing.PackOp"
    # --- PyTorch references
    REF_DET_GEMM = "rl_kernel_b200.reference.gemm.det_gemm.NativeGemmOp"
    REF_RMS_NORM = "rl_kernel_b200.reference.norm.rms_norm.NativeRMSNormOp"
    REF_ROPE = "rl_kernel_b200.reference.rope.rope.NativeRoPEOp"
    REF_SWIGLU = "rl_kernel_b200.reference.activation.swiglu.NativeSwiGLUOp"
    REF_EMBEDDING = "rl_kernel_b200.reference.embedding.embedding.NativeEmbeddingOp"
    REF_LM_HEAD = "rl_kernel_b200.reference.embedding.embedding.NativeLMHeadOp"
    REF_ATTENTION = "rl_kernel_b200.reference.attention.standard_attn.NativeAttentionOp"
    REF_CP_ATTENTION = "rl_kernel_b200.reference.attention.blockwise.DeterministicCPAttentionReferenceOp"
    REF_FFN = "rl_kernel_b200.reference.ffn.ffn.NativeQwen3FFNOp"
    REF_LOGP = "rl_kernel_b200.reference.logprob.logp.NativeLogpOp"
    REF_BI_LOGP = "rl_kernel_b200.reference.logprob.tile_logp.NativeBatchInvariantLogpOp"
    REF_LINEAR_LOGP = "rl_kernel_b200.reference.logprob.tile_logp.NativeLinearLogpOp"
    REF_VOCAB_PARALLEL_LOGP = "rl_kernel_b200.reference.logprob.tile_logp.VocabParallelLogprobOp"
    REF_GRPO_LOSS = "rl_kernel_b200.reference.loss.grpo_loss.NativeGRPOLossOp"
    REF_RATIO_KL = "rl_kernel_b200.reference.loss.ratio_kl.NativeRatioKLOp"
    REF_DIST_GRPO_LOSS = "rl_kernel_b200.reference.loss.distributed_grpo_loss.DistributedGRPOLossOp"
    REF_PACK = "rl_kernel_b200.reference.packing.pack.NativePackOp"


# operator name -> (b200 implementation or None, reference implementation)
_TABLE: dict[str, tuple[OpBackend | None, OpBackend]] = {
    "det_gemm": (OpBackend.B200_DET_GEMM, OpBackend.REF_DET_GEMM),
    "rms_norm": (OpBackend.B200_RMS_NORM, OpBackend.REF_RMS_NORM),
    "qk_norm": (OpBackend.B200_RMS_NORM, OpBackend.REF_RMS_NORM),
    "rope": (OpBackend.B200_ROPE, OpBackend.REF_ROPE),
    "swiglu": (OpBackend.B200_SWIGLU, OpBackend.REF_SWIGLU),
    "embedding": (OpBackend.B200_EMBEDDING, OpBackend.REF_EMBEDDING),
    "lm_head": (OpBackend.B200_LM_HEAD, OpBackend.REF_LM_HEAD),
    "attention": (OpBackend.B200_ATTENTION, OpBackend.REF_ATTENTION),
    "cp_attention": (OpBackend.B200_CP_ATTENTION, OpBackend.REF_CP_ATTENTION),
    "ffn": (OpBackend.B200_FFN, OpBackend.REF_FFN),
    "logp": (OpBackend.B200_LOGP, OpBackend.REF_LOGP),
    "batch_invariant_logp": (OpBackend.B200_LOGP, OpBackend.REF_BI_LOGP),
    "linear_logp": (OpBackend.B200_LINEAR_LOGP, OpBackend.REF_LINEAR_LOGP),
    "vocab_parallel_logp": (OpBackend.B200_VOCAB_PARALLEL_LOGP, OpBackend.REF_VOCAB_PARALLEL_LOGP),
    "grpo_loss": (OpBackend.B200_GRPO_LOSS, OpBackend.REF_GRPO_LOSS),
    "ratio_kl": (OpBackend.B200_RATIO_KL, OpBackend.REF_RATIO_KL),
    "distributed_grpo_loss": (OpBackend.B200_DIST_GRPO_LOSS, OpBackend.REF_DIST_GRPO_LOSS),
    "pack": (OpBackend.B200_PACK, OpBackend.REF_PACK),
}

_LOGP_ALIASES = {
    "auto": "logp", "default": "logp", "logp": "logp", "fused": "logp", "fused_logp": "logp",
    "deterministic": "batch_invariant_logp", "batch_invariant": "batch_invariant_logp",
    "batch_invariant_logp": "batch_invariant_logp", "linear": "linear_logp", "linear_logp": "linear_logp",
    "fused_linear_logp": "linear_logp", "vocab_parallel": "vocab_parallel_logp",
}


def resolve_logp_op_type(name: str = "auto", *, require_batch_invariant: bool = False) -> str:
    """Map user-facing log-prob backend names to registry operator names
    (parity: resolve_logp_op_type, registry.py:369-413)."""
    key = (name or "auto").strip().lower()
    if key not in _LOGP_ALIASES:
        raise ValueError(f"unknown logp backend {name!r}; choose from {sorted(_LOGP_ALIASES)}")
    op = _LOGP_ALIASES[key]
    if require_batch_invariant and op == "logp":
        op = "batch_invariant_logp"
    return op


@dataclass
class Resolution:
    op_name: str
    requested: str
    actual: OpBackend
    fallback: bool
    reason: str


def _load(path: OpBackend):
    mod, _, attr = path.value.rpartition(".")
    return getattr(importlib.import_module(mod), attr)


class KernelRegistry:
    def __init__(self) -> None:
        self._lock = threading.Lock()
        self._instances: dict[tuple, object] = {}
        self._failed: set[OpBackend] = set()
        self.last_resolution: Resolution | None = None
        self.history: list[Resolution] = []

    # ---- hardware gating
    @staticmethod
    def native_ready() -> tuple[bool, str]:
        if not torch.cuda.is_available():
            return False, "no CUDA device"
        if tuple(torch.cuda.get_device_capability()) != (10, 0):
            return False, f"device capability {torch.cuda.get_device_capability()} is not sm_100"
        from rl_kernel_b200.backends import extension

        if extension.load(required=False) is None:
            return False, "librlk_b200.so is not built"
        return True, "sm_100a library loaded"

    def available_ops(self) -> list[str]:
        return sorted(_TABLE)

    def resolve(self, op_name: str, prefer: str = "auto") -> Resolution:
        if op_name not in _TABLE:
            raise KeyError(f"unknown operator {op_name!r}; known: {self.available_ops()}")
        native, ref = _TABLE[op_name]
        mode = current_mode()
        ready, why = self.native_ready()
        if prefer == "reference" or mode is RLKernelMode.OFF:
            res = Resolution(op_name, prefer, ref, False, "reference requested" if prefer == "reference" else "mode off")
        elif native is not None and ready and native not in self._failed:
            res = Resolution(op_name, prefer, native, False, why)
        else:
            reason = why if native is not None else "no sm_100a kernel registered for this operator"
            if native in self._failed:
                reason = "implementation failed to construct earlier"
            fallback = native is not None
            if fallback and mode is RLKernelMode.STRICT and torch.cuda.is_available():
                raise RuntimeError(f"strict mode: operator {op_name!r} would fall back to the reference ({reason})")
            res = Resolution(op_name, prefer, ref, fallback, reason)
        route_report(op_name, res.requested, res.actual.name, res.fallback)
        self.last_resolution = res
        self.history.append(res)
        return res

    def get_op(self, op_name: str, *args, prefer: str = "auto", **kwargs):
        res = self.resolve(op_name, prefer)
        key = (res.actual, args, tuple(sorted(kwargs.items())))
        with self._lock:
            if key not in self._instances:
                try:
                    self._instances[key] = _load(res.actual)(*args, **kwargs)
                except Exception:
                    self._failed.add(res.actual)
                    raise
            return self._instances[key]

    def get_logprob_op(self, backend: str = "auto", *, contract=None, require_batch_invariant: bool = False, **kwargs):
        """Resolve a log-prob operator; with a contract the backend capability is checked first
        (parity: get_logprob_op, registry.py:1098-1186)."""
        from rl_kernel_b200.contracts.operators.logprob import (B200_LOGPROB_CAPABILITY,
                                                                REFERENCE_LOGPROB_CAPABILITY)

        op_name = resolve_logp_op_type(backend, require_batch_invariant=require_batch_invariant)
        if contract is not None:
            ready, _ = self.native_ready()
            cap = B200_LOGPROB_CAPABILITY if ready else REFERENCE_LOGPROB_CAPABILITY
            why = cap.incompatibilities(contract)
            if why:
                raise RuntimeError(f"logprob backend {cap.backend_id} cannot serve the contract: {why}")
            kwargs.setdefault("temperature", contract.temperature)
        return self.get_op(op_name, **kwargs)

    def get_attention_op(self, backend: str = "auto", *, contract=None, **kwargs):
        """Resolve an attention operator.  ``auto`` is rejected under context parallelism: the CP
        schedule must be chosen explicitly (parity: registry.py:1210-1287)."""
        from rl_kernel_b200.contracts.operators.attention import (B200_ATTENTION_CAPABILITY,
                                                                  REFERENCE_ATTENTION_CAPABILITY)

        if contract is not None:
            if contract.sharding.cp_world_size > 1 and backend == "auto":
                raise ValueError("attention backend 'auto' is not allowed with cp_size > 1; name the CP schedule")
            ready, _ = self.native_ready()
            cap = B200_ATTENTION_CAPABILITY if ready else REFERENCE_ATTENTION_CAPABILITY
            why = cap.incompatibilities(contract)
            if why:
                raise RuntimeError(f"attention backend {cap.backend_id} cannot serve the contract: {why}")
        name = "cp_attention" if backend in ("cp", "cp_native", "cp_reference") else "attention"
        prefer = "reference" if backend == "cp_reference" else "auto"
        if name == "cp_attention" and prefer == "auto" and "collective" not in kwargs:
            # the native schedule needs the context-parallel group's collective and the geometry;
            # without them only the single-process reference can be built
            prefer = "reference"
        return self.get_op(name, prefer=prefer, **kwargs)

    def provenance(self) -> list[dict]:
        return [{"op": r.op_name, "requested": r.requested, "actual": r.actual.name, "path": r.actual.value,
                 "fallback": r.fallback, "reason": r.reason} for r in self.history]


kernel_registry = KernelRegistry()
