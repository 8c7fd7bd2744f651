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
import os
import threading
from collections.abc import Callable
from dataclasses import dataclass, field
from typing import Any

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

# names the reference's callers use for the same operators
_OP_ALIASES = {"attn": "attention", "gemm": "det_gemm", "rmsnorm": "rms_norm", "fused_logp": "logp"}

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
    actual: "OpBackend | RegisteredBackend"
    fallback: bool
    reason: str


@dataclass(frozen=True)
class RegisteredBackend:
    """A backend added at run time (``KernelRegistry.register_backend``): something that only exists on some machines
    (a vendor library behind an import), a user's experiment, or a test double.  ``factory`` builds the operator object;
    ``available`` is asked at every resolution; ``capability`` (an ``AttentionBackendCapability`` or
    ``LogprobBackendCapability``) lets contract-aware dispatch decide whether the backend may serve a request."""
    op_name: str
    backend_id: str
    factory: Callable[..., Any] = field(compare=False)
    available: Callable[[], bool] = field(default=lambda: True, compare=False)
    capability: Any = field(default=None, compare=False)
    device_types: tuple[str, ...] = ("cuda", "cpu")

    @property
    def name(self) -> str:                       # the same two attributes an OpBackend member offers
        return self.backend_id

    @property
    def value(self) -> str:
        f = self.factory
        return f"{getattr(f, '__module__', '?')}.{getattr(f, '__qualname__', repr(f))}"


def _disabled_backends() -> set[str]:
    """``RL_KERNEL_DISABLE_BACKENDS=a,b``: backend ids (registered ones) or ``b200`` / ``native`` (the sm_100a kernels)
    taken out of every candidate list of this process."""
    return {x.strip().lower() for x in os.environ.get("RL_KERNEL_DISABLE_BACKENDS", "").split(",") if x.strip()}


def _env_preference(op_name: str) -> str | None:
    """``RL_KERNEL_BACKEND_<OP>=reference|b200|<registered id>`` pins one operator's backend for the process (an
    explicit ``prefer=`` argument still wins)."""
    v = os.environ.get(f"RL_KERNEL_BACKEND_{op_name.upper()}", "").strip()
    return v or None


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
        self._registered: dict[str, list[RegisteredBackend]] = {}

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
        return sorted(set(_TABLE) | {k for k, v in self._registered.items() if v})

    # ---- run-time backends
    def register_backend(self, op_name: str, backend_id: str, factory: Callable[..., Any], *, prepend: bool = True,
                         available: Callable[[], bool] | None = None, capability: Any = None,
                         device_types: tuple[str, ...] = ("cuda", "cpu")) -> RegisteredBackend:
        """Add (or replace, by id) a backend for ``op_name``.  Registered backends are tried before the built-in pair
        in list order (``prepend=False`` appends).  A new operator name is allowed: its only candidates are the
        registered ones."""
        if not backend_id or backend_id.lower() in ("auto", "reference", "b200", "native"):
            raise ValueError(f"backend id {backend_id!r} is reserved")
        rb = RegisteredBackend(op_name, backend_id, factory, available or (lambda: True), capability, tuple(device_types))
        with self._lock:
            lst = [b for b in self._registered.get(op_name, []) if b.backend_id != backend_id]
            lst.insert(0, rb) if prepend else lst.append(rb)
            self._registered[op_name] = lst
            self._instances = {k: v for k, v in self._instances.items() if not (isinstance(k[0], RegisteredBackend) and k[0] == rb)}
        return rb

    def unregister_backend(self, op_name: str, backend_id: str) -> bool:
        with self._lock:
            before = self._registered.get(op_name, [])
            after = [b for b in before if b.backend_id != backend_id]
            self._registered[op_name] = after
            return len(after) != len(before)

    def register_attention_backend(self, backend_id: str, factory: Callable[..., Any], capability, *, op_name: str = "attention",
                                   prepend: bool = False, available: Callable[[], bool] | None = None) -> RegisteredBackend:
        """Contract-aware attention backend (parity: register_attention_backend, registry.py:924-957): it is chosen by
        ``get_attention_op(contract=...)`` only when its capability has nothing against the contract."""
        from rl_kernel_b200.contracts.operators.attention import AttentionBackendCapability

        if not isinstance(capability, AttentionBackendCapability):
            raise TypeError("capability must be an AttentionBackendCapability")
        return self.register_backend(op_name, backend_id, factory, prepend=prepend, available=available, capability=capability)

    def register_logprob_backend(self, backend_id: str, factory: Callable[..., Any], capability, *, op_name: str = "logp",
                                 prepend: bool = False, available: Callable[[], bool] | None = None) -> RegisteredBackend:
        """The log-prob counterpart (parity: register_logprob_backend, registry.py:1063-1096)."""
        from rl_kernel_b200.contracts.operators.logprob import LogprobBackendCapability

        if not isinstance(capability, LogprobBackendCapability):
            raise TypeError("capability must be a LogprobBackendCapability")
        return self.register_backend(op_name, backend_id, factory, prepend=prepend, available=available, capability=capability)

    def candidates(self, op_name: str, device: torch.device | str | None = None) -> list[dict]:
        """Every backend that could serve ``op_name``, in resolution order, with whether it is usable now and why not."""
        op_name = _OP_ALIASES.get(op_name, op_name)
        if op_name not in _TABLE and not self._registered.get(op_name):
            raise KeyError(f"unknown operator {op_name!r}; known: {self.available_ops()}")
        dev = None if device is None else torch.device(device).type
        off = _disabled_backends()
        out = []
        for rb in self._registered.get(op_name, []):
            why = ""
            if rb.backend_id.lower() in off:
                why = "disabled by RL_KERNEL_DISABLE_BACKENDS"
            elif dev is not None and dev not in rb.device_types:
                why = f"does not run on {dev}"
            else:
                try:
                    why = "" if rb.available() else "reports itself unavailable"
                except Exception as exc:  # noqa: BLE001 - an availability probe must never break resolution
                    why = f"availability probe raised {type(exc).__name__}: {exc}"
            out.append({"backend": rb, "id": rb.backend_id, "kind": "registered", "usable": not why, "reason": why})
        if op_name in _TABLE:
            native, ref = _TABLE[op_name]
            ready, why = self.native_ready()
            if native is not None:
                reason = ""
                if {"b200", "native"} & off:
                    reason = "disabled by RL_KERNEL_DISABLE_BACKENDS"
                elif dev == "cpu":
                    reason = "operands are on the CPU"
                elif not ready:
                    reason = why
                elif native in self._failed:
                    reason = "implementation failed to construct earlier"
                out.append({"backend": native, "id": "b200", "kind": "native", "usable": not reason, "reason": reason})
            out.append({"backend": ref, "id": "reference", "kind": "reference", "usable": True, "reason": ""})
        return out

    def resolve(self, op_name: str, prefer: str = "auto", *, device: torch.device | str | None = None,
                accept: Callable[[dict], str] | None = None) -> Resolution:
        """Pick the backend of ``op_name``.  ``prefer``: ``auto`` (first usable candidate), ``reference``, ``b200`` or a
        registered id; ``RL_KERNEL_BACKEND_<OP>`` supplies it when the caller passes ``auto``.  ``device`` (of the
        operands) keeps CPU tensors off the GPU kernels without calling that a fallback.  ``accept(candidate)`` returns a
        reason to skip a candidate (capability checks)."""
        op_name = _OP_ALIASES.get(op_name, op_name)
        cands = self.candidates(op_name, device)
        mode = current_mode()
        requested = prefer
        if prefer == "auto":
            prefer = _env_preference(op_name) or "auto"
        if mode is RLKernelMode.OFF and prefer == "auto":
            prefer = "reference"
        rejected: list[str] = []
        chosen = None
        for c in cands:
            if prefer != "auto" and c["id"].lower() != prefer.lower():
                continue
            why = c["reason"] or (accept(c) if accept is not None else "")
            if why:
                rejected.append(f"{c['id']}: {why}")
                continue
            chosen = c
            break
        if chosen is None:
            if prefer != "auto" and not any(c["id"].lower() == prefer.lower() for c in cands):
                raise KeyError(f"operator {op_name!r} has no backend {prefer!r}; candidates: {[c['id'] for c in cands]}")
            raise RuntimeError(f"no usable backend for operator {op_name!r} (asked for {prefer!r}): {'; '.join(rejected)}")
        on_cpu = device is not None and torch.device(device).type == "cpu"
        native_skipped = next((r for r in rejected if r.startswith("b200:")), None)
        fallback = chosen["kind"] == "reference" and prefer == "auto" and native_skipped is not None and not on_cpu \
            and mode is not RLKernelMode.OFF
        if chosen["kind"] == "reference":
            reason = ("reference requested" if requested == "reference" else "mode off" if mode is RLKernelMode.OFF else
                      (native_skipped or "no sm_100a kernel registered for this operator").removeprefix("b200: "))
        elif chosen["kind"] == "native":
            reason = self.native_ready()[1]
        else:
            reason = "registered backend"
        if fallback and mode is RLKernelMode.STRICT and torch.cuda.is_available():
            raise RuntimeError(f"strict mode: operator {op_name!r} would fall back to the reference ({reason})")
        res = Resolution(op_name, requested, chosen["backend"], fallback, reason)
        route_report(op_name, res.requested, res.actual.name, res.fallback)
        self.last_resolution = res
        self.history.append(res)
        return res

    def get_op(self, op_name: str, *args, prefer: str = "auto", operand_device: torch.device | str | None = None, **kwargs):
        """A ready operator object.  ``operand_device``: where the tensors it will be called with live (CPU operands get
        the reference without that counting as a fallback); every other keyword goes to the operator's constructor."""
        res = self.resolve(op_name, prefer, device=operand_device)
        return self._instantiate(res, args, kwargs)

    def _instantiate(self, res: Resolution, args: tuple, kwargs: dict):
        try:
            key = (res.actual, args, tuple(sorted(kwargs.items())))
            hash(key)
        except TypeError:                                     # unhashable constructor arguments: build, do not cache
            key = None
        with self._lock:
            if key is not None and key in self._instances:
                return self._instances[key]
            try:
                maker = res.actual.factory if isinstance(res.actual, RegisteredBackend) else _load(res.actual)
                obj = maker(*args, **kwargs)
            except Exception:
                if isinstance(res.actual, OpBackend):
                    self._failed.add(res.actual)
                raise
            if key is not None:
                self._instances[key] = obj
            return obj

    @staticmethod
    def _capability_gate(contract, native_cap, reference_cap) -> Callable[[dict], str]:
        """Candidate filter for contract-aware dispatch: a backend whose capability objects to the contract is skipped
        with its objections as the reason (a registered backend without a capability is never chosen for a contract)."""
        def accept(c: dict) -> str:
            cap = {"native": native_cap, "reference": reference_cap}.get(c["kind"], getattr(c["backend"], "capability", None))
            if cap is None:
                return "declares no capability: cannot be matched against a contract"
            why = cap.incompatibilities(contract)
            return "" if not why else f"{cap.backend_id} cannot serve the contract: {'; '.join(why)}"
        return accept

    def get_logprob_op(self, backend: str = "auto", *, contract=None, require_batch_invariant: bool = False,
                       operand_device: torch.device | str | None = None, **kwargs):
        """Resolve a log-prob operator.  ``backend`` is a user-facing family name (``auto``, ``batch_invariant``,
        ``linear``, ``vocab_parallel``, ...) or the id of a registered backend.  With a contract every candidate's
        capability is checked and the first compatible one wins; when none is, the error lists every objection
        (parity: get_logprob_op / _logprob_policy_mismatch, registry.py:1098-1207)."""
        from rl_kernel_b200.contracts.operators.logprob import B200_LOGPROB_CAPABILITY, REFERENCE_LOGPROB_CAPABILITY

        prefer = "auto"
        key = (backend or "auto").strip().lower()
        if key in _LOGP_ALIASES:
            op_name = resolve_logp_op_type(backend, require_batch_invariant=require_batch_invariant)
        else:
            owners = [op for op, lst in self._registered.items() if any(b.backend_id.lower() == key for b in lst)]
            if not owners:
                raise ValueError(f"unknown logp backend {backend!r}; choose from {sorted(_LOGP_ALIASES)} or a registered id")
            op_name, prefer = owners[0], key
        accept = None
        if contract is not None:
            accept = self._capability_gate(contract, B200_LOGPROB_CAPABILITY, REFERENCE_LOGPROB_CAPABILITY)
            kwargs.setdefault("temperature", contract.temperature)
        res = self.resolve(op_name, prefer, device=operand_device, accept=accept)
        return self._instantiate(res, (), kwargs)

    def get_attention_op(self, backend: str = "auto", *, contract=None, operand_device: torch.device | str | None = None, **kwargs):
        """Resolve an attention operator.  ``auto`` is rejected under context parallelism: the CP schedule must be
        chosen explicitly.  ``backend`` may also be the id of a backend registered with ``register_attention_backend``
        (parity: get_attention_op / _attention_policy_mismatch, registry.py:1210-1308)."""
        from rl_kernel_b200.contracts.operators.attention import B200_ATTENTION_CAPABILITY, REFERENCE_ATTENTION_CAPABILITY

        if contract is not None and contract.sharding.cp_world_size > 1 and backend == "auto":
            raise ValueError("attention backend 'auto' is not allowed with cp_size > 1; name the CP schedule")
        accept = None if contract is None else self._capability_gate(contract, B200_ATTENTION_CAPABILITY, REFERENCE_ATTENTION_CAPABILITY)
        key = (backend or "auto").strip().lower()
        builtin = {"auto": ("attention", "auto"), "b200": ("attention", "auto"), "reference": ("attention", "reference"),
                   "cp": ("cp_attention", "auto"), "cp_native": ("cp_attention", "auto"), "cp_reference": ("cp_attention", "reference")}
        if key in builtin:
            name, prefer = builtin[key]
        else:
            owners = [op for op, lst in self._registered.items() if any(b.backend_id.lower() == key for b in lst)]
            if not owners:
                raise ValueError(f"unknown attention backend {backend!r}; choose from {sorted(builtin)} or a registered id")
            name, prefer = owners[0], key
        if name == "cp_attention" and prefer == "auto" and "collective" not in kwargs:
            # the native schedule needs the context-parallel group's collective and the geometry;
            # without them only the single-process reference can be built
            prefer = "reference"
        res = self.resolve(name, prefer, device=operand_device, accept=accept)
        return self._instantiate(res, (), kwargs)

    def describe(self) -> dict[str, list[dict]]:
        """Operator -> candidates (id, kind, usable, reason, import path): what ``rlk ops`` prints."""
        names = sorted(set(_TABLE) | {k for k, v in self._registered.items() if v})
        return {n: [{"id": c["id"], "kind": c["kind"], "usable": c["usable"], "reason": c["reason"], "path": c["backend"].value}
                    for c in self.candidates(n)] for n in names}

    def provenance(self) -> list[dict]:
        return [{"op": r.op_name, "requested": r.requested, "actual": r.actual.name, "path": r.actual.value,
                 "fallback": r.fallback, "reason": r.reason} for r in self.history]


kernel_registry = KernelRegistry()
