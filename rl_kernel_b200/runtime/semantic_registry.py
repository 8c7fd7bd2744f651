"""Semantic operator catalog: descriptors of what an implementation IS (schedule, determinism,
contract id, code fingerprint) and sessions that record what an integration actually executed
(parity: OperatorBackendDescriptor / SemanticOperatorCatalog / OperatorSession,
rl_engine/runtime/semantic_registry.py:68-790 and the defaults of registry.py:205-354)."""
from __future__ import annotations

import time
from dataclasses import asdict, dataclass, field

from rl_kernel_b200.runtime.provenance.identity import code_fingerprint, native_library_fingerprint


@dataclass(frozen=True)
class OperatorBackendDescriptor:
    semantic_op: str           # selected_logprob | attention | ffn | det_gemm | ...
    backend_id: str
    schedule: str
    contract_id: str
    deterministic: bool = True
    batch_invariant: bool = True
    tp_invariant: bool = True
    cp_invariant: bool = True
    notes: str = ""

    def key(self) -> tuple[str, str]:
        return (self.semantic_op, self.backend_id)


DEFAULT_DESCRIPTORS = (
    OperatorBackendDescriptor("det_gemm", "b200-tcgen05", "tma_umma_tmem_128xN_no_splitk_canonical_chunk_tree",
                              "det_gemm.canonical_chunk_tree.v1"),
    OperatorBackendDescriptor("attention", "b200-tcgen05", "canonical_block128_ascending_no_splitkv",
                              "attention.canonical_block128.v1"),
    OperatorBackendDescriptor("ffn", "b200-tcgen05", "packed_gate_up_canonical_tp8_tree", "ffn.canonical_tp8.v1"),
    OperatorBackendDescriptor("selected_logprob", "b200-tcgen05", "fused_lm_head_vocab_tile128_ordered_merge",
                              "logprob.vocab_tile128.v1"),
    OperatorBackendDescriptor("grpo_loss", "b200", "sequence_major_fixed_sums", "grpo_loss.sequence_major.v1"),
    OperatorBackendDescriptor("collective", "b200-symm", "balanced_tree_rank_order_bounded_waits",
                              "collective.balanced_tree.v1"),
    OperatorBackendDescriptor("attention", "reference", "blockwise_rowwise_matvec", "attention.canonical_block128.v1"),
    OperatorBackendDescriptor("selected_logprob", "reference", "tile128_reference", "logprob.vocab_tile128.v1"),
)


@dataclass
class ExecutionRecord:
    semantic_op: str
    backend_id: str
    module: str
    count: int = 0
    first_ts: float = field(default_factory=time.time)
    fallback: bool = False


class OperatorSession:
    """Collects executions of semantic operators inside one integration (one engine process)."""

    def __init__(self, catalog: "SemanticOperatorCatalog", name: str):
        self.catalog, self.name = catalog, name
        self.records: dict[tuple[str, str, str], ExecutionRecord] = {}

    def observe(self, semantic_op: str, backend_id: str, module: str = "", fallback: bool = False) -> None:
        self.catalog.describe(semantic_op, backend_id)     # must be a registered implementation
        key = (semantic_op, backend_id, module)
        rec = self.records.setdefault(key, ExecutionRecord(semantic_op, backend_id, module, fallback=fallback))
        rec.count += 1
        rec.fallback |= fallback

    def assert_no_fallback(self) -> None:
        bad = [r for r in self.records.values() if r.fallback]
        if bad:
            raise RuntimeError(f"session {self.name!r} executed fallbacks: {[(r.semantic_op, r.module) for r in bad]}")

    def readback(self) -> dict:
        return {"session": self.name, "implementation_fingerprint": self.catalog.implementation_fingerprint(),
                "records": [asdict(r) for r in self.records.values()]}


class SemanticOperatorCatalog:
    def __init__(self, descriptors=DEFAULT_DESCRIPTORS):
        self._by_key: dict[tuple[str, str], OperatorBackendDescriptor] = {}
        for d in descriptors:
            self.register(d)

    def register(self, d: OperatorBackendDescriptor) -> None:
        if d.key() in self._by_key and self._by_key[d.key()] != d:
            raise ValueError(f"descriptor {d.key()} already registered with different content")
        self._by_key[d.key()] = d

    def describe(self, semantic_op: str, backend_id: str) -> OperatorBackendDescriptor:
        try:
            return self._by_key[(semantic_op, backend_id)]
        except KeyError as exc:
            raise KeyError(f"no descriptor for {semantic_op!r} on backend {backend_id!r}") from exc

    def backends(self, semantic_op: str) -> list[OperatorBackendDescriptor]:
        return [d for (op, _), d in self._by_key.items() if op == semantic_op]

    def session(self, name: str) -> OperatorSession:
        return OperatorSession(self, name)

    def implementation_fingerprint(self) -> dict:
        return {"native_library_sha256": native_library_fingerprint(),
                "descriptors_sha256": code_fingerprint(*sorted(self._by_key.values(), key=lambda d: d.key()))}


semantic_catalog = SemanticOperatorCatalog()


# ================================================================================================ requirement-driven resolution
# (parity: OperatorRequirements / OperatorResolutionPolicy / OperatorResolution(Trace) / OperatorInstanceProvenance and
#  the implementation fingerprints of rl_engine/runtime/semantic_registry.py:19-790)
import hashlib as _hashlib
import importlib as _importlib
import json as _json
from enum import Enum as _Enum
from types import CodeType as _CodeType
from typing import Any as _Any, Callable as _Callable, Mapping as _Mapping


class OperatorLifecycle(str, _Enum):
    PRODUCTION = "production"
    REFERENCE = "reference"
    SMOKE_ONLY = "smoke_only"


class OperatorFallbackPolicy(str, _Enum):
    FORBID = "forbid"          # the requested backend or an error
    ALLOW = "allow"            # the best compatible backend, recorded as a fallback


@dataclass(frozen=True)
class OperatorResolutionPolicy:
    fallback: OperatorFallbackPolicy = OperatorFallbackPolicy.FORBID
    allow_smoke_only: bool = False
    allow_reference: bool = True

    @classmethod
    def strict(cls) -> "OperatorResolutionPolicy":
        return cls(OperatorFallbackPolicy.FORBID, False, True)

    @classmethod
    def permissive(cls) -> "OperatorResolutionPolicy":
        return cls(OperatorFallbackPolicy.ALLOW, False, True)


@dataclass(frozen=True)
class OperatorRequirements:
    """What a caller needs from an implementation of a semantic operator."""
    semantic_op: str
    device_type: str = "cuda"
    dtype: str = "bfloat16"
    deterministic: bool = True
    batch_invariant: bool = True
    tp_world_size: int = 1
    cp_world_size: int = 1
    target: str = "any"                 # rollout | training | any

    def __post_init__(self) -> None:
        if not self.semantic_op:
            raise ValueError("semantic_op must not be empty")
        if self.target not in ("rollout", "training", "any"):
            raise ValueError("target must be rollout, training or any")
        object.__setattr__(self, "device_type", str(self.device_type).split(":")[0])
        object.__setattr__(self, "dtype", str(self.dtype).removeprefix("torch."))

    def to_dict(self) -> dict:
        return asdict(self)


@dataclass(frozen=True)
class ImplementationDescriptor:
    """How to build an implementation and where it can run; joined to an ``OperatorBackendDescriptor`` by key."""
    semantic_op: str
    backend_id: str
    factory: str | _Callable[..., _Any]                  # "module.attr" or a callable returning the operator object
    device_types: frozenset = frozenset({"cuda"})
    dtypes: frozenset = frozenset({"bfloat16"})
    lifecycle: OperatorLifecycle = OperatorLifecycle.PRODUCTION
    priority: int = 0                                   # higher wins among compatible backends
    max_tp_world_size: int = 8
    max_cp_world_size: int = 8
    targets: frozenset = frozenset({"rollout", "training"})

    def key(self) -> tuple[str, str]:
        return (self.semantic_op, self.backend_id)

    @property
    def implementation_reference(self) -> str:
        f = self.factory
        return f if isinstance(f, str) else f"{getattr(f, '__module__', '?')}.{getattr(f, '__qualname__', repr(f))}"


@dataclass(frozen=True)
class OperatorCapabilityDecision:
    backend_id: str
    compatible: bool
    reasons: tuple[str, ...] = ()

    def to_dict(self) -> dict:
        return {"backend_id": self.backend_id, "compatible": self.compatible, "reasons": list(self.reasons)}


@dataclass(frozen=True)
class OperatorResolutionTrace:
    requirements: OperatorRequirements
    requested_backend: str | None
    decisions: tuple[OperatorCapabilityDecision, ...]
    policy: OperatorResolutionPolicy

    def to_dict(self) -> dict:
        return {"requirements": self.requirements.to_dict(), "requested_backend": self.requested_backend,
                "decisions": [d.to_dict() for d in self.decisions],
                "policy": {"fallback": self.policy.fallback.value, "allow_smoke_only": self.policy.allow_smoke_only,
                           "allow_reference": self.policy.allow_reference}}


@dataclass(frozen=True)
class OperatorResolution:
    semantic_op: str
    requested_backend: str | None
    actual_backend: str
    fallback: bool
    descriptor: OperatorBackendDescriptor
    implementation: ImplementationDescriptor
    trace: OperatorResolutionTrace

    def to_dict(self) -> dict:
        return {"semantic_op": self.semantic_op, "requested_backend": self.requested_backend, "actual_backend": self.actual_backend,
                "fallback": self.fallback, "descriptor": asdict(self.descriptor),
                "implementation_reference": self.implementation.implementation_reference, "trace": self.trace.to_dict()}


@dataclass(frozen=True)
class OperatorInstanceProvenance:
    semantic_op: str
    backend_id: str
    implementation_reference: str
    implementation_fingerprint: str
    instance_fingerprint: str
    native_library_sha256: str | None

    def to_dict(self) -> dict:
        return asdict(self)


class OperatorRegistrationError(ValueError):
    pass


class OperatorResolutionError(RuntimeError):
    def __init__(self, message: str, trace: OperatorResolutionTrace):
        super().__init__(message)
        self.trace = trace


class OperatorInstantiationError(RuntimeError):
    pass


def _load_factory(value):
    if callable(value):
        return value
    mod, _, attr = str(value).rpartition(".")
    try:
        return getattr(_importlib.import_module(mod), attr)
    except (ImportError, AttributeError) as exc:
        raise OperatorInstantiationError(f"cannot load operator factory {value!r}: {exc}") from exc


def _code_fingerprint(code: _CodeType) -> str:
    """Hash of what a function does: bytecode, names and constants (nested code objects included); file paths and line
    numbers are left out, so moving a file does not change the fingerprint."""
    h = _hashlib.sha256()
    h.update(code.co_code)
    h.update(repr((code.co_names, code.co_varnames, code.co_argcount, code.co_kwonlyargcount)).encode())
    for c in code.co_consts:
        h.update(_code_fingerprint(c).encode() if isinstance(c, _CodeType) else repr(c).encode())
    return h.hexdigest()


def implementation_fingerprint(obj: _Any, *, instance: _Any = None, entrypoints: tuple[str, ...] = ()) -> str:
    """sha256 identifying the code of an operator: a function's code object, or a class' methods (``entrypoints`` or all
    functions defined on it), plus the native library image when the operator is served by it."""
    cls = obj if isinstance(obj, type) or callable(obj) and hasattr(obj, "__code__") else type(obj)
    parts: dict[str, str] = {}
    if hasattr(cls, "__code__"):
        parts[getattr(cls, "__qualname__", "fn")] = _code_fingerprint(cls.__code__)
    else:
        names = entrypoints or tuple(n for n, v in sorted(vars(cls).items()) if callable(v) and hasattr(v, "__code__"))
        for n in names:
            fn = getattr(cls, n, None)
            fn = getattr(fn, "__func__", fn)
            if fn is not None and hasattr(fn, "__code__"):
                parts[n] = _code_fingerprint(fn.__code__)
    ident = {"module": getattr(cls, "__module__", None), "qualname": getattr(cls, "__qualname__", None), "code": parts,
             "backend_id": getattr(instance if instance is not None else obj, "backend_id", None)}
    return _hashlib.sha256(_json.dumps(ident, sort_keys=True).encode()).hexdigest()


def operator_instance_fingerprint(**identity: str) -> str:
    return _hashlib.sha256(_json.dumps(identity, sort_keys=True).encode()).hexdigest()


def _decide(impl: ImplementationDescriptor, desc: OperatorBackendDescriptor, req: OperatorRequirements,
            policy: OperatorResolutionPolicy) -> OperatorCapabilityDecision:
    why = []
    if req.device_type not in impl.device_types:
        why.append(f"runs on {sorted(impl.device_types)}, not on {req.device_type}")
    if req.dtype not in impl.dtypes:
        why.append(f"computes in {sorted(impl.dtypes)}, not in {req.dtype}")
    if req.deterministic and not desc.deterministic:
        why.append("is not deterministic")
    if req.batch_invariant and not desc.batch_invariant:
        why.append("is not batch-invariant")
    if req.tp_world_size > 1 and (not desc.tp_invariant or req.tp_world_size > impl.max_tp_world_size):
        why.append(f"does not keep its bits at tensor-parallel size {req.tp_world_size}")
    if req.cp_world_size > 1 and (not desc.cp_invariant or req.cp_world_size > impl.max_cp_world_size):
        why.append(f"does not keep its bits at context-parallel size {req.cp_world_size}")
    if req.target != "any" and req.target not in impl.targets:
        why.append(f"serves {sorted(impl.targets)}, not {req.target}")
    if impl.lifecycle is OperatorLifecycle.SMOKE_ONLY and not policy.allow_smoke_only:
        why.append("is a smoke-only operator")
    if impl.lifecycle is OperatorLifecycle.REFERENCE and not policy.allow_reference:
        why.append("is a reference operator")
    return OperatorCapabilityDecision(impl.backend_id, not why, tuple(why))


DEFAULT_IMPLEMENTATIONS = (
    ImplementationDescriptor("det_gemm", "b200-tcgen05", "rl_kernel_b200.ops.gemm.det_gemm.DetGemmOp", priority=10),
    ImplementationDescriptor("attention", "b200-tcgen05", "rl_kernel_b200.ops.attention.attention.AttentionOp", priority=10),
    ImplementationDescriptor("attention", "reference", "rl_kernel_b200.reference.attention.standard_attn.NativeAttentionOp",
                             frozenset({"cpu", "cuda"}), frozenset({"float32", "bfloat16"}), OperatorLifecycle.REFERENCE, 0, 1, 1),
    ImplementationDescriptor("ffn", "b200-tcgen05", "rl_kernel_b200.ops.ffn.qwen3.Qwen3FFNOp", priority=10),
    ImplementationDescriptor("selected_logprob", "b200-tcgen05", "rl_kernel_b200.ops.logprob.BatchInvariantLogpOp", priority=10),
    ImplementationDescriptor("selected_logprob", "reference", "rl_kernel_b200.reference.logprob.tile_logp.NativeBatchInvariantLogpOp",
                             frozenset({"cpu", "cuda"}), frozenset({"float32", "bfloat16", "float16"}), OperatorLifecycle.REFERENCE, 0, 8, 8),
    ImplementationDescriptor("grpo_loss", "b200", "rl_kernel_b200.ops.loss.GRPOLossOp", frozenset({"cuda"}), frozenset({"float32"}), priority=10),
)


def _install_resolution(cls):
    """Adds implementation registration / resolution / instantiation to ``SemanticOperatorCatalog``."""

    def register_backend(self, impl: ImplementationDescriptor, descriptor: OperatorBackendDescriptor | None = None) -> None:
        if descriptor is not None:
            self.register(descriptor)
        if impl.key() not in self._by_key:
            raise OperatorRegistrationError(f"implementation {impl.key()} has no operator descriptor; register one with it")
        table = self.__dict__.setdefault("_impls", {})
        if impl.key() in table and table[impl.key()] != impl:
            raise OperatorRegistrationError(f"implementation {impl.key()} already registered with different content")
        table[impl.key()] = impl

    def implementations(self, semantic_op: str) -> list[ImplementationDescriptor]:
        return sorted((i for (op, _), i in self.__dict__.get("_impls", {}).items() if op == semantic_op), key=lambda i: (-i.priority, i.backend_id))

    def resolve(self, requirements: OperatorRequirements, *, backend: str | None = None,
                policy: OperatorResolutionPolicy | None = None) -> OperatorResolution:
        policy = policy or OperatorResolutionPolicy.strict()
        impls = self.implementations(requirements.semantic_op)
        decisions = tuple(_decide(i, self._by_key[i.key()], requirements, policy) for i in impls)
        trace = OperatorResolutionTrace(requirements, backend, decisions, policy)
        if not impls:
            raise OperatorResolutionError(f"no implementation of {requirements.semantic_op!r} is registered", trace)
        ok = {d.backend_id for d in decisions if d.compatible}
        if backend not in (None, "auto"):
            if backend not in {i.backend_id for i in impls}:
                raise OperatorResolutionError(f"{requirements.semantic_op!r} has no backend {backend!r}", trace)
            if backend in ok:
                chosen, fb = backend, False
            elif policy.fallback is OperatorFallbackPolicy.ALLOW and ok:
                chosen, fb = next(i.backend_id for i in impls if i.backend_id in ok), True
            else:
                why = next(d.reasons for d in decisions if d.backend_id == backend)
                raise OperatorResolutionError(f"backend {backend!r} cannot serve {requirements.semantic_op!r}: it {'; '.join(why)}", trace)
        else:
            if not ok:
                raise OperatorResolutionError(f"no registered backend can serve {requirements.semantic_op!r} under these requirements", trace)
            chosen, fb = next(i.backend_id for i in impls if i.backend_id in ok), False
        impl = next(i for i in impls if i.backend_id == chosen)
        return OperatorResolution(requirements.semantic_op, backend, chosen, fb, self._by_key[impl.key()], impl, trace)

    def instantiate(self, resolution: OperatorResolution, **kwargs):
        factory = _load_factory(resolution.implementation.factory)
        try:
            return factory(**kwargs)
        except TypeError as exc:
            raise OperatorInstantiationError(f"{resolution.implementation.implementation_reference}({sorted(kwargs)}): {exc}") from exc

    def instance_provenance(self, resolution: OperatorResolution, instance) -> OperatorInstanceProvenance:
        impl_fp = implementation_fingerprint(type(instance) if not hasattr(instance, "__code__") else instance, instance=instance)
        ref = resolution.implementation.implementation_reference
        lib = native_library_fingerprint() if resolution.actual_backend.startswith("b200") else None
        return OperatorInstanceProvenance(resolution.semantic_op, resolution.actual_backend, ref, impl_fp,
                                          operator_instance_fingerprint(semantic_op=resolution.semantic_op, backend=resolution.actual_backend,
                                                                        implementation=impl_fp, native=str(lib)), lib)

    for fn in (register_backend, implementations, resolve, instantiate, instance_provenance):
        setattr(cls, fn.__name__, fn)
    return cls


_install_resolution(SemanticOperatorCatalog)
for _impl in DEFAULT_IMPLEMENTATIONS:
    semantic_catalog.register_backend(_impl)
