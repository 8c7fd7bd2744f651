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
