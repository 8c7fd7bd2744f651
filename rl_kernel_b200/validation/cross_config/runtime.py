"""Scoring backends of the cross-configuration runner (parity: rl_engine/validation/cross_config/
runtime.py:40-465, the per-case execution behind ``python -m rl_engine.validation.cross_config``).

``reference``: the CPU batch-invariant model (any dtype, simulated TP degree).
``engine``: ``Qwen3Engine`` on the sm_100a kernels of one GPU.  A case presents the SAME token sequences
differently -- whole batch, micro-batches, right-padded, prefill followed by cached decode -- and the
score of a logical token (the selected log-prob of token t+1 at position t) must not move by a bit.
Tensor / context parallel degrees above one need as many ranks: they run under ``torch.distributed``
(the multi-rank tests drive them) and are refused here when the process group does not match.
"""
from __future__ import annotations

import torch

from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
from rl_kernel_b200.validation.cross_config.config import CaseConfig, ExperimentConfig

REFERENCE_MODEL = {"layers": 2, "hidden": 256, "ffn": 768, "q_heads": 4, "kv_heads": 2, "head_dim": 64, "vocab": 4096}
ENGINE_MODEL = {"layers": 2, "hidden": 512, "ffn": 1536, "q_heads": 4, "kv_heads": 2, "head_dim": 128, "vocab": 4096}
ENGINE_KNOBS = {"batch_size", "padding", "decode_from", "operator_override", "dtype", "tp_size", "cp_size", "chunk_size"}


class UnsupportedCase(ValueError):
    """The backend cannot present the batch the way the case asks; the runner records the case as blocked."""


def sequences(exp: ExperimentConfig, vocab: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(exp.seed + 1)
    return torch.randint(0, vocab, (exp.num_sequences, exp.seq_len), generator=g)


def score_reference(exp: ExperimentConfig, case: CaseConfig) -> tuple[torch.Tensor, dict]:
    from rl_kernel_b200.models.qwen3.reference import Qwen3DenseBIModel

    spec = Qwen3DenseSpec.scaled(**{**REFERENCE_MODEL, **exp.model})
    dtype = torch.float32 if case.knobs.get("dtype", "float32") == "float32" else torch.bfloat16
    weights = Qwen3DenseWeights.synthetic(spec, dtype=dtype, seed=exp.seed)
    model = Qwen3DenseBIModel(spec, weights, execution_dtype=dtype, tp_size=case.knobs.get("tp_size", 1))
    ids = sequences(exp, spec.vocab_size)
    bs = case.knobs.get("batch_size", exp.num_sequences)
    decode_from = case.knobs.get("decode_from")
    rows = []
    for b0 in range(0, exp.num_sequences, bs):
        chunk = ids[b0:b0 + bs]
        if decode_from:
            cache = model.allocate_cache(chunk.shape[0], exp.seq_len + 1)
            pre = model(chunk[:, :decode_from], target_ids=chunk[:, :decode_from], kv_cache=cache, return_logits=False)
            cols = [pre["selected_logp"]]
            for t in range(decode_from - 1, exp.seq_len - 1):
                if t >= decode_from:
                    out = model.decode_step(chunk[:, t], torch.full((chunk.shape[0],), t), cache, return_logits=False)
                    h = out["hidden"].reshape(chunk.shape[0], -1)
                else:
                    h = pre["hidden"][:, -1]
                cols.append(model.selected_logprobs(h, chunk[:, t + 1]).unsqueeze(1))
            rows.append(torch.cat(cols, 1))
        else:
            rows.append(model(chunk, target_ids=chunk, return_logits=False)["selected_logp"])
    return torch.cat(rows), {"backend": "reference", "dtype": str(dtype), "tp_size": model.tp_size, "batch_size": bs,
                             "decode_from": decode_from}


_ENGINES: dict = {}


def _engine(exp: ExperimentConfig, device: torch.device):
    """One engine per (model, seed): cases of an experiment share the weights, as they must."""
    from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine

    key = (tuple(sorted({**ENGINE_MODEL, **exp.model}.items())), exp.seed, str(device))
    if key not in _ENGINES:
        _ENGINES.clear()
        spec = Qwen3DenseSpec.scaled(**{**ENGINE_MODEL, **exp.model})
        w = Qwen3DenseWeights.synthetic(spec, seed=exp.seed)
        _ENGINES[key] = (spec, Qwen3Engine(spec, PackedParams(spec, 0, 1, device).load(w), max_positions=max(512, 2 * exp.seq_len)))
    return _ENGINES[key]


def score_engine(exp: ExperimentConfig, case: CaseConfig, device: str = "cuda") -> tuple[torch.Tensor, dict]:
    """[num_sequences, seq_len - 1] fp32: log-prob of token t+1 given tokens 0..t, from the sm_100a engine."""
    if not torch.cuda.is_available():
        raise UnsupportedCase("the engine backend needs a CUDA device")
    k = case.knobs
    for name in ("tp_size", "cp_size"):
        if k.get(name, 1) != 1:
            raise UnsupportedCase(f"{name}={k[name]} needs {k[name]} ranks; the single-process runner holds one")
    if k.get("dtype", "bfloat16") != "bfloat16":
        raise UnsupportedCase("the engine computes in bfloat16")
    if k.get("padding", "none") == "left":
        raise UnsupportedCase("the engine addresses tokens by position from the sequence start; left padding shifts them")
    dev = torch.device(device)
    spec, eng = _engine(exp, dev)
    ids = sequences(exp, spec.vocab_size).to(dev)
    N, S, H = exp.num_sequences, exp.seq_len, spec.hidden_size
    bs = k.get("batch_size", N)
    decode_from = k.get("decode_from")
    pad = int(k.get("chunk_size") or 0) if k.get("padding") == "right" else 0     # right padding: chunk_size extra junk tokens
    if k.get("padding") == "right" and not pad:
        pad = 16
    out = torch.empty(N, S - 1, device=dev, dtype=torch.float32)
    for b0 in range(0, N, bs):
        chunk = ids[b0:b0 + bs]
        n = chunk.shape[0]
        if decode_from:
            kv = eng.new_kv_cache(n, S + 1)
            pre = eng.forward_hidden(chunk[:, :decode_from].contiguous(), kv=kv).view(n, decode_from, H)
            rows = pre[:, :-1].reshape(-1, H).contiguous()
            out[b0:b0 + n, : decode_from - 1] = eng.logp_from_hidden(rows, chunk[:, 1:decode_from].reshape(-1)).view(n, -1)
            h = pre[:, -1].contiguous().clone()
            tiles = eng.decode_tiles(n, S + 1)
            for t in range(decode_from - 1, S - 1):
                if t >= decode_from:
                    pos = torch.full((n,), t, dtype=torch.int32, device=dev)
                    h = eng.decode_step(chunk[:, t].contiguous(), pos, kv, tiles)
                out[b0:b0 + n, t] = eng.logp_from_hidden(h.contiguous(), chunk[:, t + 1].contiguous())
        else:
            toks = chunk
            if pad:
                junk = torch.full((n, pad), spec.vocab_size - 1, device=dev, dtype=chunk.dtype)
                toks = torch.cat([chunk, junk], 1).contiguous()
            hf = eng.forward_hidden(toks.contiguous()).view(n, toks.shape[1], H)
            rows = hf[:, : S - 1].reshape(-1, H).contiguous()
            out[b0:b0 + n] = eng.logp_from_hidden(rows, chunk[:, 1:].reshape(-1)).view(n, S - 1)
    torch.cuda.synchronize(dev)
    return out.cpu(), {"backend": "engine", "dtype": "torch.bfloat16", "tp_size": 1, "batch_size": bs, "decode_from": decode_from,
                       "right_pad": pad, "device": torch.cuda.get_device_name(dev)}


BACKENDS = {"reference": score_reference, "engine": score_engine}


def score_case(exp: ExperimentConfig, case: CaseConfig) -> tuple[torch.Tensor, dict]:
    backend = exp.backend if exp.backend != "auto" else ("engine" if torch.cuda.is_available() else "reference")
    return BACKENDS[backend](exp, case)


__all__ = ["BACKENDS", "ENGINE_MODEL", "REFERENCE_MODEL", "UnsupportedCase", "score_case", "score_engine", "score_reference",
           "sequences"]


# ================================================================================================ knob materialisation
# (parity: KnobApplication / RuntimeBinding / RuntimeTools, rl_engine/validation/cross_config/runtime.py:27-465)
import hashlib as _hashlib
import json as _json
from dataclasses import dataclass as _dataclass, field as _field
from typing import Any as _Any, Iterable as _Iterable, Mapping as _Mapping, Protocol as _Protocol, Sequence as _Sequence

from rl_kernel_b200.validation.cross_config.planner import V1_KNOBS as _V1_KNOBS, _flatten, _plain, _set_path
from rl_kernel_b200.validation.cross_config.schema import (ExperimentCase, IsolationScope, KnobDescriptor, MaterializationStatus,
                                                           MaterializedCase, SerializableModel, freeze)


def _fp(value) -> str:
    return _hashlib.sha256(_json.dumps(_plain(value), sort_keys=True, separators=(",", ":"), default=str).encode()).hexdigest()


@_dataclass(frozen=True)
class KnobApplication(SerializableModel):
    """What an adapter did with one knob on one target: the value it set, the value the runtime reports back, and how
    far the two can be trusted."""
    path: str
    target: str                                   # rollout | training
    requested: _Any
    materialized: _Any
    actual: _Any = None
    status: MaterializationStatus = MaterializationStatus.APPLIED
    evidence: _Mapping[str, _Any] = _field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "status", MaterializationStatus(self.status))
        object.__setattr__(self, "evidence", freeze(self.evidence))
        if self.target not in ("rollout", "training"):
            raise ValueError("target must be rollout or training")
        if self.status is MaterializationStatus.APPLIED and self.actual is not None and self.actual != self.materialized:
            raise ValueError(f"{self.path}: status APPLIED but the runtime reports {self.actual!r}, not {self.materialized!r}")


@_dataclass(frozen=True)
class AdapterMaterialization:
    target: str
    applications: tuple[KnobApplication, ...]
    options: _Mapping[str, _Any] = _field(default_factory=dict)      # what the scorer factory is called with

    def __post_init__(self) -> None:
        object.__setattr__(self, "applications", tuple(self.applications))
        object.__setattr__(self, "options", freeze(self.options))


class RuntimeMaterializer(_Protocol):
    """One side's adapter: turns normalised knob values into factory options and reports what it applied."""
    target: str

    def implementation_fingerprint(self) -> str: ...

    def materialize(self, case: ExperimentCase, normalized: _Mapping[str, _Any]) -> AdapterMaterialization: ...


@_dataclass(frozen=True)
class RuntimeMaterialization:
    case: MaterializedCase
    adapters: _Mapping[str, AdapterMaterialization]
    strict_fallback: bool = True

    @property
    def executable_in_strict_mode(self) -> bool:
        return self.case.status is MaterializationStatus.APPLIED

    @property
    def executable(self) -> bool:
        ok = {MaterializationStatus.APPLIED} | (set() if self.strict_fallback else {MaterializationStatus.FALLBACK,
                                                                                    MaterializationStatus.UNOBSERVABLE})
        return self.case.status in ok


class RuntimeMaterializationError(RuntimeError):
    pass


_STATUS_ORDER = (MaterializationStatus.ERROR, MaterializationStatus.UNSUPPORTED, MaterializationStatus.FALLBACK,
                 MaterializationStatus.UNOBSERVABLE, MaterializationStatus.APPLIED)


def aggregate_status(statuses: _Iterable[MaterializationStatus]) -> MaterializationStatus:
    """The worst status wins: one unsupported knob makes the case unsupported."""
    seen = set(statuses)
    for s in _STATUS_ORDER:
        if s in seen:
            return s
    return MaterializationStatus.APPLIED


class RuntimeTools:
    """Materialises a planned case on both sides and decides what can be reused between two cases."""

    def __init__(self, descriptors: _Mapping[str, KnobDescriptor] = _V1_KNOBS):
        self.descriptors = dict(descriptors)

    def materialize(self, case: ExperimentCase, adapters: _Sequence[RuntimeMaterializer], *, strict_fallback: bool = True
                    ) -> RuntimeMaterialization:
        flat = _flatten(case.requested)
        per_target: dict[str, AdapterMaterialization] = {}
        statuses, materialized, evidence = [], {}, {}
        for ad in adapters:
            mine = {p: v for p, v in flat.items() if p in self.descriptors and ad.target in self.descriptors[p].targets}
            try:
                m = ad.materialize(case, mine)
            except Exception as exc:  # noqa: BLE001 - an adapter failure is a case status, not a crash of the run
                statuses.append(MaterializationStatus.ERROR)
                evidence[ad.target] = {"error": f"{type(exc).__name__}: {exc}"}
                continue
            if m.target != ad.target:
                raise RuntimeMaterializationError(f"adapter for {ad.target} returned a materialisation for {m.target}")
            covered = {a.path for a in m.applications}
            missing = sorted(set(mine) - covered)
            if missing:
                raise RuntimeMaterializationError(f"{ad.target} adapter left knobs unreported: {missing}")
            per_target[ad.target] = m
            for a in m.applications:
                statuses.append(a.status)
                _set_path(materialized, f"{a.target}.{a.path}", a.materialized)
                if a.evidence:
                    evidence[f"{a.target}.{a.path}"] = dict(a.evidence)
        scopes = [self.descriptors[p].lifecycle for p in flat if p in self.descriptors]

        def scoped(scope: IsolationScope) -> str:
            return _fp({p: v for p, v in flat.items() if p in self.descriptors and self.descriptors[p].lifecycle.rank >= scope.rank})

        mc = MaterializedCase(case, case.requested, materialized,
                              max(scopes, key=lambda s: s.rank) if scopes else IsolationScope.REQUEST,
                              scoped(IsolationScope.ENGINE_CONSTRUCTION), scoped(IsolationScope.DISTRIBUTED_CONTEXT),
                              scoped(IsolationScope.PROCESS), aggregate_status(statuses), evidence)
        return RuntimeMaterialization(mc, per_target, strict_fallback)

    @staticmethod
    def require_executable(m: RuntimeMaterialization) -> None:
        if not m.executable:
            raise RuntimeMaterializationError(f"case {m.case.case.case_id} materialised as {m.case.status.value}: "
                                              f"{dict(m.case.evidence)}")

    @staticmethod
    def can_reuse(previous: RuntimeMaterialization, current: RuntimeMaterialization) -> str:
        """What survives from the previous case: 'engine' (only request-level knobs moved), 'context' (rebuild the engine
        inside the same distributed context), 'process' (same process, new context) or 'nothing'."""
        a, b = previous.case, current.case
        if a.process_fingerprint != b.process_fingerprint:
            return "nothing"
        if a.distributed_context_fingerprint != b.distributed_context_fingerprint:
            return "process"
        if a.construction_fingerprint != b.construction_fingerprint:
            return "context"
        return "engine"


__all__ += ["AdapterMaterialization", "KnobApplication", "RuntimeMaterialization", "RuntimeMaterializationError", "RuntimeMaterializer",
            "RuntimeTools", "aggregate_status"]
