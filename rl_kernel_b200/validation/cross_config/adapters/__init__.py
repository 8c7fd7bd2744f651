"""Scorers and knob materialisers of the paired runner (parity: rl_engine/validation/cross_config/adapters/ and the
per-framework ``cross_config`` adapters it loads).

``ReferenceModelScorer`` scores with the CPU batch-invariant model, ``EngineScorer`` with ``Qwen3Engine`` on the
sm_100a kernels.  On the rollout side both follow the path a rollout engine takes -- prefill of the first
``prefill_tokens`` positions into a KV cache, then one cached decode step per position -- and on the training side the
path a trainer takes: one full forward over the whole sequence.  Both paths score ``selected_token_ids[b, t]`` from
the hidden state at position t, so a pair of artifacts compares a sampled token's log-prob as the sampler saw it with
the one the loss sees.  ``KnobMaterializer`` maps the planner's knobs onto scorer options and reports every knob it
cannot honour as UNSUPPORTED instead of ignoring it.
"""
from __future__ import annotations

from typing import Any, Callable, Mapping, Sequence

import torch

from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
from rl_kernel_b200.validation.cross_config._execution import RankScore
from rl_kernel_b200.validation.cross_config._provenance import canonical_fingerprint
from rl_kernel_b200.validation.cross_config.runtime import AdapterMaterialization, ENGINE_MODEL, KnobApplication, REFERENCE_MODEL
from rl_kernel_b200.validation.cross_config.schema import (CanonicalScoringBatch, ExperimentCase, MaterializationStatus, ScorerSpec,
                                                           ScoreSide)


def _micro_batches(n: int, size: int | None) -> list[tuple[int, int]]:
    size = size or n
    return [(a, min(n, a + size)) for a in range(0, n, size)]


class ReferenceModelScorer:
    """CPU reference model; fp32 or bf16; ``tensor_parallel_size`` simulates the TP reduction trees in one process."""

    def __init__(self, side: ScoreSide | str, *, dtype: str = "float32", model: Mapping[str, int] | None = None, seed: int = 0,
                 prefill_tokens: int | None = None):
        self.side = ScoreSide(side)
        self.dtype = torch.float32 if dtype == "float32" else torch.bfloat16
        self.geometry = {**REFERENCE_MODEL, **(model or {})}
        self.seed, self.prefill_tokens = seed, prefill_tokens
        self.spec = ScorerSpec(self.side, "rlkernel.reference_model", dtype, "cpu", 1, {}, {"model": self.geometry, "seed": seed})
        self._spec = Qwen3DenseSpec.scaled(**self.geometry)
        self._weights = Qwen3DenseWeights.synthetic(self._spec, dtype=self.dtype, seed=seed)
        self._models: dict[int, Any] = {}

    def state_tensors(self) -> dict[str, torch.Tensor]:
        return dict(self._weights.items())

    def _model(self, tp: int):
        from rl_kernel_b200.models.qwen3.reference import Qwen3DenseBIModel

        if tp not in self._models:
            self._models[tp] = Qwen3DenseBIModel(self._spec, self._weights, execution_dtype=self.dtype, tp_size=tp)
        return self._models[tp]

    @torch.no_grad()
    def score(self, batch: CanonicalScoringBatch, *, options: Mapping[str, Any]) -> Sequence[RankScore]:
        model = self._model(int(options.get("tensor_parallel_size", 1)))
        ids, sel = batch.input_ids, batch.selected_token_ids
        B, S = ids.shape
        out = torch.zeros(B, S)
        for a, b in _micro_batches(B, options.get("batch_size")):
            x, tg = ids[a:b], sel[a:b]
            if self.side is ScoreSide.ROLLOUT:
                p = int(self.prefill_tokens or max(1, S // 2))
                cache = model.allocate_cache(b - a, S + 1)
                pre = model(x[:, :p], kv_cache=cache, return_logits=False)
                out[a:b, :p] = model.selected_logprobs(pre["hidden"].reshape((b - a) * p, -1), tg[:, :p].reshape(-1)).view(b - a, p)
                for t in range(p, S):
                    step = model.decode_step(x[:, t], torch.full((b - a,), t), cache, return_logits=False)
                    out[a:b, t] = model.selected_logprobs(step["hidden"].reshape(b - a, -1), tg[:, t])
            else:
                hid = model(x, return_logits=False)["hidden"]
                out[a:b] = model.selected_logprobs(hid.reshape((b - a) * S, -1), tg.reshape(-1)).view(b - a, S)
        actual = {"batch.size": int(options.get("batch_size") or B), f"{self.side.value}.tensor_parallel_size": model.tp_size,
                  f"{'rollout.dtype' if self.side is ScoreSide.ROLLOUT else 'training.compute_dtype'}": str(self.dtype).removeprefix("torch.")}
        return [RankScore(0, 1, out, actual)]


class EngineScorer:
    """``Qwen3Engine`` on one GPU (bf16).  Needs CUDA; construction fails loudly without it."""

    def __init__(self, side: ScoreSide | str, *, model: Mapping[str, int] | None = None, seed: int = 0, device: str = "cuda",
                 prefill_tokens: int | None = None):
        if not torch.cuda.is_available():
            raise RuntimeError("EngineScorer needs a CUDA device")
        from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine

        self.side = ScoreSide(side)
        self.geometry = {**ENGINE_MODEL, **(model or {})}
        self.dev = torch.device(device)
        self.prefill_tokens = prefill_tokens
        self._spec = Qwen3DenseSpec.scaled(**self.geometry)
        self.params = PackedParams(self._spec, 0, 1, self.dev).load(Qwen3DenseWeights.synthetic(self._spec, seed=seed))
        self.engine = Qwen3Engine(self._spec, self.params, max_positions=4096)
        self.spec = ScorerSpec(self.side, "rlkernel.b200_engine", "bfloat16", str(self.dev), 1, {"tp": 1, "cp": 1},
                               {"model": self.geometry, "seed": seed})

    def state_tensors(self) -> dict[str, torch.Tensor]:
        return dict(self.params.w)

    @torch.no_grad()
    def score(self, batch: CanonicalScoringBatch, *, options: Mapping[str, Any]) -> Sequence[RankScore]:
        eng, H = self.engine, self._spec.hidden_size
        ids, sel = batch.input_ids.to(self.dev), batch.selected_token_ids.to(self.dev)
        B, S = ids.shape
        out = torch.zeros(B, S, device=self.dev)
        for a, b in _micro_batches(B, options.get("batch_size")):
            x, tg, n = ids[a:b].contiguous(), sel[a:b].contiguous(), b - a
            if self.side is ScoreSide.ROLLOUT:
                p = int(self.prefill_tokens or max(1, S // 2))
                kv = eng.new_kv_cache(n, S + 1)
                pre = eng.forward_hidden(x[:, :p].contiguous(), kv=kv).view(n, p, H)
                out[a:b, :p] = eng.logp_from_hidden(pre.reshape(-1, H).contiguous(), tg[:, :p].reshape(-1)).view(n, p)
                tiles = eng.decode_tiles(n, S + 1)
                for t in range(p, S):
                    h = eng.decode_step(x[:, t].contiguous(), torch.full((n,), t, dtype=torch.int32, device=self.dev), kv, tiles)
                    out[a:b, t] = eng.logp_from_hidden(h.contiguous(), tg[:, t].contiguous())
            else:
                hf = eng.forward_hidden(x)
                out[a:b] = eng.logp_from_hidden(hf.reshape(-1, H).contiguous(), tg.reshape(-1)).view(n, S)
        torch.cuda.synchronize(self.dev)
        dkey = "rollout.dtype" if self.side is ScoreSide.ROLLOUT else "training.compute_dtype"
        return [RankScore(0, 1, out.cpu(), {"batch.size": int(options.get("batch_size") or B), dkey: "bfloat16",
                                            f"{self.side.value}.tensor_parallel_size": 1})]


class KnobMaterializer:
    """Maps knob paths onto scorer options.  ``handlers[path](value) -> (option_name, option_value)`` or raises
    ``ValueError`` for a value the runtime cannot honour; paths without a handler are UNSUPPORTED."""

    def __init__(self, target: str, handlers: Mapping[str, Callable[[Any], tuple[str, Any]]], *, implementation: str = ""):
        self.target, self.handlers, self._impl = target, dict(handlers), implementation

    def implementation_fingerprint(self) -> str:
        return canonical_fingerprint({"target": self.target, "paths": sorted(self.handlers), "implementation": self._impl})

    def materialize(self, case: ExperimentCase, normalized: Mapping[str, Any]) -> AdapterMaterialization:
        apps, options = [], {}
        for path, value in sorted(normalized.items()):
            h = self.handlers.get(path)
            if h is None:
                apps.append(KnobApplication(path, self.target, value, None, None, MaterializationStatus.UNSUPPORTED,
                                            {"reason": f"the {self.target} adapter has no handler for this knob"}))
                continue
            try:
                name, mat = h(value)
            except ValueError as exc:
                apps.append(KnobApplication(path, self.target, value, None, None, MaterializationStatus.UNSUPPORTED, {"reason": str(exc)}))
                continue
            if name:
                options[name] = mat
            apps.append(KnobApplication(path, self.target, value, mat, None, MaterializationStatus.APPLIED))
        return AdapterMaterialization(self.target, tuple(apps), options)


def _only(allowed, name: str = ""):
    def h(v):
        if v not in allowed:
            raise ValueError(f"this runtime supports {sorted(allowed, key=str)} only")
        return name, v

    return h


def reference_materializers() -> tuple[KnobMaterializer, KnobMaterializer]:
    """Knobs the CPU reference scorers honour: batch size, simulated TP, dtype, the reference log-prob backend."""
    common = {"batch.size": lambda v: ("batch_size", v), "logp.backend": _only({"native", "rlkernel.reference_logp"})}
    ro = KnobMaterializer("rollout", {**common, "rollout.tensor_parallel_size": lambda v: ("tensor_parallel_size", v),
                                      "rollout.context_parallel_size": _only({1}), "rollout.dtype": _only({"float32", "bfloat16"}),
                                      "rollout.enforce_eager": _only({True, False}), "rollout.enable_prefix_caching": _only({False})},
                          implementation="reference")
    tr = KnobMaterializer("training", {**common, "training.compute_dtype": _only({"float32", "bfloat16"}),
                                       "training.attention_backend": _only({"eager", "model_default"}),
                                       "training.sharding": _only({"unsharded"})}, implementation="reference")
    return ro, tr


def engine_materializers() -> tuple[KnobMaterializer, KnobMaterializer]:
    """Knobs the single-GPU engine scorers honour."""
    common = {"batch.size": lambda v: ("batch_size", v), "logp.backend": _only({"native", "rlkernel.b200_linear_logp"})}
    ro = KnobMaterializer("rollout", {**common, "rollout.tensor_parallel_size": _only({1}), "rollout.context_parallel_size": _only({1}),
                                      "rollout.dtype": _only({"bfloat16"}), "rollout.enforce_eager": _only({True, False}),
                                      "rollout.enable_prefix_caching": _only({False})}, implementation="b200-engine")
    tr = KnobMaterializer("training", {**common, "training.compute_dtype": _only({"bfloat16"}),
                                       "training.attention_backend": _only({"model_default"}),
                                       "training.sharding": _only({"unsharded"})}, implementation="b200-engine")
    return ro, tr


__all__ = ["EngineScorer", "KnobMaterializer", "ReferenceModelScorer", "engine_materializers", "reference_materializers"]
