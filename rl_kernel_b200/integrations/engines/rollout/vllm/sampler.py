"""Group rollout samplers (parity: rl_engine/integrations/engines/rollout/vllm/sampler.py:12-302).

``VLLMSharedPrefixSampler`` drives a vLLM ``LLM`` (or any object with ``generate(prompts, params)``):
each prompt is repeated ``num_generations`` times back to back so the engine's prefix cache serves the
group from one prefill, and request outputs are folded into ``NormalizedRolloutCandidate`` records
that do not depend on the vLLM version.  ``SharedPrefixSampler`` is the in-process counterpart over
this package's own engine, whose page tables share the prompt pages inside a group.
"""
from __future__ import annotations

import importlib
from dataclasses import asdict, dataclass, field
from typing import Any, Mapping, Optional, Sequence

import torch


@dataclass(frozen=True)
class VLLMSamplerConfig:
    model: Optional[str] = None
    num_generations: int = 1
    enable_prefix_caching: bool = True
    sampling_params: Mapping[str, Any] = field(default_factory=dict)
    engine_kwargs: Mapping[str, Any] = field(default_factory=dict)
    backend: str = "vllm"

    def __post_init__(self):
        if self.num_generations < 1:
            raise ValueError("num_generations must be >= 1")
        if self.backend != "vllm":
            raise ValueError(f"Unsupported rollout sampler backend: {self.backend}")

    @classmethod
    def from_model_config(cls, model_config: Optional[Mapping[str, Any]]) -> "VLLMSamplerConfig":
        """From the executor's loose dictionary: top-level keys win over ``sampler`` keys, which win over ``vllm``."""
        cfg = dict(model_config or {})
        merged: dict[str, Any] = {}
        merged.update(dict(cfg.get("vllm", {})))
        merged.update(dict(cfg.get("sampler", {})))
        merged.update({k: v for k, v in cfg.items() if k not in {"sampler", "vllm"}})
        return cls(model=merged.get("model"), num_generations=int(merged.get("num_generations", 1)),
                   enable_prefix_caching=bool(merged.get("enable_prefix_caching", True)),
                   sampling_params=dict(merged.get("sampling_params", {})), engine_kwargs=dict(merged.get("engine_kwargs", {})),
                   backend=merged.get("backend", "vllm"))


@dataclass(frozen=True)
class NormalizedRolloutCandidate:
    """Version-independent view of one generated candidate."""
    prompt_index: int
    candidate_index: int
    request_id: Optional[str]
    prompt_token_ids: Optional[list[int]]
    token_ids: list[int]
    text: str
    finish_reason: Optional[str]
    cumulative_logprob: Optional[float]
    logprobs: Optional[Any] = None
    raw_output: Optional[Any] = field(default=None, repr=False, compare=False)

    def to_dict(self, *, include_raw: bool = False) -> dict[str, Any]:
        data = asdict(self)
        if not include_raw:
            data.pop("raw_output", None)
        return data


def _get(value: Any, attr: str) -> Any:
    if isinstance(value, Mapping):
        return value.get(attr)
    return getattr(value, attr, None)


def _ints(value: Any) -> Optional[list[int]]:
    if value is None:
        return None
    if isinstance(value, torch.Tensor):
        value = value.tolist()
    try:
        return [int(v) for v in value]
    except (TypeError, ValueError):
        return None


def _float(value: Any) -> Optional[float]:
    try:
        return None if value is None else float(value)
    except (TypeError, ValueError):
        return None


def _normalize_prompts(prompts) -> list[Any]:
    if isinstance(prompts, (str, Mapping)):
        return [prompts]
    out = list(prompts)
    if not out:
        raise ValueError("at least one prompt is required")
    for p in out:
        if not isinstance(p, (str, Mapping)):
            raise TypeError(f"prompts must be strings or mappings (e.g. {{'prompt_token_ids': [...]}}); got {type(p).__name__}")
    return out


def _expand_prompts(prompts: Sequence[Any], num_generations: int) -> list[Any]:
    """[p0, p0, ..., p1, p1, ...]: a group's requests are adjacent, so the prefix cache sees them together."""
    return [p for p in prompts for _ in range(num_generations)]


def _group_outputs(outputs: Sequence[Any], num_prompts: int, num_generations: int) -> list[list[Any]]:
    outputs = list(outputs)
    if len(outputs) != num_prompts * num_generations:
        raise ValueError(f"the engine returned {len(outputs)} outputs for {num_prompts} prompts x {num_generations} generations")
    return [outputs[i * num_generations:(i + 1) * num_generations] for i in range(num_prompts)]


def normalize_output_candidate(output: Any, *, prompt_index: int, candidate_index: int) -> NormalizedRolloutCandidate:
    """One request output (``RequestOutput`` with ``outputs[0]``, a bare completion, or a mapping) -> record."""
    inner = _get(output, "outputs")
    first = inner[0] if isinstance(inner, (list, tuple)) and inner else output
    return NormalizedRolloutCandidate(
        prompt_index=prompt_index, candidate_index=candidate_index, request_id=_get(output, "request_id"),
        prompt_token_ids=_ints(_get(output, "prompt_token_ids")), token_ids=_ints(_get(first, "token_ids")) or [],
        text=str(_get(first, "text") or ""), finish_reason=_get(first, "finish_reason"),
        cumulative_logprob=_float(_get(first, "cumulative_logprob")), logprobs=_get(first, "logprobs"), raw_output=output)


def normalize_grouped_outputs(grouped: Sequence[Sequence[Any]]) -> list[list[NormalizedRolloutCandidate]]:
    return [[normalize_output_candidate(o, prompt_index=i, candidate_index=j) for j, o in enumerate(group)]
            for i, group in enumerate(grouped)]


class VLLMSharedPrefixSampler:
    """Lazy vLLM wrapper that keeps each prompt prefix byte-identical across its candidates."""

    def __init__(self, config: VLLMSamplerConfig, *, engine: Optional[Any] = None, llm_cls: Optional[type] = None,
                 sampling_params_cls: Optional[type] = None):
        self.config = config
        self._engine, self._llm_cls, self._sampling_params_cls = engine, llm_cls, sampling_params_cls

    @property
    def engine(self) -> Any:
        if self._engine is None:
            self._engine = self._build_engine()
        return self._engine

    def generate(self, prompts, *, num_generations: Optional[int] = None,
                 sampling_params: Optional[Mapping[str, Any]] = None) -> dict[str, Any]:
        plist = _normalize_prompts(prompts)
        n = num_generations or self.config.num_generations
        if n < 1:
            raise ValueError("num_generations must be >= 1")
        outputs = self.engine.generate(_expand_prompts(plist, n), self._build_sampling_params(sampling_params))
        grouped = _group_outputs(outputs, len(plist), n)
        return {"backend": self.config.backend, "prefix_cache_enabled": self.config.enable_prefix_caching,
                "num_prompts": len(plist), "num_generations": n, "outputs": grouped,
                "normalized_outputs": normalize_grouped_outputs(grouped)}

    def _load_vllm_classes(self) -> tuple[type, type]:
        if self._llm_cls is None or self._sampling_params_cls is None:
            vllm = importlib.import_module("vllm")
            self._llm_cls = self._llm_cls or vllm.LLM
            self._sampling_params_cls = self._sampling_params_cls or vllm.SamplingParams
        return self._llm_cls, self._sampling_params_cls

    def _build_engine(self) -> Any:
        if not self.config.model:
            raise ValueError("A model path or model name is required for vLLM rollout sampling.")
        llm_cls, _ = self._load_vllm_classes()
        kwargs = dict(self.config.engine_kwargs)
        kwargs.update(model=self.config.model, enable_prefix_caching=self.config.enable_prefix_caching)
        kwargs.setdefault("block_size", 128)            # the deterministic paged kernel's page
        try:
            return llm_cls(**kwargs)
        except TypeError as exc:
            raise TypeError("Failed to construct the vLLM engine with enable_prefix_caching / block_size; check that the "
                            "installed vLLM version supports these engine arguments.") from exc

    def _build_sampling_params(self, overrides: Optional[Mapping[str, Any]]) -> Any:
        _, cls = self._load_vllm_classes()
        kwargs = dict(self.config.sampling_params)
        kwargs.update(overrides or {})
        return cls(**kwargs)


class SharedPrefixSampler:
    """The same grouping over this package's own engine: ``trainer`` is a ``models.qwen3.grpo.GRPOTrainer`` whose
    rollout prefills every distinct prompt once and points the group's page tables at the same prompt pages."""

    def __init__(self, trainer):
        self.trainer = trainer

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, seed: int = 0):
        return self.trainer.rollout(prompts, step_seed=seed)

    def generate_candidates(self, prompts: torch.Tensor, seed: int = 0) -> list[list[NormalizedRolloutCandidate]]:
        """Rollout result as candidate records, [prompt][candidate]."""
        tokens, logp = self.generate(prompts, seed)              # [B * G, P + R], [B * G, R]
        G = self.trainer.cfg.group_size
        P = prompts.shape[1]
        out: list[list[NormalizedRolloutCandidate]] = []
        for i in range(prompts.shape[0]):
            group = []
            for j in range(G):
                row = i * G + j
                group.append(NormalizedRolloutCandidate(
                    prompt_index=i, candidate_index=j, request_id=f"{seed}-{i}-{j}", prompt_token_ids=_ints(tokens[row, :P]),
                    token_ids=_ints(tokens[row, P:]) or [], text="", finish_reason="length",
                    cumulative_logprob=_float(logp[row].sum()), logprobs=logp[row].tolist()))
            out.append(group)
        return out
