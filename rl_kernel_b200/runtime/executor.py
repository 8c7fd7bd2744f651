"""Stateless forward executor: scores sequences with a frozen policy (reference / reward scoring)
without any KV cache, in micro-batches, and reports metrics (parity: StatelessForwardExecutor,
rl_engine/runtime/executor.py:95-272)."""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch


@dataclass
class ScoreMetrics:
    sequences: int = 0
    tokens: int = 0
    seconds: float = 0.0
    micro_batches: int = 0
    backend: str = ""
    extra: dict = field(default_factory=dict)

    @property
    def tokens_per_s(self) -> float:
        return self.tokens / self.seconds if self.seconds > 0 else 0.0


class StatelessForwardExecutor:
    """``model`` is anything with ``forward(input_ids, target_ids=...) -> {"selected_logp": ...}``
    (the reference model) or a ``score(tokens) -> logp`` callable (the sm_100a trainer)."""

    def __init__(self, model, micro_batch: int = 8, reject_kv_cache: bool = True):
        self.model, self.micro_batch, self.reject_kv_cache = model, micro_batch, reject_kv_cache
        self.metrics = ScoreMetrics(backend=type(model).__name__)

    @torch.no_grad()
    def score(self, input_ids: torch.Tensor, loss_mask: torch.Tensor | None = None, **kwargs) -> torch.Tensor:
        if self.reject_kv_cache and kwargs.get("kv_cache") is not None:
            raise ValueError("the stateless executor scores without a KV cache")
        t0 = time.perf_counter()
        outs = []
        for b0 in range(0, input_ids.shape[0], self.micro_batch):
            ids = input_ids[b0:b0 + self.micro_batch]
            if callable(getattr(self.model, "score", None)):
                lp = self.model.score(ids)
            else:
                lp = self.model.forward(ids, target_ids=ids, return_logits=False)["selected_logp"]
            outs.append(lp)
            self.metrics.micro_batches += 1
        out = torch.cat(outs)
        if loss_mask is not None:
            out = out.masked_fill(~loss_mask[:, -out.shape[1]:].bool(), 0.0)
        if out.is_cuda:
            torch.cuda.synchronize(out.device)
        self.metrics.sequences += input_ids.shape[0]
        self.metrics.tokens += input_ids.numel()
        self.metrics.seconds += time.perf_counter() - t0
        return out


def score_reference_logprobs(model, input_ids, loss_mask=None, micro_batch: int = 8) -> torch.Tensor:
    return StatelessForwardExecutor(model, micro_batch).score(input_ids, loss_mask)


# ================================================================================================ nn.Module scoring
# (parity: StatelessForwardConfig / Inputs / Outputs / Result, attention-backend fallback, reward scoring and metrics of
#  rl_engine/runtime/executor.py:24-672)
from typing import Any, Callable, Optional


@dataclass(frozen=True)
class StatelessForwardConfig:
    micro_batch: int = 8
    temperature: float = 1.0
    attention_backend: Optional[str] = None            # e.g. "flash_attention_2"; None keeps the model's own
    attention_backend_fallbacks: tuple[str, ...] = ("sdpa", "eager")
    reject_kv_cache: bool = True
    use_cache: bool = False
    output_dtype: torch.dtype = torch.float32

    def __post_init__(self) -> None:
        if self.micro_batch <= 0:
            raise ValueError("micro_batch must be positive")
        if not self.temperature > 0:
            raise ValueError("temperature must be positive")
        if self.use_cache:
            raise ValueError("the stateless executor never asks a model for a KV cache")


@dataclass(frozen=True)
class StatelessForwardInputs:
    input_ids: torch.Tensor                    # [B, S]
    attention_mask: Optional[torch.Tensor] = None
    completion_mask: Optional[torch.Tensor] = None      # [B, S] or [B, L] (the last L positions)
    position_ids: Optional[torch.Tensor] = None


@dataclass
class StatelessForwardOutputs:
    selected_logprobs: torch.Tensor            # [B, S - 1]: log p(token t+1 | tokens 0..t), masked entries 0
    logits: Optional[torch.Tensor] = None


@dataclass
class TensorTreeSummary:
    tensors: int = 0
    nbytes: int = 0

    @property
    def total_mb(self) -> float:
        return self.nbytes / 2 ** 20


@dataclass
class StatelessForwardResult:
    outputs: StatelessForwardOutputs
    metrics: dict
    attention_backend: Optional[str]
    fallback_reason: Optional[str] = None


def summarize_tensor_tree(value: Any) -> TensorTreeSummary:
    s = TensorTreeSummary()

    def visit(node):
        if isinstance(node, torch.Tensor):
            s.tensors += 1
            s.nbytes += node.numel() * node.element_size()
        elif isinstance(node, dict):
            for v in node.values():
                visit(v)
        elif isinstance(node, (list, tuple)):
            for v in node:
                visit(v)
        elif hasattr(node, "__dict__") and not isinstance(node, type):
            for v in vars(node).values():
                visit(v)

    visit(value)
    return s


def extract_kv_cache_outputs(raw_outputs: Any) -> Optional[Any]:
    """The KV cache a model returned, if it returned one (``past_key_values`` attribute / key)."""
    if raw_outputs is None or isinstance(raw_outputs, torch.Tensor):
        return None
    if isinstance(raw_outputs, dict):
        return raw_outputs.get("past_key_values")
    return getattr(raw_outputs, "past_key_values", None)


def _model_configs(model) -> list:
    out, seen = [], set()
    for m in [model, getattr(model, "model", None), getattr(model, "module", None)]:
        cfg = getattr(m, "config", None)
        if cfg is not None and id(cfg) not in seen:
            seen.add(id(cfg))
            out.append(cfg)
    return out


class _temporarily_configured:
    """Sets ``use_cache=False`` (and an attention implementation) on the model's config objects for one call and restores them."""

    def __init__(self, model, attention_backend: Optional[str]):
        self.model, self.backend, self.saved = model, attention_backend, []

    def __enter__(self):
        for cfg in _model_configs(self.model):
            for name, val in (("use_cache", False), ("_attn_implementation", self.backend)):
                if val is None and name != "use_cache":
                    continue
                if hasattr(cfg, name):
                    self.saved.append((cfg, name, getattr(cfg, name)))
                    setattr(cfg, name, val)
        return self

    def __exit__(self, *exc):
        for cfg, name, val in reversed(self.saved):
            setattr(cfg, name, val)
        return False


def _should_fallback(exc: Exception) -> bool:
    text = str(exc).lower()
    return isinstance(exc, (ImportError, NotImplementedError, ValueError, RuntimeError)) and any(
        w in text for w in ("flash", "attention", "attn_implementation", "sdpa", "not supported", "not installed"))


class ModuleForwardExecutor:
    """Scores an ``nn.Module`` causal LM without a KV cache: micro-batches, selected log-probs through this framework's
    log-prob operator, an attention implementation with a fallback chain, and per-call metrics."""

    def __init__(self, model: torch.nn.Module, config: StatelessForwardConfig | None = None):
        self.model, self.config = model, config or StatelessForwardConfig()

    def _forward(self, ids, mask, pos, backend):
        from rl_kernel_b200.models.wrappers import extract_logits

        kw = {}
        if mask is not None:
            kw["attention_mask"] = mask
        if pos is not None:
            kw["position_ids"] = pos
        with _temporarily_configured(self.model, backend):
            raw = self.model(ids, **kw)
        if self.config.reject_kv_cache and extract_kv_cache_outputs(raw) is not None:
            raise ValueError("the model returned a KV cache; the stateless executor scores without one")
        return extract_logits(raw)

    @torch.no_grad()
    def score(self, inputs: StatelessForwardInputs) -> StatelessForwardResult:
        from rl_kernel_b200.ops.logprob import logp_from_logits

        c = self.config
        ids = inputs.input_ids
        if ids.dim() != 2 or ids.shape[1] < 2:
            raise ValueError("input_ids must be [B, S] with S >= 2")
        B, S = ids.shape
        chain = [c.attention_backend] + [b for b in c.attention_backend_fallbacks if b != c.attention_backend] if c.attention_backend else [None]
        t0 = time.perf_counter()
        backend_used, reason, rows, peak = None, None, [], TensorTreeSummary()
        for b0 in range(0, B, c.micro_batch):
            sl = slice(b0, b0 + c.micro_batch)
            logits = None
            for i, backend in enumerate(chain if backend_used is None else [backend_used]):
                try:
                    logits = self._forward(ids[sl], None if inputs.attention_mask is None else inputs.attention_mask[sl],
                                           None if inputs.position_ids is None else inputs.position_ids[sl], backend)
                    backend_used = backend
                    break
                except Exception as exc:  # noqa: BLE001 - only attention-backend problems move down the chain
                    if i + 1 < len(chain) and _should_fallback(exc):
                        reason = f"{backend}: {type(exc).__name__}: {exc}"
                        continue
                    raise
            lp = logp_from_logits(logits[:, :-1].reshape(-1, logits.shape[-1]), ids[sl, 1:].reshape(-1), temperature=c.temperature)
            rows.append(lp.view(-1, S - 1).to(c.output_dtype))
            s = summarize_tensor_tree(logits)
            peak = s if s.nbytes > peak.nbytes else peak
        out = torch.cat(rows)
        cm = inputs.completion_mask
        if cm is not None:
            cm = cm.bool()
            m = cm[:, 1:] if cm.shape[1] == S else torch.cat([torch.zeros(B, S - 1 - cm.shape[1], dtype=torch.bool, device=cm.device), cm], 1)
            out = out.masked_fill(~m.to(out.device), 0.0)
        if out.is_cuda:
            torch.cuda.synchronize(out.device)
        dt = time.perf_counter() - t0
        metrics = {"sequences": B, "tokens": int(ids.numel()), "seconds": dt, "tokens_per_s": ids.numel() / dt if dt > 0 else 0.0,
                   "micro_batches": (B + c.micro_batch - 1) // c.micro_batch, "peak_logits_mb": peak.total_mb}
        return StatelessForwardResult(StatelessForwardOutputs(out), metrics, backend_used, reason)


def default_reward_adapter(raw_outputs: Any) -> torch.Tensor:
    """A reward model's scalar per sequence: ``.rewards`` / ``.logits`` / ``.scores`` / the tensor itself, squeezed to [B]."""
    for name in ("rewards", "scores", "logits"):
        v = raw_outputs.get(name) if isinstance(raw_outputs, dict) else getattr(raw_outputs, name, None)
        if isinstance(v, torch.Tensor):
            raw_outputs = v
            break
    if not isinstance(raw_outputs, torch.Tensor):
        raise TypeError("cannot find a reward tensor in the model output")
    t = raw_outputs.float()
    while t.dim() > 1 and t.shape[-1] == 1:
        t = t.squeeze(-1)
    if t.dim() == 2:                                   # per-position scores: the last position carries the reward
        t = t[:, -1]
    return t


@torch.no_grad()
def score_rewards(model: torch.nn.Module, input_ids: torch.Tensor, *, attention_mask: Optional[torch.Tensor] = None, micro_batch: int = 8,
                  adapter: Callable[[Any], torch.Tensor] = default_reward_adapter) -> torch.Tensor:
    out = []
    for b0 in range(0, input_ids.shape[0], micro_batch):
        kw = {} if attention_mask is None else {"attention_mask": attention_mask[b0:b0 + micro_batch]}
        out.append(adapter(model(input_ids[b0:b0 + micro_batch], **kw)))
    return torch.cat(out)


def collect_stateless_metrics(*results: StatelessForwardResult) -> dict:
    tok = sum(r.metrics["tokens"] for r in results)
    sec = sum(r.metrics["seconds"] for r in results)
    return {"calls": len(results), "tokens": tok, "seconds": sec, "tokens_per_s": tok / sec if sec > 0 else 0.0,
            "fallbacks": [r.fallback_reason for r in results if r.fallback_reason],
            "peak_logits_mb": max((r.metrics["peak_logits_mb"] for r in results), default=0.0)}
