"""Executing one paired case (parity: rl_engine/validation/cross_config/_execution.py:28-617).

A *paired scorer* scores the canonical batch on one side and returns one ``RankScore`` per rank of
its world.  Scoring must be read-only: a guard fingerprints the scorer's model state before and
after and fails the case if anything moved.  Rank outputs are validated for completeness (every
rank once, one world size, TP-replicated bits) before rank 0's score becomes the side's artifact.
Scorers that need their own process group run in supervised child processes with a deadline; the
supervisor kills exactly the children it started.
"""
from __future__ import annotations

import contextlib
import hashlib
import inspect
import multiprocessing as mp
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Iterator, Mapping, Optional, Protocol, Sequence

import torch

from rl_kernel_b200.validation.cross_config._provenance import canonical_fingerprint
from rl_kernel_b200.validation.cross_config.schema import CanonicalScoringBatch, ScorerSpec, ScoreSide


class PairedRunnerError(RuntimeError):
    pass


class OperatorExecutionError(PairedRunnerError):
    pass


class ChildScoringError(PairedRunnerError):
    pass


class ScoringTimeoutError(PairedRunnerError):
    pass


class RankCompletenessError(PairedRunnerError):
    pass


class ScorerIdentityError(PairedRunnerError):
    pass


@dataclass(frozen=True)
class RankScore:
    rank: int
    world_size: int
    selected_logprobs: torch.Tensor          # [B, S] fp32; entries outside active_mask are ignored
    actual: Mapping[str, Any] = field(default_factory=dict)       # knob values read back from the runtime

    def __post_init__(self) -> None:
        if self.world_size < 1 or not 0 <= self.rank < self.world_size:
            raise ValueError("rank must lie in [0, world_size)")
        if not isinstance(self.selected_logprobs, torch.Tensor) or self.selected_logprobs.dim() != 2:
            raise ValueError("selected_logprobs must be a [batch, seq] tensor")
        object.__setattr__(self, "selected_logprobs", self.selected_logprobs.detach().float().cpu())
        object.__setattr__(self, "actual", dict(self.actual))


class PairedScorer(Protocol):
    spec: ScorerSpec

    def score(self, batch: CanonicalScoringBatch, *, options: Mapping[str, Any]) -> Sequence[RankScore]: ...


# ------------------------------------------------------------------------------------------------ identity
def scorer_spec(scorer: PairedScorer, expected_side: ScoreSide) -> ScorerSpec:
    spec = getattr(scorer, "spec", None)
    if not isinstance(spec, ScorerSpec):
        raise ScorerIdentityError(f"{type(scorer).__name__} has no ScorerSpec")
    if spec.side is not expected_side:
        raise ScorerIdentityError(f"{type(scorer).__name__} scores the {spec.side.value} side, expected {expected_side.value}")
    return spec


def validate_scorer_identity(rollout: PairedScorer, training: PairedScorer) -> tuple[ScorerSpec, ScorerSpec]:
    r, t = scorer_spec(rollout, ScoreSide.ROLLOUT), scorer_spec(training, ScoreSide.TRAINING)
    if rollout is training:
        raise ScorerIdentityError("the two sides must be scored by two scorer objects")
    return r, t


def _source_text(obj: Any) -> str:
    try:
        return inspect.getsource(obj if inspect.isclass(obj) or inspect.isfunction(obj) else type(obj))
    except (OSError, TypeError):
        return repr(type(obj))


def scorer_implementation_fingerprint(scorer: PairedScorer) -> str:
    return canonical_fingerprint({"class": f"{type(scorer).__module__}.{type(scorer).__qualname__}",
                                  "source": hashlib.sha256(_source_text(scorer).encode()).hexdigest(),
                                  "spec": scorer.spec.to_dict()})


# ------------------------------------------------------------------------------------------------ read-only guard
def scorer_state_tensors(scorer: PairedScorer) -> dict[str, torch.Tensor]:
    """Tensors that make up the scorer's model: an ``nn.Module`` at ``.model``, or a name -> tensor mapping returned by
    ``state_tensors()`` (the engine's packed parameter shards)."""
    fn = getattr(scorer, "state_tensors", None)
    if callable(fn):
        return dict(fn())
    model = getattr(scorer, "model", None)
    if isinstance(model, torch.nn.Module):
        return {**dict(model.named_parameters()), **dict(model.named_buffers())}
    return {}


def _tensor_digest(t: torch.Tensor) -> str:
    t = t.detach()
    if t.numel() > (1 << 22):                              # large shards: exact checksums on the device, no host copy
        v = t.contiguous().view(torch.uint8).view(-1)
        n = v.numel() // 8 * 8
        words = v[:n].view(torch.int64)
        return f"{tuple(t.shape)}:{t.dtype}:{int(words.sum())}:{int((words * torch.arange(1, words.numel() + 1, device=words.device)).sum())}:{int(v[n:].sum())}"
    return hashlib.sha256(str((t.dtype, tuple(t.shape))).encode() + t.contiguous().cpu().view(torch.uint8).numpy().tobytes()).hexdigest()


def model_state_fingerprint(scorer: PairedScorer) -> Optional[str]:
    tensors = scorer_state_tensors(scorer)
    if not tensors:
        return None
    return canonical_fingerprint({k: _tensor_digest(v) for k, v in sorted(tensors.items())})


def paired_model_state_fingerprints(rollout: PairedScorer, training: PairedScorer) -> dict[str, Optional[str]]:
    return {"rollout": model_state_fingerprint(rollout), "training": model_state_fingerprint(training)}


@contextlib.contextmanager
def read_only_scoring_guard(scorer: PairedScorer) -> Iterator[None]:
    """Scoring may not change the model: any parameter or buffer whose digest moved fails the case."""
    before = {k: _tensor_digest(v) for k, v in scorer_state_tensors(scorer).items()}
    yield
    after = {k: _tensor_digest(v) for k, v in scorer_state_tensors(scorer).items()}
    moved = sorted(k for k in before if after.get(k) != before[k]) + sorted(set(after) - set(before))
    if moved:
        raise OperatorExecutionError(f"scoring mutated model state: {moved[:8]}{' ...' if len(moved) > 8 else ''}")


# ------------------------------------------------------------------------------------------------ rank outputs
def validate_rank_outputs(scores: Sequence[RankScore], batch: CanonicalScoringBatch, *, expected_world_size: Optional[int] = None,
                          replicated: bool = True) -> RankScore:
    """Every rank exactly once, one world size, the batch's shape, finite active scores and -- when the ranks hold
    replicas of the result -- equal bits on all of them.  Returns rank 0's score."""
    if not scores:
        raise RankCompletenessError("the scorer returned no rank outputs")
    world = scores[0].world_size
    if expected_world_size is not None and world != expected_world_size:
        raise RankCompletenessError(f"scorer ran on {world} ranks, the case asks for {expected_world_size}")
    ranks = sorted(s.rank for s in scores)
    if any(s.world_size != world for s in scores) or ranks != list(range(world)):
        raise RankCompletenessError(f"expected ranks 0..{world - 1} once each, got {ranks}")
    by_rank = {s.rank: s for s in scores}
    shape = tuple(batch.input_ids.shape)
    mask = batch.active_mask
    for s in scores:
        if tuple(s.selected_logprobs.shape) != shape:
            raise RankCompletenessError(f"rank {s.rank} returned shape {tuple(s.selected_logprobs.shape)}, expected {shape}")
        if not bool(torch.isfinite(s.selected_logprobs[mask]).all()):
            raise OperatorExecutionError(f"rank {s.rank} returned non-finite scores on active tokens")
    if replicated:
        ref = by_rank[0].selected_logprobs[mask].view(torch.int32)
        for r in range(1, world):
            if not torch.equal(by_rank[r].selected_logprobs[mask].view(torch.int32), ref):
                raise RankCompletenessError(f"rank {r} does not hold the bits rank 0 holds")
    return by_rank[0]


# ------------------------------------------------------------------------------------------------ supervised children
def _child_entry(fn: Callable, args: tuple, out_path: str) -> None:
    try:
        torch.save({"ok": True, "value": fn(*args)}, out_path)
    except BaseException as exc:  # noqa: BLE001 - the parent needs the reason whatever it was
        import traceback

        torch.save({"ok": False, "error": f"{type(exc).__name__}: {exc}", "traceback": traceback.format_exc()}, out_path)
        raise


class ChildSupervisor:
    """Runs ``fn(rank, *args)`` in ``nprocs`` children with a deadline and returns their saved values in rank order."""

    def __init__(self, start_method: Optional[str] = None):
        self.start_method = start_method or "spawn"
        self.ctx = mp.get_context(self.start_method)
        self._children: list = []

    def active_child_pids(self) -> tuple[int, ...]:
        return tuple(p.pid for p in self._children if p.is_alive())

    def run(self, fn: Callable, args: tuple, *, nprocs: int, work_dir: Path, timeout_s: float = 600.0) -> list[Any]:
        work_dir.mkdir(parents=True, exist_ok=True)
        outs = [work_dir / f"rank{r}.pt" for r in range(nprocs)]
        self._children = [self.ctx.Process(target=_child_entry, args=(fn, (r, *args), str(outs[r])), daemon=False)
                          for r in range(nprocs)]
        for p in self._children:
            p.start()
        try:
            self._wait(timeout_s)
        finally:
            self._stop()
        results = []
        for r, path in enumerate(outs):
            if not path.exists():
                raise ChildScoringError(f"rank {r} exited without a result")
            payload = torch.load(path, weights_only=False)
            if not payload.get("ok"):
                raise ChildScoringError(f"rank {r}: {payload.get('error')}\n{payload.get('traceback', '')}")
            results.append(payload["value"])
        return results

    def _wait(self, timeout_s: float) -> None:
        deadline = time.monotonic() + timeout_s
        while True:
            alive = [p for p in self._children if p.is_alive()]
            failed = [p for p in self._children if not p.is_alive() and p.exitcode not in (0, None)]
            if failed or not alive:
                return
            if time.monotonic() > deadline:
                raise ScoringTimeoutError(f"scoring children still running after {timeout_s:.0f} s")
            time.sleep(0.05)

    def _stop(self) -> None:
        for p in self._children:                      # exactly the processes this supervisor started
            if p.is_alive():
                p.terminate()
        for p in self._children:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=5)


def device_type(value: str) -> str:
    return str(value).split(":")[0]


def torch_dtype(value: str) -> torch.dtype:
    name = {"bf16": "bfloat16", "fp16": "float16", "half": "float16", "fp32": "float32", "float": "float32"}.get(
        str(value).removeprefix("torch."), str(value).removeprefix("torch."))
    dt = getattr(torch, name, None)
    if not isinstance(dt, torch.dtype):
        raise ValueError(f"unknown dtype {value!r}")
    return dt


__all__ = ["ChildScoringError", "ChildSupervisor", "OperatorExecutionError", "PairedRunnerError", "PairedScorer", "RankCompletenessError",
           "RankScore", "ScorerIdentityError", "ScoringTimeoutError", "device_type", "model_state_fingerprint",
           "paired_model_state_fingerprints", "read_only_scoring_guard", "scorer_implementation_fingerprint", "scorer_spec",
           "scorer_state_tensors", "torch_dtype", "validate_rank_outputs", "validate_scorer_identity"]
