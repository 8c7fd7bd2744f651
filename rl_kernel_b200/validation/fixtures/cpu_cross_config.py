"""CPU-only execution target for cross-configuration smoke runs (parity: rl_engine/validation/fixtures/cpu_cross_config.py:
60-696): a tiny deterministic causal LM as an ``nn.Module``, a stateless paired scorer over it with a pluggable
selected-log-prob operator (the reference tile operator or a smoke-only one), a materialiser for the knobs a CPU run can
honour, and ``run_cpu_experiment`` which drives the paired runner with them.  Lives with the fixtures on purpose: it
implies nothing about CUDA, distributed, serving or training runtimes."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping, Sequence

import torch

from rl_kernel_b200.validation.cross_config._execution import RankScore
from rl_kernel_b200.validation.cross_config.adapters import KnobMaterializer, _only
from rl_kernel_b200.validation.cross_config.config import AlignmentExperimentConfig
from rl_kernel_b200.validation.cross_config.schema import CanonicalScoringBatch, ScorerSpec, ScoreSide
from rl_kernel_b200.validation.fixtures.smoke_ops import SMOKE_OPERATORS, load_smoke_operator


class SyntheticCpuCausalLM(torch.nn.Module):
    """Embedding -> one causal mixing layer (a cumulative mean: position t sees tokens 0..t) -> MLP -> LM head.  Small,
    seeded, and batch-invariant by construction (every row is computed from its own sequence only)."""

    def __init__(self, vocab_size: int = 4096, hidden: int = 64, seed: int = 0, dtype: torch.dtype = torch.float32):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        mk = lambda *s, sc=1.0: torch.nn.Parameter((torch.randn(*s, generator=g) * sc).to(dtype))  # noqa: E731
        self.embed = mk(vocab_size, hidden)
        self.w1, self.w2 = mk(hidden, 2 * hidden, sc=hidden ** -0.5), mk(2 * hidden, hidden, sc=(2 * hidden) ** -0.5)
        self.head = mk(vocab_size, hidden, sc=hidden ** -0.5)
        self.vocab_size = vocab_size

    def forward(self, input_ids: torch.Tensor, **_: Any) -> torch.Tensor:
        x = self.embed[input_ids].float()                                     # [B, S, H]
        steps = torch.arange(1, x.shape[1] + 1, dtype=torch.float32).view(1, -1, 1)
        ctx = torch.stack([x[:, : t + 1].sum(1) for t in range(x.shape[1])], 1) / steps     # per-position prefix mean, fixed order
        h = torch.nn.functional.silu(torch.stack([r @ self.w1.float() for r in (x + ctx)]))  # row-wise products: batch size cannot matter
        h = torch.stack([r @ self.w2.float() for r in h]) + x
        return torch.stack([r @ self.head.float().t() for r in h])              # [B, S, V]


class CpuStatelessScorer:
    """Paired scorer over an ``nn.Module`` LM.  Stateless: every call recomputes from the token ids; the selected-log-prob
    operator is chosen per case through ``options['logp_backend']``."""

    def __init__(self, side: ScoreSide | str, *, model: torch.nn.Module | None = None, dtype: str = "float32", seed: int = 0):
        self.side = ScoreSide(side)
        self.model = model if model is not None else SyntheticCpuCausalLM(seed=seed)
        for p in self.model.parameters():
            if p.device.type != "cpu":
                raise ValueError("the CPU scorer takes a model on the CPU")
            p.requires_grad_(False)
        self.model.eval()
        self.spec = ScorerSpec(self.side, "cpu.stateless_forward", dtype, "cpu", 1, {}, {"model": type(self.model).__name__, "seed": seed})

    def _operator(self, backend: str):
        if backend in SMOKE_OPERATORS:
            return load_smoke_operator(backend)
        if backend in ("native", "rlkernel.reference_logp"):
            from rl_kernel_b200.reference.logprob.tile_logp import NativeBatchInvariantLogpOp

            op = NativeBatchInvariantLogpOp()
            return lambda logits, ids: op.apply_fp32(logits.reshape(-1, logits.shape[-1]), ids.reshape(-1)).view(ids.shape)
        raise ValueError(f"the CPU scorer has no selected-log-prob backend {backend!r}")

    @torch.no_grad()
    def score(self, batch: CanonicalScoringBatch, *, options: Mapping[str, Any]) -> Sequence[RankScore]:
        op = self._operator(str(options.get("logp_backend", "native")))
        B = batch.input_ids.shape[0]
        size = int(options.get("batch_size") or B)
        rows = []
        for a in range(0, B, size):
            logits = self.model(batch.input_ids[a:a + size])
            rows.append(op(logits, batch.selected_token_ids[a:a + size]))
        dkey = "rollout.dtype" if self.side is ScoreSide.ROLLOUT else "training.compute_dtype"
        return [RankScore(0, 1, torch.cat(rows).float(), {"batch.size": size, dkey: "float32", "logp.backend": options.get("logp_backend", "native")})]


class CpuSmokeMaterializer(KnobMaterializer):
    """Knobs a CPU smoke run honours: batch size, fp32, and the log-prob backend (reference or a ``smoke_only.`` operator,
    which may differ per side through the config's explicit operator selection)."""

    def __init__(self, target: str, *, logp_backend: str | None = None):
        dkey = "rollout.dtype" if target == "rollout" else "training.compute_dtype"
        allowed = {"native", "rlkernel.reference_logp", *SMOKE_OPERATORS}
        handlers = {"batch.size": lambda v: ("batch_size", v), dkey: _only({"float32"}),
                    "logp.backend": lambda v: ("logp_backend", logp_backend or _only(allowed)(v)[1])}
        if target == "rollout":
            handlers.update({"rollout.tensor_parallel_size": _only({1}), "rollout.context_parallel_size": _only({1}),
                             "rollout.enforce_eager": _only({True, False}), "rollout.enable_prefix_caching": _only({False})})
        else:
            handlers.update({"training.attention_backend": _only({"eager", "model_default"}), "training.sharding": _only({"unsharded"})})
        super().__init__(target, handlers, implementation="cpu-smoke")


def canonical_cpu_batch(config: AlignmentExperimentConfig) -> CanonicalScoringBatch:
    return CanonicalScoringBatch.from_identity(config.definition.identity)


def run_cpu_experiment(config: AlignmentExperimentConfig, out_dir: str | Path, *, model: torch.nn.Module | None = None,
                       bitwise: bool = True, resume: bool = True) -> dict:
    """Both sides on the same CPU model; with an explicit operator selection in the config the training side may run a
    different (e.g. smoke-only offset) operator, which the run must then report as a failure."""
    from rl_kernel_b200.validation.cross_config.runner import run_alignment

    model = model if model is not None else SyntheticCpuCausalLM()
    ops = config.operators
    mats = (CpuSmokeMaterializer("rollout", logp_backend=ops.rollout_backend if ops else None),
            CpuSmokeMaterializer("training", logp_backend=ops.training_backend if ops else None))
    return run_alignment(config, out_dir, rollout=CpuStatelessScorer("rollout", model=model), training=CpuStatelessScorer("training", model=model),
                         materializers=mats, bitwise=bitwise, resume=resume)


def run_cpu_case(config: AlignmentExperimentConfig, case_index: int = 0, **kw) -> dict:
    """One planned case (by index) scored on both sides without touching the disk: -> {side: [B, S] scores, ...}."""
    case = config.plan().cases[case_index]
    batch = canonical_cpu_batch(config)
    model = kw.get("model") or SyntheticCpuCausalLM()
    from rl_kernel_b200.validation.cross_config.runtime import RuntimeTools

    m = RuntimeTools().materialize(case, (CpuSmokeMaterializer("rollout"), CpuSmokeMaterializer("training")))
    out = {"case_id": case.case_id, "status": m.case.status.value}
    for side in ("rollout", "training"):
        out[side] = CpuStatelessScorer(side, model=model).score(batch, options=dict(m.adapters[side].options))[0].selected_logprobs
    return out


__all__ = ["CpuSmokeMaterializer", "CpuStatelessScorer", "SyntheticCpuCausalLM", "canonical_cpu_batch", "run_cpu_case", "run_cpu_experiment"]
