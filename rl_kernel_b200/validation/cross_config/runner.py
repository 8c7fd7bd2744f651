"""Cross-configuration log-prob drift runner: score the same sequences under several
configurations (batching, padding, decode vs prefill, simulated TP degree, operator overrides) and
compare every case with the reference case token by token, bit by bit (parity:
``python -m rl_engine.validation.cross_config``)."""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys
from pathlib import Path

import torch

from rl_kernel_b200.validation.cross_config.artifacts import AttemptStore
from rl_kernel_b200.validation.cross_config.config import CaseConfig, ExperimentConfig
from rl_kernel_b200.validation.cross_config.runtime import REFERENCE_MODEL, UnsupportedCase, score_case
from rl_kernel_b200.validation.fixtures.smoke_ops import apply_operator_override

DEFAULT_MODEL = REFERENCE_MODEL


def _score_case(exp: ExperimentConfig, case: CaseConfig) -> tuple[torch.Tensor, dict]:
    score, actual = score_case(exp, case)
    return apply_operator_override(case.knobs.get("operator_override"), score), actual


def compare(score: torch.Tensor, ref: torch.Tensor) -> dict:
    diff = (score.double() - ref.double()).abs()
    mism = score.view(torch.int32 if score.dtype == torch.float32 else torch.int16) != \
        ref.view(torch.int32 if ref.dtype == torch.float32 else torch.int16)
    first = mism.nonzero()
    return {"mismatch_count": int(mism.sum()), "elements": int(mism.numel()), "max_abs": float(diff.max()),
            "mean_abs": float(diff.mean()), "first_mismatch": first[0].tolist() if first.numel() else None}


def run_experiment(exp: ExperimentConfig, out_dir: str | Path, resume: bool = True) -> dict:
    store = AttemptStore(out_dir, exp.experiment_id)
    scores: dict[str, torch.Tensor] = {}
    reused: dict[str, bool] = {}
    order = sorted(exp.cases, key=lambda c: c.name != exp.reference_case)
    summary = {"experiment_id": exp.experiment_id, "reference_case": exp.reference_case, "cases": {}}
    for case in order:
        requested = {"case": case.name, "knobs": case.knobs, "seed": exp.seed, "num_sequences": exp.num_sequences,
                     "seq_len": exp.seq_len, "model": exp.model, "backend": exp.backend}
        prev = store.reusable(case.name, requested) if resume else None
        if prev is not None:
            scores[case.name] = torch.load(prev / "score.pt")
            reused[case.name] = True
        else:
            try:
                score, actual = _score_case(exp, case)
            except UnsupportedCase as exc:
                if case.name == exp.reference_case:
                    raise
                summary["cases"][case.name] = {"blocked": str(exc), "mismatch_count": None, "reused": False}
                continue
            scores[case.name] = score
            reused[case.name] = False
            comparison = None if case.name == exp.reference_case else compare(score, scores[exp.reference_case])
            store.write(store.new_attempt(case.name), requested, actual, score, comparison)
        cmp = {"mismatch_count": 0} if case.name == exp.reference_case else compare(scores[case.name], scores[exp.reference_case])
        summary["cases"][case.name] = {**cmp, "reused": reused[case.name]}
    ran = [c for c in summary["cases"].values() if "blocked" not in c]
    summary["blocked_cases"] = sorted(n for n, c in summary["cases"].items() if "blocked" in c)
    summary["all_bitwise_equal"] = bool(ran) and all(c["mismatch_count"] == 0 for c in ran)
    summary["run_seal"] = store.seal_run()
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("config")
    ap.add_argument("--out", default="runs")
    ap.add_argument("--no-resume", action="store_true")
    ap.add_argument("--backend", choices=("auto", "reference", "engine"), default=None,
                    help="override the experiment's scoring backend (engine = the sm_100a Qwen3Engine)")
    a = ap.parse_args(argv)
    exp = ExperimentConfig.load(a.config)
    if a.backend:
        exp = dataclasses.replace(exp, backend=a.backend)
    summary = run_experiment(exp, a.out, resume=not a.no_resume)
    print(json.dumps(summary, indent=1))
    return 0 if summary["all_bitwise_equal"] else 1


if __name__ == "__main__":
    sys.exit(main())


# ================================================================================================ paired alignment runs
def run_alignment(config, out_dir, *, rollout, training, materializers, bitwise: bool = False, resume: bool = True) -> dict:
    """Plan ``config`` (an ``AlignmentExperimentConfig``), materialise every case on both sides, score it with the two
    paired scorers under the read-only guard, compare the artifacts under the tolerance contract (``bitwise``: at
    threshold zero) and keep sealed, resumable attempts under ``out_dir/<experiment>/paired/<case>/<n>/`` (parity: the
    paired runner of rl_engine/validation/cross_config/runner.py:60-714)."""
    from rl_kernel_b200.validation.cross_config import _execution as ex, _provenance as pv, _resume as rs
    from rl_kernel_b200.validation.cross_config._json import strict_json_dumps
    from rl_kernel_b200.validation.cross_config.comparison import FixedThresholdComparator
    from rl_kernel_b200.validation.cross_config.execution_plan import build_execution_plan
    from rl_kernel_b200.validation.cross_config.runtime import RuntimeTools
    from rl_kernel_b200.validation.cross_config.schema import CanonicalScoringBatch, ScoreArtifact, ScoreSide

    plan = build_execution_plan(config)
    r_spec, t_spec = ex.validate_scorer_identity(rollout, training)
    tools = RuntimeTools()
    env = pv.execution_environment_provenance()
    fps = {"rollout": ex.scorer_implementation_fingerprint(rollout), "training": ex.scorer_implementation_fingerprint(training),
           **{f"materializer.{m.target}": m.implementation_fingerprint() for m in materializers}}
    root = Path(out_dir) / config.definition.experiment_id / "paired"
    batch = CanonicalScoringBatch.from_identity(config.definition.identity)
    comparator = FixedThresholdComparator(bitwise=bitwise)
    summary = {"experiment_id": config.definition.experiment_id, "bitwise": bitwise, "cases": {}, "issues": [i.to_dict() for i in plan.issues],
               "environment": env, "model_state": ex.paired_model_state_fingerprints(rollout, training)}
    for entry in plan.entries:
        case = entry.case
        m = tools.materialize(case, materializers, strict_fallback=config.definition.strict_fallback)
        row = {"changed_paths": list(case.changed_paths), "materialization": m.case.status.value, "isolation_scope": m.case.isolation_scope.value}
        summary["cases"][case.case_id] = row
        if not m.executable:
            row.update(status="not_executable", evidence=pv.json_safe(dict(m.case.evidence)))
            continue
        efp = pv.execution_fingerprint(m, scorer_fingerprints=fps, environment=env)
        case_dir = root / case.case_id
        attempts = sorted((p for p in case_dir.iterdir() if p.is_dir()), key=lambda p: int(p.name)) if case_dir.exists() else []
        stored = next((r for a in reversed(attempts) if (r := rs.completed_attempt_matches(a, execution_fingerprint=efp, case_id=case.case_id))), None) if resume else None
        if stored is not None:
            row.update(status=stored["status"], passed=stored["passed"], mismatch_count=stored["mismatch_count"],
                       active_token_count=stored["active_token_count"], reused=True)
            continue
        attempt = case_dir / str(len(attempts))
        attempt.mkdir(parents=True)
        attempt_id = f"{case.case_id}/{attempt.name}"
        arts = {}
        for side, scorer, spec in ((ScoreSide.ROLLOUT, rollout, r_spec), (ScoreSide.TRAINING, training, t_spec)):
            opts = dict(m.adapters[side.value].options) if side.value in m.adapters else {}
            with ex.read_only_scoring_guard(scorer):
                ranks = scorer.score(batch, options=opts)
            top = ex.validate_rank_outputs(ranks, batch, expected_world_size=spec.world_size)
            prov = pv.side_provenance(side, m, actual={k: v for k, v in top.actual.items()}, implementation_fingerprint=fps[side.value],
                                      world_size=spec.world_size)
            arts[side] = ScoreArtifact(case.case_id, attempt_id, side, case.identity, spec, top.selected_logprobs, batch.active_mask, prov)
            (attempt / f"{side.value}.json").write_text(strict_json_dumps({**pv.score_metadata(arts[side]), "provenance": prov.to_dict()}, indent=1))
        result = comparator.compare(arts[ScoreSide.ROLLOUT], arts[ScoreSide.TRAINING])
        tokens = result.token_artifact
        torch.save({"rollout_logprobs": arts[ScoreSide.ROLLOUT].selected_logprobs.masked_fill(~batch.active_mask, 0.0),
                    "training_logprobs": arts[ScoreSide.TRAINING].selected_logprobs.masked_fill(~batch.active_mask, 0.0),
                    "active_mask": batch.active_mask, **({"mismatch_mask": tokens.mismatch_mask} if tokens is not None else {})},
                   attempt / "tensors.pt")
        rd = {k: v for k, v in result.to_dict().items() if k != "token_artifact"}
        (attempt / "request.json").write_text(strict_json_dumps({"case_id": case.case_id, "execution_fingerprint": efp,
                                                                  "requested": pv.json_safe(dict(case.requested)),
                                                                  "operators": entry.operators.to_dict()}, indent=1))
        (attempt / "result.json").write_text(strict_json_dumps(rd, indent=1))
        rs.seal_attempt(attempt)
        row.update(status=result.status.value, passed=result.passed, mismatch_count=result.mismatch_count,
                   active_token_count=result.active_token_count, reused=False, diagnostics=pv.json_safe(dict(result.diagnostics)))
    ran = [c for c in summary["cases"].values() if "passed" in c]
    summary["all_passed"] = bool(ran) and all(c["passed"] for c in ran)
    summary["not_executable"] = sorted(k for k, c in summary["cases"].items() if c.get("status") == "not_executable")
    (Path(out_dir) / config.definition.experiment_id).mkdir(parents=True, exist_ok=True)
    (Path(out_dir) / config.definition.experiment_id / "paired_summary.json").write_text(strict_json_dumps(pv.json_safe(summary), indent=1))
    return summary


# ================================================================================================ one case, one attempt
@dataclasses.dataclass(frozen=True)
class PairedRunResult:
    """A completed attempt of one case, or a validated earlier attempt that was reused."""
    case_id: str
    attempt_id: str
    attempt_dir: Path
    resumed: bool
    rollout_score: object = None
    training_score: object = None
    alignment: object = None
    summary: dict = dataclasses.field(default_factory=dict)


class PairedRunner:
    """Score ONE materialised case on both sides and publish it as one append-only attempt of an ``ArtifactStore``
    (parity: PairedRunner, rl_engine/validation/cross_config/runner.py:88-440).  ``run`` refuses a case that is not
    executable, checks that the two scorers name opposite sides of the same model, scores under the read-only guard,
    checks every rank's output, compares under the fixed-threshold contract and seals the attempt; with ``resume`` an
    intact earlier attempt made for the same execution fingerprint is returned instead."""

    def __init__(self, artifact_store, *, timeout_seconds: float = 30.0, start_method=None):
        import math

        from rl_kernel_b200.validation.cross_config._execution import ChildSupervisor
        if not math.isfinite(timeout_seconds) or timeout_seconds <= 0.0:
            raise ValueError("timeout_seconds must be finite and greater than zero")
        self.artifact_store = artifact_store
        self.timeout_seconds = float(timeout_seconds)
        self._children = ChildSupervisor(start_method)
        self.start_method = self._children.start_method

    @property
    def active_child_pids(self) -> tuple[int, ...]:
        return self._children.active_child_pids()

    def run(self, experiment_id: str, case, materialization, batch, rollout_scorer, training_scorer, *, materializers=(),
            bitwise: bool = False, resume: bool = True) -> PairedRunResult:
        from rl_kernel_b200.validation.cross_config import _execution as ex, _provenance as pv
        from rl_kernel_b200.validation.cross_config.comparison import FixedThresholdComparator
        from rl_kernel_b200.validation.cross_config.schema import ScoreArtifact, ScoreSide

        if materialization.case.case.case_id != case.case_id:
            raise ex.PairedRunnerError(f"materialization is for case {materialization.case.case.case_id!r}, not {case.case_id!r}")
        if not materialization.executable:
            raise ex.PairedRunnerError(f"case {case.case_id!r} is not executable: {materialization.case.status.value}")
        r_spec, t_spec = ex.validate_scorer_identity(rollout_scorer, training_scorer)
        env = pv.execution_environment_provenance()
        fps = {"rollout": ex.scorer_implementation_fingerprint(rollout_scorer), "training": ex.scorer_implementation_fingerprint(training_scorer),
               **{f"materializer.{m.target}": m.implementation_fingerprint() for m in materializers}}
        efp = pv.execution_fingerprint(materialization, scorer_fingerprints=fps, environment=env)
        request = {"case_id": case.case_id, "execution_fingerprint": efp, "bitwise": bool(bitwise),
                   "requested": pv.json_safe(dict(case.requested))}
        store = self.artifact_store
        store.experiment_dir(experiment_id).mkdir(parents=True, exist_ok=True)
        if resume:
            prev = store.completed_attempt(experiment_id, case.case_id, request)
            if prev is not None:
                rec = store.validate_completed_attempt(prev)
                return PairedRunResult(case.case_id, f"{case.case_id}/{prev.name}", prev, True, summary=dict(rec["summary"]))
        attempt = store.create_attempt(experiment_id, case.case_id, request)
        attempt_id = f"{case.case_id}/{attempt.name}"
        arts = {}
        for side, scorer, spec in ((ScoreSide.ROLLOUT, rollout_scorer, r_spec), (ScoreSide.TRAINING, training_scorer, t_spec)):
            opts = dict(materialization.adapters[side.value].options) if side.value in materialization.adapters else {}
            with ex.read_only_scoring_guard(scorer):
                ranks = scorer.score(batch, options=opts)
            top = ex.validate_rank_outputs(ranks, batch, expected_world_size=spec.world_size)
            prov = pv.side_provenance(side, materialization, actual=dict(top.actual), implementation_fingerprint=fps[side.value],
                                      world_size=spec.world_size)
            arts[side] = ScoreArtifact(case.case_id, attempt_id, side, case.identity, spec, top.selected_logprobs, batch.active_mask, prov)
            store.write_json(attempt, side.value, pv.json_safe({**pv.score_metadata(arts[side]), "provenance": prov.to_dict()}))
        result = FixedThresholdComparator(bitwise=bitwise).compare(arts[ScoreSide.ROLLOUT], arts[ScoreSide.TRAINING])
        tokens = result.token_artifact
        store.write_tensor_bundle(attempt, "tensors", {
            "rollout_logprobs": arts[ScoreSide.ROLLOUT].selected_logprobs.masked_fill(~batch.active_mask, 0.0),
            "training_logprobs": arts[ScoreSide.TRAINING].selected_logprobs.masked_fill(~batch.active_mask, 0.0),
            "active_mask": batch.active_mask, **({"mismatch_mask": tokens.mismatch_mask} if tokens is not None else {})},
            metadata={"case_id": case.case_id, "attempt_id": attempt_id})
        store.write_json(attempt, "result", pv.json_safe({k: v for k, v in result.to_dict().items() if k != "token_artifact"}))
        summary = {"status": result.status.value, "passed": bool(result.passed), "mismatch_count": int(result.mismatch_count),
                   "active_token_count": int(result.active_token_count), "execution_fingerprint": efp}
        store.complete_attempt(attempt, summary)
        return PairedRunResult(case.case_id, attempt_id, attempt, False, arts[ScoreSide.ROLLOUT], arts[ScoreSide.TRAINING], result, summary)
