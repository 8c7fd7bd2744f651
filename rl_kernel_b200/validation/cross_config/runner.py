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
