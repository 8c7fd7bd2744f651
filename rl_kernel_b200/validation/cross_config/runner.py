"""Cross-configuration log-prob drift runner: score the same sequences under several
configurations (batching, padding, decode vs prefill, simulated TP degree, operator overrides) and
compare every case with the reference case token by token, bit by bit (parity:
``python -m rl_engine.validation.cross_config``)."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
from rl_kernel_b200.models.qwen3.reference import Qwen3DenseBIModel
from rl_kernel_b200.validation.cross_config.artifacts import AttemptStore
from rl_kernel_b200.validation.cross_config.config import CaseConfig, ExperimentConfig
from rl_kernel_b200.validation.fixtures.smoke_ops import apply_operator_override

DEFAULT_MODEL = {"layers": 2, "hidden": 256, "ffn": 768, "q_heads": 4, "kv_heads": 2, "head_dim": 64, "vocab": 4096}


def _score_case(exp: ExperimentConfig, case: CaseConfig) -> tuple[torch.Tensor, dict]:
    spec = Qwen3DenseSpec.scaled(**{**DEFAULT_MODEL, **exp.model})
    dtype = torch.float32 if case.knobs.get("dtype", "float32") == "float32" else torch.bfloat16
    weights = Qwen3DenseWeights.synthetic(spec, dtype=dtype, seed=exp.seed)
    model = Qwen3DenseBIModel(spec, weights, execution_dtype=dtype, tp_size=case.knobs.get("tp_size", 1))
    g = torch.Generator().manual_seed(exp.seed + 1)
    ids = torch.randint(0, spec.vocab_size, (exp.num_sequences, exp.seq_len), generator=g)
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
    score = torch.cat(rows)
    score = apply_operator_override(case.knobs.get("operator_override"), score)
    return score, {"dtype": str(dtype), "tp_size": model.tp_size, "batch_size": bs, "decode_from": decode_from}


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
                     "seq_len": exp.seq_len, "model": exp.model}
        prev = store.reusable(case.name, requested) if resume else None
        if prev is not None:
            scores[case.name] = torch.load(prev / "score.pt")
            reused[case.name] = True
        else:
            score, actual = _score_case(exp, case)
            scores[case.name] = score
            reused[case.name] = False
            comparison = None if case.name == exp.reference_case else compare(score, scores[exp.reference_case])
            store.write(store.new_attempt(case.name), requested, actual, score, comparison)
        cmp = {"mismatch_count": 0} if case.name == exp.reference_case else compare(scores[case.name], scores[exp.reference_case])
        summary["cases"][case.name] = {**cmp, "reused": reused[case.name]}
    summary["all_bitwise_equal"] = all(c["mismatch_count"] == 0 for c in summary["cases"].values())
    summary["run_seal"] = store.seal_run()
    return summary


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("config")
    ap.add_argument("--out", default="runs")
    ap.add_argument("--no-resume", action="store_true")
    a = ap.parse_args(argv)
    summary = run_experiment(ExperimentConfig.load(a.config), a.out, resume=not a.no_resume)
    print(json.dumps(summary, indent=1))
    return 0 if summary["all_bitwise_equal"] else 1


if __name__ == "__main__":
    sys.exit(main())
