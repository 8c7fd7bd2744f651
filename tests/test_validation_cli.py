"""Validation harness and CLI on CPU."""
import json

import pytest
import torch

from rl_engine.validation.cross_config.artifacts import AttemptStore
from rl_engine.validation.cross_config.config import ExperimentConfig
from rl_engine.validation.cross_config.runner import run_experiment
from rl_engine.validation.operators.four_judgment_matrix import four_judgment_matrix
from rl_engine.validation.reports.drift_report import write_drift_report


def test_four_judgment_matrix_is_green_on_cpu():
    m = four_judgment_matrix(device="cpu", dtype=torch.float32)
    assert m.green, m.render() + "\n" + str(m.red_cells())


def test_forward_invariance_reports_an_injected_row_dependence():
    from rl_engine.validation.operators import operator_specs as specs
    from rl_engine.validation.operators.forward_invariance import run_forward_invariance

    good = specs.FACTORIES["swiglu"]

    class Leaky:
        def __call__(self, g, u):
            y = good()(g, u).clone()
            y[1::2] += 1.0e-2
            return y

    specs.FACTORIES["swiglu"] = Leaky
    try:
        rep = run_forward_invariance("swiglu", device="cpu", dtype=torch.float32)
    finally:
        specs.FACTORIES["swiglu"] = good
    assert not rep.forward_invariant and "B1/singletons" in rep.failing()
    assert run_forward_invariance("swiglu", device="cpu", dtype=torch.float32).forward_invariant


def _exp(extra_case=None):
    cases = [{"name": "ref", "knobs": {}}, {"name": "b1", "knobs": {"batch_size": 1}},
             {"name": "tp2", "knobs": {"tp_size": 2}}, {"name": "decode", "knobs": {"decode_from": 8}}]
    if extra_case:
        cases.append(extra_case)
    return ExperimentConfig.from_dict({"experiment_id": "t", "reference_case": "ref", "cases": cases,
                                       "num_sequences": 2, "seq_len": 16})


def test_cross_config_runner_detects_equality_and_injected_offset(tmp_path):
    s = run_experiment(_exp(), tmp_path)
    assert s["all_bitwise_equal"], s
    s2 = run_experiment(_exp(), tmp_path)
    assert all(c["reused"] for c in s2["cases"].values()), "sealed attempts must be reused on resume"
    bad = run_experiment(_exp({"name": "offset", "knobs": {"operator_override": "smoke_only.logp_offset"}}), tmp_path)
    assert not bad["all_bitwise_equal"] and bad["cases"]["offset"]["mismatch_count"] > 0
    paths = write_drift_report(bad, tmp_path / "report")
    assert json.loads(paths["trace"].read_text())["traceEvents"]


def test_tampered_attempt_is_not_reused(tmp_path):
    run_experiment(_exp(), tmp_path)
    store = AttemptStore(tmp_path, "t")
    a = store.attempts("b1")[-1]
    (a / "actual.json").write_text("{}")                 # break the seal
    assert not store.verify(a)
    s = run_experiment(_exp(), tmp_path)
    assert not s["cases"]["b1"]["reused"] and len(store.attempts("b1")) == 2


def test_strict_config_loading():
    with pytest.raises(ValueError):
        ExperimentConfig.from_dict({"experiment_id": "x", "reference_case": "a", "cases": [{"name": "a"}], "bogus": 1})
    with pytest.raises(ValueError):
        ExperimentConfig.from_dict({"experiment_id": "x", "reference_case": "a",
                                    "cases": [{"name": "a", "knobs": {"warp_speed": 9}}]})
    with pytest.raises(ValueError):
        ExperimentConfig.from_dict({"experiment_id": "x", "reference_case": "zzz", "cases": [{"name": "a"}]})


def test_cli_plan_doctor_validate(capsys, tmp_path):
    from rl_engine.entrypoints.repro import main

    assert main(["plan", "--case", "R/R"]) == 0
    assert json.loads(capsys.readouterr().out)["bitwise_guarantee"] is True
    assert main(["doctor"]) == 0
    capsys.readouterr()
    cfg = tmp_path / "exp.json"
    cfg.write_text(json.dumps({"experiment_id": "cli", "reference_case": "ref", "num_sequences": 2, "seq_len": 12,
                               "cases": [{"name": "ref"}, {"name": "b1", "knobs": {"batch_size": 1}}]}))
    assert main(["validate", "--device", "cpu", "--config", str(cfg), "--out", str(tmp_path / "runs"), "--seal"]) == 0
    with pytest.raises(SystemExit):
        main(["run", "--gpus", "2", "--tp", "1", "--cp", "1"])


def test_chain_gate_on_reference_model():
    from rl_engine.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_engine.models.qwen3.reference import Qwen3DenseBIModel
    from rl_engine.validation.models.chain_gate import run_chain_gate

    spec = Qwen3DenseSpec.scaled(layers=2, hidden=128, ffn=256, q_heads=4, kv_heads=2, head_dim=32, vocab=512)
    w = Qwen3DenseWeights.synthetic(spec, dtype=torch.float32, seed=1)
    ids = torch.randint(0, 512, (3, 12), generator=torch.Generator().manual_seed(0))
    res = run_chain_gate(Qwen3DenseBIModel(spec, w, tp_size=2), Qwen3DenseBIModel(spec, w), ids, decode_from=6)
    assert res.passed, (res.cells, res.aggregates, res.first_drift)


def test_pyproject_entry_points_resolve():
    import importlib
    import tomllib
    from pathlib import Path

    data = tomllib.loads((Path(__file__).resolve().parents[1] / "pyproject.toml").read_text())
    targets = {**data["project"]["scripts"], **data["project"]["entry-points"]["vllm.general_plugins"]}
    assert set(data["project"]["scripts"]) == {"rlk", "rlk-repro", "rlk-drift-view"}
    for name, target in targets.items():
        mod, fn = target.split(":")
        assert callable(getattr(importlib.import_module(mod), fn)), name


def test_rlk_verify_checks_sealed_attempts_and_case_ids(tmp_path, capsys):
    from rl_engine.entrypoints.repro import _parse_plan, launch_command, main as rlk

    run_experiment(_exp(), tmp_path)
    assert rlk(["verify", str(tmp_path)]) == 0
    assert rlk(["verify", str(tmp_path), "--case-id", "tp2"]) == 0
    victim = next((tmp_path / "t" / "cases" / "b1").iterdir()) / "score.pt"
    victim.write_bytes(victim.read_bytes() + b"x")
    assert rlk(["verify", str(tmp_path)]) == 2
    with pytest.raises(SystemExit):
        rlk(["verify", str(tmp_path), "--case-id", "nope"])
    assert _parse_plan("tp4xcp2") == {"tp": 4, "cp": 2, "dp": 1} and _parse_plan("tp2xdp4")["dp"] == 4
    with pytest.raises(SystemExit):
        _parse_plan("pp2")
    cmd = launch_command(["run", "--gpus", "8", "--plan", "tp4xcp2"], 8, port=29511)
    assert cmd[1:4] == ["-m", "torch.distributed.run", "--nnodes=1"] and "--nproc-per-node=8" in cmd and cmd[-4:] == ["--gpus", "8", "--plan", "tp4xcp2"]
    assert "127.0.0.1" in cmd
