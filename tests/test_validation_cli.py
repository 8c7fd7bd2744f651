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


def test_dense_experiment_planning_validation_and_collection(tmp_path):
    from rl_engine.integrations.orchestrators.vime.experiments.dense import collect_results, run, run_arm, validate_run, weight_audit

    plan = run.run_phase(tmp_path, "module_ablation", dry_run=True)["arms"]
    assert plan["module_ablation/M011/seed1234"]["status"] == "unavailable" and plan["module_ablation/M111/seed1234"]["status"] == "planned"
    with pytest.raises(run_arm.ArmUnavailable):
        run_arm.resolve_arm(run_arm.load_matrix(), "short", "native")
    assert run_arm.resolve_arm(run_arm.load_matrix(), "short", "G11")["framework_use_rollout_logprobs"] is True

    def fake_arm(group, logp_case, mism, lib=None, steps=3):
        d = tmp_path / "short" / group / "seed1234"
        d.mkdir(parents=True)
        (d / "arm.json").write_text(json.dumps({"phase": "short", "group": group, "seed": 1234, "num_rollout": steps, "attention_case": "R/R",
                                                "ffn_case": "R/R", "logp_case": logp_case}))
        recs = [{"step": i, "tokens_compared": 512, "mismatch_count": mism if i == 1 else 0, "max_abs_dlogp": 0.0, "reward_mean": 0.5,
                 "grad_norm": 1.0, "step_seconds": 0.1 + i, **({"library_mismatch_count": lib} if lib is not None else {})} for i in range(steps)]
        (d / "rounds.jsonl").write_text("\n".join(json.dumps(r) for r in recs) + "\n")
        (d / "readback.json").write_text(json.dumps({"fallbacks": []}))
        (d / "summary.json").write_text("{}")
        (d / "DONE").write_text("ok")
        return d

    good, lib, bad = fake_arm("consistency", "R/R", 0), fake_arm("library_logp", "R/P", 0, lib=200), fake_arm("G11", "R/R", 7)
    assert validate_run.validate_run(good)["valid"] and validate_run.validate_run(lib)["library_mismatches"] == 600
    v = validate_run.validate_run(bad)
    assert not v["valid"] and "bit-equal" in v["issues"][0]
    (good / "DONE").unlink()
    assert not validate_run.validate_run(good)["valid"]
    (good / "DONE").write_text("ok")
    rows = collect_results.collect(tmp_path)
    assert [r["group"] for r in rows] == ["G11", "consistency", "library_logp"] and [r["valid"] for r in rows] == [False, True, True]
    paths = collect_results.write_tables(rows, tmp_path / "out")
    assert paths["markdown"].read_text().count("\n") == 5 and paths["csv"].read_text().startswith("phase,group,seed")
    a = weight_audit.audit_weights({"w": torch.ones(2), "v": torch.zeros(1)}, {"w": torch.ones(2) * 2})
    assert not a["in_sync"] and a["differing"] == ["w"] and a["missing_in_rollout"] == ["v"]


def test_rlk_verify_acceptance_checks_on_training_rounds(tmp_path):
    from rl_engine.entrypoints.repro import main as rlk

    def write(recs, steps=None):
        (tmp_path / "rounds.jsonl").write_text("\n".join(json.dumps(r) for r in recs) + "\n")
        (tmp_path / "summary.json").write_text(json.dumps({"steps": len(recs) if steps is None else steps}))

    rec = lambda i, **kw: {"step": i, "mismatch_count": 0, "tokens_compared": 100, "max_abs_dlogp": 0.0, "reward_mean": 0.5, "grad_norm": 1.0,  # noqa: E731
                           "loss": 0.1, "weight_version": i + 1, **kw}
    write([rec(0), rec(1), rec(2)])
    assert rlk(["verify", str(tmp_path)]) == 0
    for bad in ([rec(0), rec(1, mismatch_count=3)], [rec(0), rec(1, grad_norm=float("nan"))], [rec(0), rec(1, weight_version=5)], [rec(0), rec(2)]):
        write(bad)
        assert rlk(["verify", str(tmp_path)]) == 2
    write([rec(0), rec(1)], steps=200)
    assert rlk(["verify", str(tmp_path)]) == 2


def test_operator_check_cli_and_weight_preparation(tmp_path, capsys):
    from rl_engine.models.qwen3.prepare_weights import main as prepare
    from rl_engine.validation.operators.__main__ import main as check

    assert check(["list"]) == 0 and "rms_norm" in capsys.readouterr().out
    assert check(["operator", "swiglu"]) == 0
    assert check(["forward-invariance", "rope"]) == 0
    assert check(["gradient-invariance", "rms_norm"]) == 0
    assert check(["stateful-kv"]) == 0
    capsys.readouterr()
    assert check(["sweep", "--json", "--output", str(tmp_path / "evidence.json")]) == 0
    doc = json.loads((tmp_path / "evidence.json").read_text())
    assert doc["green"] and doc["inventory"] == {"unexecuted": [], "needs_fix": []} and doc["accelerator"]["arch_key"] == "cpu"
    if not torch.cuda.is_available():
        with pytest.raises(Exception):
            check(["operator", "swiglu", "--device", "cuda"])
    out = tmp_path / "w"
    assert prepare(["--output", str(out), "--synthetic", "--layers", "1", "--hidden", "256", "--ffn", "512", "--vocab", "1024"]) == 0
    first = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert prepare(["--output", str(out), "--verify-only"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["content_hash"] == first["content_hash"]
    shard = next(out.glob("*.safetensors"))
    (tmp_path / "sha.json").write_text(json.dumps({shard.name: "0" * 64}))
    with pytest.raises(ValueError, match="checksum"):
        prepare(["--output", str(out), "--verify-only", "--sha256-file", str(tmp_path / "sha.json")])


def test_operator_spec_paths_resolve():
    import importlib

    from rl_engine.validation.operators.operator_specs import OP_SPECS, _local

    for name, spec in OP_SPECS.items():
        for path in {**spec.candidate_paths, "gold": spec.gold_path}.values():
            mod, attr = _local(path).rsplit(".", 1)
            assert hasattr(importlib.import_module(mod), attr), (name, path)


def test_gradient_adapter_registry_and_status_matrix():
    import dataclasses

    from rl_kernel_b200.config.workload import load_manifest
    from rl_kernel_b200.validation.operators import gradient_adapters as ga

    assert set(ga.adapter_names()) == set(ga.OP_SPECS) and ga.get_adapter("rms_norm").chain_nodes == ("input_layernorm", "post_attention_layernorm",
                                                                                                  "final_layernorm")
    with pytest.raises(KeyError, match="unknown gradient adapter"):
        ga.get_adapter("nope")
    req = {a.op_name for a in ga.required_gradient_adapters()}
    assert {"rms_norm", "det_gemm", "attention", "linear_logp", "swiglu", "rope", "embedding"} <= req and "sampling" not in req
    assert "pack" in {a.op_name for a in ga.required_forward_adapters()}
    rows = ga.gradient_adapter_status_matrix()
    m = load_manifest()
    assert not [r for r in rows if r.untracked_red or r.tracked_red]                       # every node a profile runs can be judged
    for profile in m.backend_profiles:
        nodes = [r.chain_node for r in rows if r.backend_profile == profile and r.chain_node != "-"]
        assert nodes == list(m.chain_semantics["nodes"])
    b200 = {r.chain_node: r for r in rows if r.backend_profile == "b200_bf16"}
    assert b200["logprob"].op_name == "linear_logp" and b200["logprob"].expected_backend_id == "b200" and "weight" in b200["o_proj"].grad_tensor_names
    assert {r.candidate_status for r in rows if r.chain_node == "-"} <= {"optional", "declared", "absent_not_required"}
    assert b200["rope"].to_dict()["candidate_path"].endswith("RoPESM100Op")
    # a chain node nobody maps is an untracked red row
    saved = ga.CHAIN_NODE_OPERATORS.pop("rope")
    try:
        red = [r for r in ga.gradient_adapter_status_matrix(profiles=("b200_bf16",)) if r.untracked_red]
        assert [r.chain_node for r in red] == ["rope"] and not red[0].adapter_registered
    finally:
        ga.CHAIN_NODE_OPERATORS["rope"] = saved
    gold = ga.load_adapter_gold("swiglu")
    g, u = torch.randn(3, 8), torch.randn(3, 8)
    assert torch.allclose(gold(g, u), torch.nn.functional.silu(g) * u, atol=1e-6)
    assert type(ga.load_adapter_operator("rms_norm", "pytorch")).__name__ == "NativeRMSNormOp"
    with pytest.raises(RuntimeError, match="no candidate"):
        ga.load_adapter_operator("rms_norm", "triton")
    paths = ga.listed_source_paths(ga.get_adapter("attention"))
    assert paths and all(p.exists() for p in paths)
    assert dataclasses.is_dataclass(ga.get_adapter("pack")) and ga.get_adapter("pack").requirement == "layout_supported"


def test_manifest_chain_gate_cells_accuracy_and_first_drift():
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.reference import Qwen3DenseBIModel
    from rl_kernel_b200.validation.models.chain_gate import run_manifest_chain_gate

    spec = Qwen3DenseSpec.scaled(layers=1, hidden=64, ffn=128, q_heads=4, kv_heads=2, head_dim=16, vocab=6600)
    w = Qwen3DenseWeights.synthetic(spec, seed=1)
    gold = Qwen3DenseBIModel(spec, w)
    rep = run_manifest_chain_gate(Qwen3DenseBIModel(spec, w), gold_model=gold)
    assert rep.passed and {c.cell_id for c in rep.invariance} == {"BN/permuted", "BN/long_padding", "B1-singleton_aggregate/full", "B1/chunked",
                                                                    "B1/decode"}
    assert all(c.tokens == 27 and c.mismatching_tokens == 0 for c in rep.invariance) and rep.accuracy["passed"] and rep.first_drift is None
    d = rep.to_dict()
    assert d["cells"]["BN/full"]["n_logp_tokens"] == 27 and "embedding" in d["cells"]["BN/full"]["node_digests"] and d["fixture_hash"]
    # a bf16 candidate is judged against the fp32 gold with the bf16 thresholds
    bf = run_manifest_chain_gate(Qwen3DenseBIModel(spec, w, execution_dtype=torch.bfloat16), gold_model=gold, cells=("singletons",),
                                 execution_dtype=torch.bfloat16)
    assert bf.passed and bf.accuracy["aggregates"]["max_abs_dlogp"] > 0
    # a model whose arithmetic depends on which rows share a call is caught by the cells, with the worst token named

    class Leaky(Qwen3DenseBIModel):
        def selected_logprobs(self, rows, targets):
            lp = super().selected_logprobs(rows, targets)
            return lp + (1e-3 if rows.shape[0] > 30 else 0.0)

    bad = run_manifest_chain_gate(Leaky(spec, w), cells=("singletons", "permuted"))
    by = {c.cell_id: c for c in bad.invariance}
    assert not bad.passed and by["B1-singleton_aggregate/full"].mismatching_tokens == 27 and by["BN/permuted"].passed
    assert by["B1-singleton_aggregate/full"].worst_key is not None
    # a candidate with one perturbed layer fails the accuracy judgment and the first drifting node is reported
    w2 = Qwen3DenseWeights.synthetic(spec, seed=1)
    key = next(k for k in w2.tensors if "mlp" in k and "down" in k) if hasattr(w2, "tensors") else None
    if key is not None:
        w2.tensors[key] = w2.tensors[key] * 4.0
        off = run_manifest_chain_gate(Qwen3DenseBIModel(spec, w2), gold_model=gold, cells=())
        assert not off.passed and off.first_drift == "layers.0.residual_mlp"
    with pytest.raises(ValueError, match="unknown cell"):
        run_manifest_chain_gate(Qwen3DenseBIModel(spec, w), cells=("nope",))


def test_classified_four_judgment_grid():
    from rl_kernel_b200.validation.operators import four_judgment_matrix as fj

    rep = fj.build_classified_matrix()
    assert len(rep.cells) == 2 * len(fj.REQUIRED_OPS) * len(fj.TIERS) * len(fj.JUDGMENTS)
    assert set(rep.counts) <= {"pending_execution", "N/A"} and not fj.undefined_cells(rep) and not fj.hidden_required_na(rep), rep.counts
    assert all(c.status == "N/A" and "layout_supported" in c.detail for c in rep.cells if c.op_name == "pack")
    cell = next(c for c in rep.cells if c.profile == "b200_bf16" and c.op_name == "det_gemm" and c.tier == "short" and c.judgment == "forward_accuracy")
    assert cell.case_id.startswith("gemm-short") and cell.candidate == "b200" and cell.evidence_kind == "representative_accuracy"
    assert not rep.green                                                       # nothing has been executed yet
    # executed judgments turn pending cells green (or red)
    ran = fj.executed_results("reference_fp32", ("rms_norm", "swiglu"), candidate="pytorch")
    ran[("reference_fp32", "swiglu")] = {**ran[("reference_fp32", "swiglu")], "gradient_invariance": ("fail", "B1/singletons:dx")}
    rep2 = fj.build_classified_matrix(profiles=("reference_fp32",), executed=ran)
    by = {(c.op_name, c.tier, c.judgment): c for c in rep2.cells}
    assert by[("rms_norm", "primary", "forward_invariance")].status == "green"
    assert by[("swiglu", "short", "gradient_invariance")].status == "red" and "B1/singletons" in by[("swiglu", "short", "gradient_invariance")].detail
    assert by[("rope", "primary", "forward_accuracy")].status == "pending_execution"
    with pytest.raises(ValueError, match="unknown backend profiles"):
        fj.build_classified_matrix(profiles=("cuda_fp8",))
    # an operator the profile runs but nothing can judge is red, never N/A
    from rl_kernel_b200.validation.operators import gradient_adapters as ga

    saved = ga.OP_SPECS["rope"].candidate_paths.pop("b200")
    try:
        red = [c for c in fj.build_classified_matrix(profiles=("b200_bf16",)).cells if c.op_name == "rope"]
        assert red and all(c.status == "red" and "missing_candidate" in c.detail for c in red)
    finally:
        ga.OP_SPECS["rope"].candidate_paths["b200"] = saved


def test_operators_cli_grid_and_adapters(capsys):
    import json

    from rl_kernel_b200.validation.operators.__main__ import main as check

    assert check(["adapters", "--json"]) == 0
    rows = json.loads(capsys.readouterr().out)
    assert {r["backend_profile"] for r in rows} == {"b200_bf16", "reference_fp32"} and not any(r["untracked_red"] for r in rows)
    assert check(["grid", "--profile", "b200_bf16", "--json"]) == 0
    grid = json.loads(capsys.readouterr().out)
    assert grid["counts"] == {"pending_execution": 72, "N/A": 8}
    assert check(["grid", "--profile", "reference_fp32"]) == 0 and "pending_execution" in capsys.readouterr().out
