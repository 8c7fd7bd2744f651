"""Alignment experiments: schema, planner, materialisation, paired scoring on the CPU reference model, comparison,
determinism probes, strict JSON, sealed resume."""
import json

import pytest
import torch

from rl_engine.validation.cross_config import _execution as ex
from rl_engine.validation.cross_config._json import strict_json_loads
from rl_engine.validation.cross_config._resume import completed_attempt_matches, verify_seal
from rl_engine.validation.cross_config.adapters import KnobMaterializer, ReferenceModelScorer, reference_materializers
from rl_engine.validation.cross_config.comparison import compare_score_artifacts, recompute_mismatch_mask
from rl_engine.validation.cross_config.config import config_from_dict
from rl_engine.validation.cross_config.determinism import (compare_determinism, engine_probe, megatron_probe_from_config,
                                                           vllm_probe_from_env)
from rl_engine.validation.cross_config.execution_plan import build_execution_plan
from rl_engine.validation.cross_config.planner import MAX_PLAN_CASES, Planner, PlanningError
from rl_engine.validation.cross_config.runner import run_alignment
from rl_engine.validation.cross_config.runtime import RuntimeTools
from rl_engine.validation.cross_config.schema import (AlignmentStatus, CanonicalScoringBatch, IsolationScope, MaterializationStatus,
                                                      RuntimeProvenance, ScoreArtifact, ScorerSpec, ScoreSide, SemanticIdentitySpec)


def _identity(B=3, S=12, vocab=4096, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, vocab, (B, S), generator=g)
    sel = torch.roll(ids, -1, 1)
    act = torch.ones(B, S, dtype=torch.bool)
    act[:, -1] = False
    act[:, :3] = False
    return SemanticIdentitySpec.from_tensors(checkpoint_id="synthetic-seed0", model_version="qwen3-scaled", token_ids=ids,
                                             selected_token_ids=sel, active_mask=act)


def _raw(**over):
    i = _identity()
    raw = {"schema_version": "cross_config.experiment_config.v1", "experiment_id": "exp", "scenario_id": "s0",
           "identity": {k: v for k, v in i.to_dict().items() if k != "schema_version"},
           "baseline": {"batch": {"size": 3}, "rollout": {"tensor_parallel_size": 1, "dtype": "fp32"},
                        "training": {"compute_dtype": "fp32"}, "logp": {"backend": "reference"}},
           "interventions": [{"path": "batch.size", "values": [3, 1]}, {"path": "rollout.tensor_parallel_size", "values": [1, 2]}]}
    raw.update(over)
    return raw


def test_identity_and_batch_validation():
    i = _identity()
    assert i.active_token_count == 3 * 8
    b = CanonicalScoringBatch.from_identity(i)
    assert b.input_ids.shape == (3, 12)
    with pytest.raises(ValueError):
        SemanticIdentitySpec("c", "m", "p", ((1, 2), (3,)), ((1, 2), (3,)), ((True, True), (True,)), "pre")
    with pytest.raises(ValueError):
        CanonicalScoringBatch(i, b.input_ids + 1, b.selected_token_ids, b.active_mask, b.attention_mask)
    json.loads(i.to_json())


def test_planner_cases_issues_and_bounds():
    cfg = config_from_dict(_raw())
    plan = cfg.plan()
    assert [c.changed_paths for c in plan.cases] == [(), ("batch.size",), ("rollout.tensor_parallel_size",)]
    assert plan.cases[0].requested["rollout"]["dtype"] == "float32" and plan.cases[0].requested["logp"]["backend"] == "rlkernel.reference_logp"
    assert len({c.case_id for c in plan.cases}) == 3
    assert Planner().isolation_scope(("batch.size",)) is IsolationScope.REQUEST
    assert Planner().isolation_scope(("batch.size", "rollout.tensor_parallel_size")) is IsolationScope.PROCESS
    pair = config_from_dict(_raw(strategy="pairwise", pairwise_paths=[["batch.size", "rollout.tensor_parallel_size"]]))
    assert len(pair.plan().cases) == 4
    for bad, code in ((_raw(baseline={"batch": {"size": 0}}), "UNSUPPORTED_VALUE"), (_raw(baseline={"nope": 1}), "UNSUPPORTED_PATH"),
                      (_raw(interventions=[{"path": "logp.backend", "values": ["pytorch"]}]), "DERIVED_KNOB"),
                      (_raw(pairwise_paths=[["batch.size", "rollout.dtype"]]), "PAIRS_WITHOUT_STRATEGY")):
        with pytest.raises(PlanningError) as e:
            config_from_dict(bad).plan()
        assert code in {i.code for i in e.value.issues}
    big = _raw(interventions=[{"path": "batch.size", "values": list(range(1, MAX_PLAN_CASES + 3))}])
    with pytest.raises(PlanningError, match="PLAN_TOO_LARGE"):
        config_from_dict(big).plan()
    for bad in (_raw(extra=1), _raw(schema_version="v0"), _raw(scenario={"atol": 1.0})):
        with pytest.raises(ValueError):
            config_from_dict(bad)
    ep = build_execution_plan(cfg)
    assert all(e.case.case_id.startswith("cross-config-") and e.case.execution_binding["base_case_id"] for e in ep.entries)
    assert len(ep.rows()) == 3


def test_materialisation_reports_unsupported_knobs_and_reuse_scope():
    cfg = config_from_dict(_raw(interventions=[{"path": "batch.size", "values": [1]}, {"path": "training.sharding", "values": ["fsdp"]},
                                               {"path": "rollout.dtype", "values": ["bf16"]}],
                                baseline={"batch": {"size": 3}, "rollout": {"dtype": "fp32"}, "training": {"sharding": "unsharded"}}))
    cases = cfg.plan().cases
    tools, mats = RuntimeTools(), reference_materializers()
    ms = [tools.materialize(c, mats) for c in cases]
    assert [m.case.status for m in ms] == [MaterializationStatus.APPLIED, MaterializationStatus.APPLIED, MaterializationStatus.UNSUPPORTED,
                                           MaterializationStatus.APPLIED]
    assert not ms[2].executable and "training.training.sharding" in ms[2].case.evidence
    assert tools.can_reuse(ms[0], ms[1]) == "engine" and tools.can_reuse(ms[0], ms[3]) == "context" and tools.can_reuse(ms[0], ms[2]) == "nothing"
    assert ms[1].adapters["rollout"].options["batch_size"] == 1
    lazy = KnobMaterializer("rollout", {})
    lazy.materialize = lambda case, normalized: type(ms[0].adapters["rollout"])("rollout", ())     # reports nothing
    with pytest.raises(Exception, match="unreported"):
        tools.materialize(cases[0], (lazy,))


def test_paired_run_on_reference_model_is_bitwise_and_resumes(tmp_path):
    cfg = config_from_dict(_raw())
    ro, tr = ReferenceModelScorer("rollout", prefill_tokens=5), ReferenceModelScorer("training")
    s = run_alignment(cfg, tmp_path, rollout=ro, training=tr, materializers=reference_materializers(), bitwise=True)
    assert s["all_passed"] and len(s["cases"]) == 3 and not s["not_executable"], s
    assert all(c["mismatch_count"] == 0 and c["active_token_count"] == 24 and not c["reused"] for c in s["cases"].values())
    again = run_alignment(cfg, tmp_path, rollout=ro, training=tr, materializers=reference_materializers(), bitwise=True)
    assert all(c["reused"] for c in again["cases"].values()) and again["all_passed"]
    cid = next(iter(s["cases"]))
    attempt = tmp_path / "exp" / "paired" / cid / "0"
    assert verify_seal(attempt)
    (attempt / "result.json").write_text((attempt / "result.json").read_text().replace('"mismatch_count": 0', '"mismatch_count": 1'))
    assert not verify_seal(attempt) and completed_attempt_matches(attempt, execution_fingerprint="x", case_id=cid) is None
    third = run_alignment(cfg, tmp_path, rollout=ro, training=tr, materializers=reference_materializers(), bitwise=True)
    assert not third["cases"][cid]["reused"] and (tmp_path / "exp" / "paired" / cid / "1").exists()


def test_scoring_guard_and_rank_validation():
    sc = ReferenceModelScorer("training")
    with pytest.raises(ex.OperatorExecutionError, match="mutated"):
        with ex.read_only_scoring_guard(sc):
            next(iter(sc.state_tensors().values())).view(-1)[0] += 1
    b = CanonicalScoringBatch.from_identity(_identity())
    good = torch.zeros(3, 12)
    assert ex.validate_rank_outputs([ex.RankScore(0, 2, good), ex.RankScore(1, 2, good)], b).rank == 0
    with pytest.raises(ex.RankCompletenessError):
        ex.validate_rank_outputs([ex.RankScore(0, 2, good)], b)
    with pytest.raises(ex.RankCompletenessError, match="bits"):
        ex.validate_rank_outputs([ex.RankScore(0, 2, good), ex.RankScore(1, 2, good + 1e-6)], b)
    with pytest.raises(ex.OperatorExecutionError):
        ex.validate_rank_outputs([ex.RankScore(0, 1, good * float("nan"))], b)
    with pytest.raises(ex.ScorerIdentityError):
        ex.validate_scorer_identity(sc, sc)
    with pytest.raises(ex.ScorerIdentityError):
        ex.scorer_spec(sc, ScoreSide.ROLLOUT)


def _artifact(side, lp, identity=None, dtype="bfloat16", case="c", attempt="c/0"):
    i = identity or _identity()
    spec = ScorerSpec(side, "x", dtype)
    return ScoreArtifact(case, attempt, side, i, spec, lp, torch.tensor(i.active_mask), RuntimeProvenance({}, {}, {}, {}))


def test_comparator_statuses():
    base = -torch.rand(3, 12)
    r = _artifact(ScoreSide.ROLLOUT, base)
    assert compare_score_artifacts(r, _artifact(ScoreSide.TRAINING, base + 0.01)).status is AlignmentStatus.PASS
    res = compare_score_artifacts(r, _artifact(ScoreSide.TRAINING, base + 0.01), bitwise=True)
    assert res.status is AlignmentStatus.FAIL and res.mismatch_count == 24 and res.diagnostics["bitwise_mismatch_count"] == 24
    far = base.clone()
    far[1, 5] -= 0.2
    res = compare_score_artifacts(r, _artifact(ScoreSide.TRAINING, far))
    assert res.status is AlignmentStatus.FAIL and res.mismatch_count == 1 and tuple(res.diagnostics["worst_token"]) == (1, 5)
    assert compare_score_artifacts(r, _artifact(ScoreSide.TRAINING, base, dtype="float32")).fixed_threshold == 0.06
    nanpad = base.clone()
    nanpad[:, -1] = float("nan")                       # inactive positions may hold anything
    assert compare_score_artifacts(r, _artifact(ScoreSide.TRAINING, nanpad)).passed
    nanact = base.clone()
    nanact[0, 5] = float("nan")
    assert compare_score_artifacts(r, _artifact(ScoreSide.TRAINING, nanact)).status is AlignmentStatus.INVALID_ARTIFACT
    other = compare_score_artifacts(r, _artifact(ScoreSide.TRAINING, base, identity=_identity(seed=1)))
    assert other.status is AlignmentStatus.INVALID_IDENTITY and any("token_ids" in e for e in other.identity_errors)
    assert compare_score_artifacts(r, _artifact(ScoreSide.TRAINING, base, case="d")).status is AlignmentStatus.INVALID_ARTIFACT
    z = recompute_mismatch_mask(torch.tensor([0.0]), torch.tensor([-0.0]), torch.tensor([True]), 0.0)
    assert bool(z[0])                                  # threshold zero means equal bits


def test_determinism_probes():
    class Cfg:
        deterministic_mode = True
        tensor_model_parallel_size = 2

    env = {"NCCL_ALGO": "Ring", "VLLM_BATCH_INVARIANT": "1"}
    rep = compare_determinism(rollout=vllm_probe_from_env(env), training=megatron_probe_from_config(Cfg(), env))
    assert rep.compatible and "tf32_disabled" in rep.differences
    rep = compare_determinism(rollout=vllm_probe_from_env({**env, "NCCL_ALGO": "Tree"}), training=megatron_probe_from_config(Cfg(), env))
    assert not rep.compatible and rep.issues[0].field == "env.NCCL_ALGO"
    rep = compare_determinism(rollout=vllm_probe_from_env({}), training=megatron_probe_from_config(Cfg(), {}))
    assert not rep.compatible and rep.issues[0].field == "rollout.VLLM_BATCH_INVARIANT"
    own = compare_determinism(rollout=engine_probe("rollout", env={"NCCL_ALGO": "Tree"}), training=engine_probe("training", env={"NCCL_ALGO": "Ring"}))
    assert own.compatible and "NCCL_ALGO" in own.differences       # own collectives: NCCL's algorithm is recorded, not blocking
    json.dumps(own.to_dict())
    with pytest.raises(ValueError):
        compare_determinism(rollout=engine_probe("training"), training=engine_probe("training"))


def test_strict_json():
    assert strict_json_loads('{"a": 1.5}') == {"a": 1.5}
    for bad in ('{"a": 1, "a": 2}', '{"a": NaN}', '{"a": 1e999}', '{"a": Infinity}'):
        with pytest.raises(ValueError):
            strict_json_loads(bad)


def test_cpu_fixture_detects_a_smoke_offset_operator_and_viewer_renders(tmp_path, capsys):
    from rl_engine.validation.fixtures.cpu_cross_config import run_cpu_case, run_cpu_experiment
    from rl_engine.validation.reports.viewer import load_bundle, main as view, worst_tokens

    base = _raw(baseline={"batch": {"size": 3}, "rollout": {"dtype": "fp32"}, "training": {"compute_dtype": "fp32"},
                          "logp": {"backend": "reference"}}, interventions=[{"path": "batch.size", "values": [1]}])
    good = run_cpu_experiment(config_from_dict(base), tmp_path)
    assert good["all_passed"] and len(good["cases"]) == 2
    one = run_cpu_case(config_from_dict(base), 1)
    assert torch.equal(one["rollout"], one["training"])
    bad_raw = dict(base, experiment_id="exp-bad", operators={"selected_logprob": {"rollout": {"backend": "reference"},
                                                                                  "training": {"backend": "smoke_only.logp_offset"}}})
    bad = run_cpu_experiment(config_from_dict(bad_raw), tmp_path, bitwise=False)
    assert not bad["all_passed"] and all(c["mismatch_count"] == c["active_token_count"] for c in bad["cases"].values())
    bundle = load_bundle(tmp_path / "exp-bad")
    cid = next(iter(bundle["cases"]))
    assert abs(worst_tokens(bundle, cid, 3)[0]["abs_diff"] - 0.25) < 1e-5
    assert view([str(tmp_path / "exp-bad"), "--case", cid, "--html", str(tmp_path / "v.html")]) == 1
    assert "RED" in capsys.readouterr().out and (tmp_path / "v.html").read_text().startswith("<!doctype html>")
    assert view([str(tmp_path / "exp")]) == 0 and view([str(tmp_path / "nothing-here")]) == 2


def test_framework_materialisers_translate_attention_knobs():
    from rl_engine.integrations.common.knobs import WS2_ATTENTION_KNOBS, WS2_ATTENTION_NORMALIZERS
    from rl_engine.integrations.common.state import clear_active_integration, get_active_integration, set_active_integration
    from rl_engine.integrations.engines.rollout.vllm.adapter import VllmIntegration
    from rl_engine.integrations.engines.rollout.vllm.cross_config import VllmProvenanceAdapter, VllmRolloutMaterializer
    from rl_engine.integrations.engines.train.megatron.cross_config import MegatronAttentionMaterializer, MegatronProvenanceAdapter
    from rl_engine.validation.cross_config.schema import ExperimentDefinition, InterventionSpec

    d = ExperimentDefinition("e", "s", _identity(), {"batch": {"size": 2}, "rollout": {"tensor_parallel_size": 2, "kv_block_size": 128, "batch_invariant": True},
                                                     "training": {"tensor_parallel_size": 2, "context_parallel_size": 1, "deterministic_mode": True,
                                                                  "cp_comm_type": "peer_memory"}, "attention": {"reduction_order": "global_block_index"}},
                             (InterventionSpec("training.context_parallel_size", (2,)), InterventionSpec("attention.reduction_order", ("arrival",)),
                              InterventionSpec("rollout.kv_block_size", (16,)), InterventionSpec("training.cp_comm_type", ("p2p",))))
    plan = Planner(knobs=WS2_ATTENTION_KNOBS, normalizers=WS2_ATTENTION_NORMALIZERS).plan(d)
    tools = RuntimeTools(WS2_ATTENTION_KNOBS)
    got = {c.changed_paths: tools.materialize(c, (VllmRolloutMaterializer(), MegatronAttentionMaterializer())) for c in plan.cases}
    assert got[()].case.status is MaterializationStatus.APPLIED and "attention_contract_fingerprint" in got[()].adapters["training"].options
    assert got[("training.context_parallel_size",)].case.status is MaterializationStatus.APPLIED
    for path in ("attention.reduction_order", "rollout.kv_block_size", "training.cp_comm_type"):
        assert got[(path,)].case.status is MaterializationStatus.UNSUPPORTED, path
    assert tools.can_reuse(got[()], got[("training.context_parallel_size",)]) == "nothing"
    pa = VllmProvenanceAdapter(cache_config={"block_size": 128, "cache_dtype": "fp8"}, env={"VLLM_BATCH_INVARIANT": "1"})
    assert pa.frozen_scope_violations() == ("cache_dtype='fp8' (expected 'auto')",) and pa.kv_page_size == 128 and pa.determinism_probe().enabled
    ma = MegatronProvenanceAdapter({"deterministic_mode": True, "pipeline_model_parallel_size": 2})
    assert ma.frozen_scope_violations() and ma.determinism_probe().enabled
    integ = VllmIntegration()
    set_active_integration("vllm", integ)
    try:
        assert get_active_integration("vllm") is integ
        with pytest.raises(RuntimeError):
            set_active_integration("vllm", VllmIntegration())
        with pytest.raises(ValueError):
            set_active_integration("megatron", integ)
    finally:
        clear_active_integration("vllm")


def test_drift_report_bundle_from_sealed_attempts(tmp_path):
    from rl_engine.validation.fixtures.cpu_cross_config import run_cpu_experiment
    from rl_engine.validation.reports.drift_report import (build_cross_config_attempt_report, build_drift_report, build_drift_trace,
                                                           load_drift_bundle, render_drift_report, write_drift_bundle)

    base = _raw(experiment_id="rep", baseline={"batch": {"size": 3}, "rollout": {"dtype": "fp32"}, "training": {"compute_dtype": "fp32"},
                                               "logp": {"backend": "reference"}},
                interventions=[{"path": "batch.size", "values": [1]}],
                operators={"selected_logprob": {"rollout": {"backend": "reference"}, "training": {"backend": "smoke_only.logp_offset"}}})
    run_cpu_experiment(config_from_dict(base), tmp_path, bitwise=False)
    rep = build_drift_report(tmp_path / "rep")
    assert rep["overall"] == "failure" and len(rep["cases"]) == 2
    c = rep["cases"][0]
    assert c["status"] == "fail" and c["recomputed_comparison_matches"] and abs(c["worst_tokens"][0]["abs_diff"] - 0.25) < 1e-5
    assert c["sides"]["training"]["actual"]["logp.backend"] == "smoke_only.logp_offset" and sum(c["delta_histogram"]) == 24
    trace = build_drift_trace(rep)
    assert sum(1 for e in trace["traceEvents"] if e.get("cat") == "case") == 2
    page = render_drift_report(rep)
    assert page.startswith("<!doctype html>") and "FAIL" in page and "<script" not in page
    bundle = load_drift_bundle(write_drift_bundle(rep, tmp_path / "b.zip"))
    assert bundle["report"]["experiment_id"] == "rep" and bundle["html"]
    attempt = next((tmp_path / "rep" / "paired").iterdir()) / "0"
    (attempt / "result.json").write_text("{}")
    broken = build_cross_config_attempt_report(attempt)
    assert broken["level"] == "failure" and "seal" in broken["reason"]


def test_artifact_store_is_append_only_atomic_and_sealed(tmp_path):
    import torch

    from rl_kernel_b200.validation.cross_config.artifacts import ArtifactError, ArtifactStore

    store = ArtifactStore(tmp_path)
    cfg = {"model": "tiny", "knobs": {"tp": [1, 2]}}
    d = store.initialize_experiment("exp-1", cfg, plan={"cases": ["a", "b"]})
    assert store.initialize_experiment("exp-1", cfg, plan={"cases": ["a", "b"]}) == d                    # re-opening with the same content
    with pytest.raises(ArtifactError, match="different content"):
        store.initialize_experiment("exp-1", {**cfg, "model": "other"})
    for bad in ("../x", "a/b", "", ".hidden", "x" * 200):
        with pytest.raises(ArtifactError, match="safe path component"):
            store.experiment_dir(bad)
    req = {"case": "a", "seed": 1}
    a0 = store.create_attempt("exp-1", "case-a", req)
    a1 = store.create_attempt("exp-1", "case-a", req)
    assert (a0.name, a1.name) == ("0", "1") and (a0 / "request.json").exists()
    store.write_json(a0, "rollout", {"x": 1})
    store.write_json(a0, "rollout.json", {"x": 1})                                                        # identical content: a no-op
    with pytest.raises(ArtifactError, match="different content"):
        store.write_json(a0, "rollout", {"x": 2})
    with pytest.raises(ArtifactError):
        store.write_json(a0, "../escape", {"x": 1})
    bundle = store.write_tensor_bundle(a0, "tensors", {"logp": torch.arange(6.0)}, metadata={"tokens": 6})
    with pytest.raises(ArtifactError, match="append-only"):
        store.write_tensor_bundle(a0, "tensors", {"logp": torch.zeros(1)})
    loaded = store.load_tensor_bundle(bundle)
    assert torch.equal(loaded["tensors"]["logp"], torch.arange(6.0)) and loaded["metadata"] == {"tokens": 6}
    assert store.completed_attempt("exp-1", "case-a") is None
    store.complete_attempt(a0, {"mismatches": 0})
    rec = store.validate_completed_attempt(a0)
    assert set(rec["artifacts"]) == {"request.json", "rollout.json", "tensors.pt"} and rec["summary"] == {"mismatches": 0}
    assert store.completed_attempt("exp-1", "case-a", req) == a0 and store.completed_attempt("exp-1", "case-a", {"case": "a", "seed": 2}) is None
    with pytest.raises(ArtifactError, match="already complete"):
        store.complete_attempt(a0)
    with pytest.raises(ArtifactError, match="nothing can be added"):
        store.write_json(a0, "late", {})
    assert not [p for p in a0.iterdir() if ".tmp" in p.name]                                              # no half-written files are left behind
    # tampering is found, and a newer intact attempt is preferred
    (a0 / "rollout.json").write_text("{}")
    with pytest.raises(ArtifactError, match="modified after completion"):
        store.validate_completed_attempt(a0)
    assert store.completed_attempt("exp-1", "case-a") is None
    store.complete_attempt(a1)
    assert store.completed_attempt("exp-1", "case-a") == a1
    (a1 / "extra.json").write_text("{}")
    with pytest.raises(ArtifactError, match="added"):
        store.validate_completed_attempt(a1)
    with pytest.raises(ArtifactError, match="not a tensor bundle"):
        torch.save({"x": 1}, tmp_path / "other.pt")
        store.load_tensor_bundle(tmp_path / "other.pt")


def test_paired_runner_publishes_one_append_only_attempt_per_case(tmp_path):
    import rl_kernel_b200.validation.cross_config as cc
    from rl_kernel_b200.validation.cross_config.execution_plan import build_execution_plan

    assert {"PairedRunner", "PairedRunResult", "Planner", "ArtifactStore", "compare_score_artifacts", "load_config"} <= set(cc.__all__)
    cfg = config_from_dict(_raw())
    ro, tr = ReferenceModelScorer("rollout", prefill_tokens=5), ReferenceModelScorer("training")
    store, runner = cc.ArtifactStore(tmp_path), cc.PairedRunner(cc.ArtifactStore(tmp_path), timeout_seconds=20.0)
    with pytest.raises(ValueError):
        cc.PairedRunner(store, timeout_seconds=0.0)
    mats, tools = reference_materializers(), RuntimeTools()
    batch = CanonicalScoringBatch.from_identity(cfg.definition.identity)
    case = build_execution_plan(cfg).entries[0].case
    m = tools.materialize(case, mats)
    r = runner.run("exp", case, m, batch, ro, tr, materializers=mats, bitwise=True)
    assert not r.resumed and r.alignment.passed and r.summary["mismatch_count"] == 0 and r.summary["active_token_count"] == 24
    rec = store.validate_completed_attempt(r.attempt_dir)
    assert set(rec["artifacts"]) == {"request.json", "rollout.json", "training.json", "tensors.pt", "result.json"}
    bundle = store.load_tensor_bundle(r.attempt_dir / "tensors.pt")
    assert torch.equal(bundle["tensors"]["rollout_logprobs"], bundle["tensors"]["training_logprobs"])
    again = runner.run("exp", case, m, batch, ro, tr, materializers=mats, bitwise=True)
    assert again.resumed and again.attempt_dir == r.attempt_dir and again.summary == r.summary
    fresh = runner.run("exp", case, m, batch, ro, tr, materializers=mats, bitwise=True, resume=False)
    assert not fresh.resumed and fresh.attempt_dir.name == "1"
    other = runner.run("exp", case, m, batch, ro, tr, materializers=mats, bitwise=False)                  # another request: a new attempt
    assert not other.resumed and other.attempt_dir.name == "2"
    with pytest.raises(ex.PairedRunnerError, match="not executable|is for case"):
        runner.run("exp", build_execution_plan(cfg).entries[1].case, m, batch, ro, tr)
    assert runner.active_child_pids == ()
