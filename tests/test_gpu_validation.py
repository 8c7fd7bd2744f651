"""The operator validation harness on the sm_100a candidates: every operator green in all four judgments
(forward / gradient accuracy against the fp32 gold, forward / gradient invariance per logical token across
packed, permuted, singleton, chunked and padded presentations of one logical batch)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_four_judgment_matrix_is_green_for_the_device_candidates():
    from rl_kernel_b200.validation.operators.four_judgment_matrix import four_judgment_matrix

    m = four_judgment_matrix(device="cuda", dtype=torch.bfloat16, candidate="b200")
    assert m.green, m.render() + "\n" + "\n".join(str(c) for c in m.red_cells())


def test_forward_invariance_reports_an_injected_row_dependence():
    """The harness is not vacuous: a candidate whose output depends on its row index turns the matrix red."""
    from rl_kernel_b200.validation.operators import operator_specs as specs
    from rl_kernel_b200.validation.operators.forward_invariance import run_forward_invariance

    good = specs.FACTORIES["swiglu"]

    class Leaky:
        def __call__(self, g, u):
            y = good()(g, u)
            y[1::2] += 1.0e-2
            return y

    specs.FACTORIES["swiglu"] = Leaky
    try:
        rep = run_forward_invariance("swiglu", candidate="b200", device="cuda", dtype=torch.bfloat16)
    finally:
        specs.FACTORIES["swiglu"] = good
    assert not rep.forward_invariant and "BN/permuted" in rep.failing()


def test_cross_config_runner_drives_the_engine_and_sees_an_injected_offset(tmp_path):
    """Same sequences as whole batch, singletons, micro-batches, right-padded and prefill + cached decode through
    Qwen3Engine: every logical token's log-prob keeps its bits; a smoke-only operator override is reported."""
    from rl_kernel_b200.validation.cross_config.config import ExperimentConfig
    from rl_kernel_b200.validation.cross_config.runner import run_experiment

    cases = [{"name": "ref", "knobs": {}}, {"name": "b1", "knobs": {"batch_size": 1}}, {"name": "b3", "knobs": {"batch_size": 3}},
             {"name": "padr", "knobs": {"padding": "right", "chunk_size": 40}}, {"name": "decode", "knobs": {"decode_from": 100}},
             {"name": "tp2", "knobs": {"tp_size": 2}}]
    base = {"experiment_id": "eng", "reference_case": "ref", "num_sequences": 4, "seq_len": 136, "backend": "engine"}
    s = run_experiment(ExperimentConfig.from_dict({**base, "cases": cases}), tmp_path)
    assert s["all_bitwise_equal"], s
    assert s["blocked_cases"] == ["tp2"]
    bad = cases + [{"name": "off", "knobs": {"operator_override": "smoke_only.logp_offset"}}]
    s2 = run_experiment(ExperimentConfig.from_dict({**base, "experiment_id": "eng2", "cases": bad}), tmp_path)
    assert not s2["all_bitwise_equal"] and s2["cases"]["off"]["mismatch_count"] > 0


def test_paired_alignment_run_on_the_engine_rollout_path_equals_training_path_bitwise(tmp_path):
    """Rollout side = prefill + cached decode, training side = one full forward, both through Qwen3Engine: every
    active token's selected log-prob has the same bits, for the whole batch and for singleton requests."""
    from rl_kernel_b200.validation.cross_config.adapters import EngineScorer, engine_materializers
    from rl_kernel_b200.validation.cross_config.config import config_from_dict
    from rl_kernel_b200.validation.cross_config.runner import run_alignment
    from rl_kernel_b200.validation.cross_config.schema import SemanticIdentitySpec

    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 4096, (4, 160), generator=g)
    act = torch.ones(4, 160, dtype=torch.bool)
    act[:, -1] = False
    act[:, :32] = False
    ident = SemanticIdentitySpec.from_tensors(checkpoint_id="synthetic-seed0", model_version="qwen3-scaled", token_ids=ids,
                                              selected_token_ids=torch.roll(ids, -1, 1), active_mask=act)
    raw = {"schema_version": "cross_config.experiment_config.v1", "experiment_id": "eng-pair", "scenario_id": "s0",
           "identity": {k: v for k, v in ident.to_dict().items() if k != "schema_version"},
           "baseline": {"batch": {"size": 4}, "rollout": {"dtype": "bf16", "tensor_parallel_size": 1}, "training": {"compute_dtype": "bf16"}, "logp": {"backend": "b200"}},
           "interventions": [{"path": "batch.size", "values": [4, 1]}, {"path": "rollout.tensor_parallel_size", "values": [1, 2]}]}
    s = run_alignment(config_from_dict(raw), tmp_path, rollout=EngineScorer("rollout", prefill_tokens=100), training=EngineScorer("training"),
                      materializers=engine_materializers(), bitwise=True)
    ran = [c for c in s["cases"].values() if "passed" in c]
    assert len(ran) == 2 and s["all_passed"], s
    assert len(s["not_executable"]) == 1           # tensor parallel size 2 is refused by the one-GPU adapter, not ignored


def test_chain_gate_on_the_engine_forward_cells_bitwise_and_gradients_against_fp32_autograd():
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.validation.models.chain_gate import run_engine_chain_gate

    spec = Qwen3DenseSpec.scaled(layers=2, hidden=512, ffn=1536, q_heads=4, kv_heads=2, head_dim=128, vocab=4096)
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    ids = torch.randint(0, spec.vocab_size, (4, 256), generator=torch.Generator().manual_seed(0))
    res = run_engine_chain_gate(spec, w, ids, prompt_len=128, decode_from=200)
    assert res.passed, (res.cells, res.aggregates, res.gradient_cells, res.gradient_accuracy, res.missing_grads)
    assert set(res.cells) == {"packed/full", "singletons", "permuted", "padded_batch", "micro_batches", "chunked/decode"}
