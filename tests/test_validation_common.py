"""validation.common: attention attribution paths, log-prob comparison, RL batches, distributed vocabulary-parallel
comparison over gloo ranks."""
import json
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from rl_engine.validation.common import (AttentionComparisonInputs, DecodeAttentionInputs, DecodeKVCacheMetadata,
                                         compare_decode_kv_replay, compare_single_gpu_attention, compare_single_gpu_rope_attention,
                                         decode_kv_cache_fingerprint, decode_prefix_cache_fingerprint,
                                         decode_rope_identity_fingerprint, make_synthetic_rl_kernel_batch,
                                         run_decode_strict_shared_core, run_strict_shared_core_attention, summarize_logprob_drift)
from rl_engine.validation.common.distributed_logprob_comparison import (DistributedLogprobCase, plan_distributed_logprob_cases,
                                                                        rank_topology, run_distributed_logprob_case,
                                                                        token_shard_bounds, vocab_shard_bounds)
from rl_engine.validation.common.logprob_comparison import (LogprobBackendUnavailable, LogprobComparisonInputs,
                                                            compare_single_gpu_logprob, make_logprob_candidate)


def _qkv(B=2, S=40, Hq=4, Hkv=2, D=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(B, S, Hq, D, generator=g), torch.randn(B, S, Hkv, D, generator=g), torch.randn(B, S, Hkv, D, generator=g), g)


def test_strict_attention_paths_are_bitwise_and_tolerance_paths_are_close():
    q, k, v, g = _qkv()
    W = torch.randn(50, 64, generator=g) * 0.1
    tg = torch.randint(0, 50, (2, 40), generator=g)
    inp = AttentionComparisonInputs(q, k, v, lm_head_weight=W, target_ids=tg)
    loose = compare_single_gpu_attention(inp, query_chunk_size=7, kv_page_size=16)
    assert [d.candidate_name for d in loose.drifts] == ["chunked_query_attention", "paged_kv_attention"]
    assert all(d.out.max_abs < 1e-5 and d.dlogp.max_abs < 1e-5 for d in loose.drifts)
    strict = compare_single_gpu_attention(inp, query_chunk_size=7, kv_page_size=16, strict_bitwise=True, include_transformer_engine=True)
    assert strict.bitwise and all(d.dlogp.max_abs == 0.0 for d in strict.drifts)
    assert strict.unavailable and "transformer_engine" in strict.unavailable[0]
    json.dumps(strict.to_dict())
    with pytest.raises(ValueError):
        compare_single_gpu_attention(AttentionComparisonInputs(q, k[:, :30], v[:, :30]))


def test_rope_placement_drift_is_attributed_to_the_rotated_operands():
    q, k, v, _ = _qkv()
    same = compare_single_gpu_rope_attention(AttentionComparisonInputs(q.bfloat16(), k.bfloat16(), v.bfloat16()))
    assert same.drifts[0].out.max_abs == 0.0 and same.drifts[0].post_rope_q.max_abs == 0.0
    late = compare_single_gpu_rope_attention(AttentionComparisonInputs(q.bfloat16(), k.bfloat16(), v.bfloat16(),
                                                                       rope_cast_at="after_attention"))
    assert late.drifts[0].post_rope_q.max_abs > 0.0 and late.drifts[0].out.max_abs > 0.0


def _decode_inputs(q, k, v, table, n, page=8, pages=10, **md_kw):
    B, _, Hkv, D = k.shape
    kc, vc = torch.zeros(pages, page, Hkv, D), torch.zeros(pages, page, Hkv, D)
    cpos = torch.full((pages, page), -1)
    for b in range(B):
        for p in range(n[b]):
            pg = table[b, p // page]
            kc[pg, p % page], vc[pg, p % page], cpos[pg, p % page] = k[b, p], v[b, p], p
    last = torch.tensor([x - 1 for x in n])
    md = DecodeKVCacheMetadata(cpos, torch.tensor(n), table, last, last, torch.arange(32).repeat(B, 1), page, prefix_length=8,
                               prefix_cache_enabled=True, **md_kw)
    return DecodeAttentionInputs(torch.stack([q[b, n[b] - 1] for b in range(B)]), kc, vc, md)


def test_decode_replay_matches_prefill_and_fingerprints_ignore_the_page_assignment():
    q, k, v, _ = _qkv()
    n = [21, 13]
    a = _decode_inputs(q, k, v, torch.tensor([[7, 2, 5, -1], [1, 9, -1, -1]]), n)
    b = _decode_inputs(q, k, v, torch.tensor([[0, 1, 2, -1], [3, 4, -1, -1]]), n)
    rep = compare_decode_kv_replay(a, strict_bitwise=True)
    assert all(d.out.max_abs < 1e-5 and d.lse.max_abs < 1e-5 for d in rep.drifts)
    full = run_strict_shared_core_attention(AttentionComparisonInputs(q, k, v))
    sd = run_decode_strict_shared_core(a)
    assert torch.equal(sd.out[0], full.out[0, 20]) and torch.equal(sd.out[1], full.out[1, 12])
    assert torch.equal(run_decode_strict_shared_core(b).out, sd.out)
    for fp in (decode_kv_cache_fingerprint, decode_prefix_cache_fingerprint, decode_rope_identity_fingerprint):
        assert fp(a) == fp(b)
    k2 = k.clone()
    k2[0, 3, 0, 0] += 1
    c = _decode_inputs(q, k2, v, torch.tensor([[7, 2, 5, -1], [1, 9, -1, -1]]), n)
    assert decode_kv_cache_fingerprint(c) != decode_kv_cache_fingerprint(a)
    assert decode_prefix_cache_fingerprint(c) != decode_prefix_cache_fingerprint(a)
    # owners under paged context parallelism change the merge tree, not the result beyond rounding
    owners = torch.tensor([[0, 1, 0, 0], [1, 0, 0, 0]])
    d = _decode_inputs(q, k, v, torch.tensor([[7, 2, 5, -1], [1, 9, -1, -1]]), n, cp_block_owners=owners, cp_world_size=2)
    assert compare_decode_kv_replay(d).drifts[0].out.max_abs < 1e-5
    bad = _decode_inputs(q, k, v, torch.tensor([[7, 2, 5, -1], [1, 9, -1, -1]]), n)
    bad.metadata.cache_position[7, 0] = 5
    with pytest.raises(ValueError, match="cache_position"):
        compare_decode_kv_replay(bad)


def test_logprob_comparison_and_drift_summary():
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(33, 1000, generator=g) * 3
    tg = torch.randint(0, 1000, (33,), generator=g)
    tg[4] = -100
    rep = compare_single_gpu_logprob(LogprobComparisonInputs(logits, tg), ("pytorch",))
    d = rep.drifts[0]
    assert d.dlogp.active_count == 32 and d.dlogp.max_abs < 1e-5 and d.lse.max_abs < 1e-5
    assert rep.input_provenance["active"] == 32
    if not torch.cuda.is_available():
        with pytest.raises(LogprobBackendUnavailable):
            make_logprob_candidate("cuda-sm100")
    with pytest.raises(ValueError):
        make_logprob_candidate("rocm")
    s = summarize_logprob_drift(torch.tensor([1.0, 2.0, 4.0]), torch.tensor([1.0, 2.5, 4.0]), mask=torch.tensor([True, True, False]))
    assert s.max_abs == 0.5 and s.active_count == 2 and s.mean_abs == 0.25
    with pytest.raises(ValueError):
        summarize_logprob_drift(torch.zeros(2), torch.zeros(3))


def test_synthetic_rl_batch_is_deterministic_and_group_shaped():
    a = make_synthetic_rl_kernel_batch(num_prompts=3, samples_per_prompt=4, prompt_len=5, completion_len=7, vocab_size=100,
                                       valid_density=0.5, seed=9)
    b = make_synthetic_rl_kernel_batch(num_prompts=3, samples_per_prompt=4, prompt_len=5, completion_len=7, vocab_size=100,
                                       valid_density=0.5, seed=9)
    assert torch.equal(a.input_ids, b.input_ids) and torch.equal(a.completion_mask, b.completion_mask)
    assert a.batch_size == 12 and a.prompt_len == 5 and a.completion_len == 7 and a.total_seq_len == 12
    assert torch.equal(a.input_ids[0, :5], a.input_ids[3, :5]) and int(a.completion_mask.sum()) == 42 == a.valid_indices.numel()
    vals = torch.arange(42.0)
    assert torch.equal(a.compact_completion_values(a.dense_completion_values(vals)), vals)
    assert a.benchmark_metadata()["valid_fraction"] == 0.5
    with pytest.raises(ValueError):
        make_synthetic_rl_kernel_batch(num_prompts=0, samples_per_prompt=1, prompt_len=1, completion_len=1, vocab_size=10)


def test_distributed_case_planning():
    cases = plan_distributed_logprob_cases(real_vocab_size=1000, padded_vocab_size=1024, num_vocab_tiles=8)
    assert [(c.tp_world_size, c.cp_world_size) for c in cases] == [(1, 1), (1, 2), (2, 1), (2, 2), (4, 1), (4, 2)]
    c = cases[3]
    assert rank_topology(c, 3).tp_group_ranks == (2, 3) and rank_topology(c, 3).cp_rank == 1
    assert token_shard_bounds(7, 3) == ((0, 3), (3, 5), (5, 7))
    assert vocab_shard_bounds(DistributedLogprobCase(3, 1, real_vocab_size=1000, padded_vocab_size=1024, num_vocab_tiles=8)) == \
        ((0, 384), (384, 768), (768, 1024))
    assert len({x.case_id for x in cases}) == 6
    with pytest.raises(ValueError):
        DistributedLogprobCase(2, 1, real_vocab_size=1000, padded_vocab_size=1024, num_vocab_tiles=7)
    with pytest.raises(ValueError):
        DistributedLogprobCase(1, 1, requested_backend="auto")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dist_worker(rank, world, port, case_kw, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    run_distributed_logprob_case(DistributedLogprobCase(**case_kw), device="cpu", dist_backend="gloo", output=out)


def test_distributed_logprob_comparison_is_topology_invariant(tmp_path):
    kw = dict(dtype="fp32", real_vocab_size=1000, padded_vocab_size=1024, num_vocab_tiles=8, batch_size=2, sequence_length=9,
              prompt_tokens=4)
    prints = {}
    for tp, cp in ((1, 1), (2, 2)):
        out = str(tmp_path / f"tp{tp}cp{cp}.json")
        mp.spawn(_dist_worker, args=(tp * cp, _free_port(), dict(kw, tp_world_size=tp, cp_world_size=cp), out), nprocs=tp * cp,
                 join=True)
        rep = json.loads(open(out).read())
        assert rep["passed"] and len(rep["ranks"]) == tp * cp
        assert all(r["tp_outputs_bitwise_replicated"] for r in rep["ranks"])
        prints[(tp, cp)] = (rep["bitwise_fingerprints"]["logp_active_sha256"], rep["bitwise_fingerprints"]["lse_active_sha256"])
    assert prints[(1, 1)] == prints[(2, 2)]


def test_attention_debug_matrix_runs_every_row():
    from rl_engine.contracts.diagnostics.attention_axes import attention_debug_probe_metadata, attention_debug_taxonomy
    from rl_engine.contracts.diagnostics.attention_matrix import attention_debug_matrix_row
    from rl_engine.contracts.diagnostics.modules import module_debug_axis, module_debug_matrix
    from rl_engine.reference.attention.ablation import PROBES, make_debug_inputs, run_attention_debug_matrix, run_attention_subprobe

    r = run_attention_debug_matrix(make_debug_inputs(seq=160, head_dim=16))
    by_id = {row["id"]: row for row in r["rows"]}
    assert r["passed"] and len(by_id) == 11 and by_id["A0"]["status"] == "baseline" and by_id["A4"]["status"] == "rejected"
    assert all(by_id[f"C{i}"]["status"] == "pass" and by_id[f"C{i}"]["out_max_abs"] == 0.0 for i in range(3))
    assert all(by_id[f"A{i}"]["out_max_abs"] > 0 for i in (1, 2, 3, 5, 6, 7))
    tax = attention_debug_taxonomy()
    assert tax["root_cause_axis_count"] == 7 and set(PROBES) == {p for a in tax["root_cause_axes"].values() for p in a["subprobes"]} - {"tp_head_ownership"}
    assert run_attention_subprobe("rope_theta", make_debug_inputs(seq=64, head_dim=16))["out_max_abs"] > 0
    assert attention_debug_probe_metadata("split_kv")["root_cause_axis"] == "distributed_schedule"
    assert attention_debug_matrix_row("A7").probe == "merge_order" and module_debug_axis("logp", "vocab_lse_reduction").kind == "diagnostic"
    assert module_debug_matrix()["modules"]["ffn"]["rows"] == ["F0", "F1", "F2", "F3", "F4"]


def test_cp_attention_reference_strict_and_ring_paths():
    from rl_engine.reference.attention.cp_attention import (AttentionRingSchedule, DeterministicCPAttentionReferenceOp,
                                                            compare_cp_attention_backward)

    g = torch.Generator().manual_seed(0)
    S = 96
    q, k, v = torch.randn(S, 4, 16, generator=g), torch.randn(S, 2, 16, generator=g), torch.randn(S, 2, 16, generator=g)
    one = DeterministicCPAttentionReferenceOp(1)(q, k, v)
    for cp in (2, 4):
        assert torch.equal(DeterministicCPAttentionReferenceOp(cp)(q, k, v)[0], one[0])
        ring = DeterministicCPAttentionReferenceOp(cp, strict_bitwise=False)(q, k, v)
        assert 0 < float((ring[0] - one[0]).abs().max()) < 1e-5
    s = AttentionRingSchedule.build(cp_world_size=2, seq_len=96)
    assert s.owned(1) == [(24, 48), (48, 72)] and len(s.arrivals(0)) == 4 and s.provenance()["blocks"] == 8
    rep = compare_cp_attention_backward(q, k, v, torch.randn(S, 4, 16, generator=g), cp_world_size=2)
    assert rep.dq.max_abs == 0.0 and rep.dk.max_rel < 1e-5 and len(rep.ranks) == 2


def test_kv_consistency_op_checks_inventory_and_accelerator():
    from rl_engine.validation.models.chain_gradients import missing_required_grads, required_grad_names
    from rl_engine.validation.operators import accelerator as acc
    from rl_engine.validation.operators.elementwise_inventory import inventory_items, unexecuted_cells, unresolved_needs_fix
    from rl_engine.validation.operators.kv_consistency import (DecodePrefillCase, assert_decode_prefill_consistent,
                                                               assert_stateful_kv_consistent)

    r = assert_decode_prefill_consistent(device="cpu", cases=[DecodePrefillCase("b", 1, 132, 127, head_dim=16)])
    assert r.bitwise and len(r.cells) == 5
    s = assert_stateful_kv_consistent(device="cpu", case=DecodePrefillCase("s", 1, 50, 44, head_dim=16))
    assert s.bitwise and s.writes == 7
    assert not unexecuted_cells() and not unresolved_needs_fix() and len(inventory_items()) >= 15
    assert len(required_grad_names(num_hidden_layers=36)) == 3 + 36 * 11
    assert missing_required_grads([f"model.{n}" for n in required_grad_names(num_hidden_layers=2)][1:], num_hidden_layers=2) == ("embed_tokens.weight",)
    assert acc.arch_key(acc.resolve_device("cpu")) == "cpu" and acc.disable_tf32("cpu") is False
    if not torch.cuda.is_available():
        with pytest.raises(acc.AcceleratorUnavailable):
            acc.resolve_device(profile="b200_bf16")


def test_every_legacy_alias_resolves():
    import importlib

    from rl_engine._legacy import LEGACY_ALIASES

    bad = []
    for old in sorted(LEGACY_ALIASES):
        if old.endswith("__main__"):
            continue
        try:
            importlib.import_module("rl_engine." + old)
        except Exception as exc:  # noqa: BLE001
            bad.append(f"{old}: {type(exc).__name__}: {exc}")
    assert not bad, "\n".join(bad)
