"""The framework-facing linear log-prob wrapper on the CPU definition of the tile contract: single rank against
log_softmax, tensor-parallel (gloo, 2 ranks) against the single-rank bits, gradients, restricted supports from id
lists, the rollout hand-over context and the diagnostics records."""
import datetime
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rl_kernel_b200.integrations.common.linear_logp import (LinearLogpWrapper, alignment_tensor_summary,
                                                          clear_rollout_linear_logp_context,
                                                          publish_rollout_linear_logp_context,
                                                          take_rollout_linear_logp_context)

BF = torch.bfloat16


def _case(seed=0, n=11, h=64, real=1900, padded=2048):
    g = torch.Generator().manual_seed(seed)
    hidden = torch.randn(n, h, generator=g).to(BF)
    weight = (torch.randn(padded, h, generator=g) * 0.3).to(BF)
    weight[real:] = 0
    targets = torch.randint(0, real, (n,), generator=g)
    return hidden, weight, targets, real, padded


def _ref_logp(hidden, weight, targets, real, temperature):
    logits = (hidden.float() @ weight[:real].float().t()).to(BF).float()          # logits are rounded to the compute dtype
    return torch.log_softmax(logits / temperature, -1).gather(1, targets[:, None])[:, 0]


def test_single_rank_matches_log_softmax_and_is_batch_invariant():
    hidden, weight, targets, real, padded = _case()
    w = LinearLogpWrapper()
    lp, lse = w(hidden, weight, targets, real_vocab_size=real, temperature=0.7, return_lse=True)
    ref = _ref_logp(hidden, weight, targets, real, 0.7)
    assert (lp - ref).abs().max().item() < 2e-5
    assert torch.equal(w(hidden, weight, targets, real_vocab_size=real, temperature=0.7), lp)        # fused path, no lse
    assert torch.equal(w(hidden[3:4], weight, targets[3:4], real_vocab_size=real, temperature=0.7), lp[3:4])
    prov = w.provenance
    assert prov["strict_entrypoint"] == "fused_lm_head" and prov["real_vocab_size"] == real and prov["tp_world_size"] == 1
    assert prov["arithmetic_contract"]["summary_merge_order"] == "ascending_tile"
    # [B, S] shaped ids and a mask
    m = torch.tensor([True, False] * 5 + [True])
    lp2 = w(hidden, weight, targets, real_vocab_size=real, temperature=0.7, mask=m)
    assert torch.equal(lp2[m], lp[m]) and (lp2[~m] == 0).all()


def test_per_row_temperature_equals_rows_scored_alone():
    hidden, weight, targets, real, _ = _case(1)
    temps = torch.tensor([0.5, 1.0, 0.5, 2.0, 1.0, 1.0, 0.5, 2.0, 2.0, 0.5, 1.0])
    w = LinearLogpWrapper()
    lp = w(hidden, weight, targets, real_vocab_size=real, temperature=temps)
    assert w.provenance["temperature"] == "per_row"
    for i in range(hidden.shape[0]):
        assert torch.equal(lp[i:i + 1], w(hidden[i:i + 1], weight, targets[i:i + 1], real_vocab_size=real, temperature=float(temps[i])))
    with pytest.raises(ValueError):
        w(hidden, weight, targets, real_vocab_size=real, temperature=torch.tensor([1.0, 0.0] + [1.0] * 9))
    with pytest.raises(ValueError):
        w(hidden, weight, targets, real_vocab_size=real, temperature=torch.ones(3))


def test_gradients_match_autograd_of_the_reference_expression():
    hidden, weight, targets, real, _ = _case(2, n=7, h=32, real=300, padded=384)
    g = torch.randn(7, generator=torch.Generator().manual_seed(9))
    for return_lse in (False, True):
        h1, w1 = hidden.clone().requires_grad_(True), weight.clone().requires_grad_(True)
        out = LinearLogpWrapper()(h1, w1, targets, real_vocab_size=real, temperature=0.9, return_lse=return_lse)
        lp = out[0] if return_lse else out
        (lp * g).sum().backward()
        h2, w2 = hidden.float().requires_grad_(True), weight.float().requires_grad_(True)
        ref = torch.log_softmax((h2 @ w2[:real].t()) / 0.9, -1).gather(1, targets[:, None])[:, 0]
        (ref * g).sum().backward()
        assert (h1.grad.float() - h2.grad).abs().max().item() < 0.05 * h2.grad.abs().max().item() + 1e-3
        assert (w1.grad.float() - w2.grad).abs().max().item() < 0.05 * w2.grad.abs().max().item() + 1e-3
        assert (w1.grad[real:] == 0).all()


def test_bias_and_reused_logits_paths_agree():
    hidden, weight, targets, real, padded = _case(3)
    bias = (torch.randn(padded, generator=torch.Generator().manual_seed(4)) * 0.2).to(BF)
    w = LinearLogpWrapper()
    lp = w(hidden, weight, targets, bias, real_vocab_size=real, temperature=1.3)
    assert w.provenance["logits_materialized"] is True
    from rl_kernel_b200.reference.gemm import det_gemm_reference

    logits = (det_gemm_reference(hidden, weight).float() + bias.float()).to(BF)
    again, lse = w.from_local_logits(logits, targets, global_vocab_size=padded, real_vocab_size=real, temperature=1.3, return_lse=True)
    assert torch.equal(again, lp)
    ref = torch.log_softmax(logits[:, :real].float() / 1.3, -1)
    assert (lp - ref.gather(1, targets[:, None])[:, 0]).abs().max().item() < 2e-5
    assert (lse - torch.logsumexp(logits[:, :real].float() / 1.3, -1)).abs().max().item() < 2e-5
    # fp32 logits are accepted too; a restricted support by threshold equals masking first
    z = logits[:, :real].float() * (1.0 / 1.3)                      # the contract scales by the reciprocal temperature
    thr = z.topk(20, -1).values[:, -1]
    tk = z.topk(20, -1).indices[:, 0]
    a = w.from_local_logits(logits, tk, global_vocab_size=padded, real_vocab_size=real, temperature=1.3, min_keep=thr)
    masked = logits.clone()
    masked[:, :real] = torch.where(z < thr[:, None], torch.full_like(logits[:, :real], float("-inf")), logits[:, :real])
    assert torch.equal(a, w.from_local_logits(masked, tk, global_vocab_size=padded, real_vocab_size=real, temperature=1.3))


def test_argument_checks():
    hidden, weight, targets, real, padded = _case(5)
    w = LinearLogpWrapper()
    with pytest.raises(ValueError, match="real_vocab_size"):
        w(hidden, weight, targets, real_vocab_size=padded + 1)
    with pytest.raises(ValueError, match="target_ids"):
        w(hidden, weight, torch.full_like(targets, real), real_vocab_size=real)
    with pytest.raises(TypeError):
        w(hidden, weight, targets.float(), real_vocab_size=real)
    with pytest.raises(ValueError, match="explicit TP process group"):
        w(hidden, weight, targets, vocab_start_index=2048, real_vocab_size=real)
    with pytest.raises(ValueError, match="complete local vocab"):
        w(hidden, weight, targets, global_vocab_size=4096, real_vocab_size=real)
    with pytest.raises(ValueError, match="bias"):
        w(hidden, weight, targets, torch.zeros(3), real_vocab_size=real)
    with pytest.raises(ValueError, match="hidden width"):
        w(hidden[:, :32], weight, targets, real_vocab_size=real)


def test_sparse_nucleus_equals_masked_scoring_with_entropy():
    hidden, weight, _, real, padded = _case(6, n=9)
    from rl_kernel_b200.reference.gemm import det_gemm_reference

    logits = det_gemm_reference(hidden, weight)
    z = logits[:, :real].float() / 0.8
    for K in (12, 100):                                             # compact replay and the wide (masked) route
        ids = z.topk(K, -1).indices
        targets = ids[torch.arange(9), torch.randint(0, K, (9,), generator=torch.Generator().manual_seed(K))]
        ids_padded = torch.cat([ids, torch.full((9, 3), -1)], 1)  # padding entries
        w = LinearLogpWrapper()
        lp, ent = w.from_local_logits_sparse_nucleus(logits, targets, ids_padded, global_vocab_size=padded, real_vocab_size=real,
                                                     temperature=0.8, return_entropy=True)
        masked = torch.full_like(z, float("-inf")).scatter(1, ids, z.gather(1, ids))
        ref = torch.log_softmax(masked, -1)
        assert (lp - ref.gather(1, targets[:, None])[:, 0]).abs().max().item() < 2e-5
        p = torch.softmax(masked, -1)
        want_ent = -(p * torch.where(p > 0, torch.log(p), torch.zeros_like(p))).sum(-1)
        assert (ent - want_ent).abs().max().item() < 1e-4
        assert w.provenance["strict_entrypoint"] == ("sparse_nucleus_compact" if K <= 64 else "sparse_nucleus_masked")
        # the sampler's transport format: finite log-probs mark the retained ids
        rl = torch.where(ids_padded >= 0, torch.zeros(ids_padded.shape), torch.full(ids_padded.shape, float("-inf")))
        assert torch.equal(w.from_local_logits_top_p(logits, targets, ids_padded.clamp_min(0), rl, global_vocab_size=padded,
                                                     real_vocab_size=real, temperature=0.8), lp)
        with torch.no_grad():
            rep = w.from_replicated_logits_sparse_nucleus(logits[:, :real].contiguous(), targets, ids, real_vocab_size=real, temperature=0.8)
        assert torch.equal(rep, lp)
    with pytest.raises(ValueError, match="does not contain every target"):
        LinearLogpWrapper().from_local_logits_sparse_nucleus(logits, torch.full((9,), 5), (torch.zeros(9, 4, dtype=torch.long) + 7),
                                                             global_vocab_size=padded, real_vocab_size=real, temperature=0.8)


def test_rollout_context_hand_over():
    hidden, weight, _, real, padded = _case(7)
    clear_rollout_linear_logp_context()
    with pytest.raises(RuntimeError, match="no matching"):
        take_rollout_linear_logp_context()
    publish_rollout_linear_logp_context(hidden, weight, None, tp_group=None, vocab_start_index=0, global_vocab_size=padded,
                                        real_vocab_size=real)
    ctx = take_rollout_linear_logp_context()
    assert ctx.hidden is hidden and ctx.real_vocab_size == real and ctx.global_vocab_size == padded
    with pytest.raises(RuntimeError):
        take_rollout_linear_logp_context()                          # consumed
    with pytest.raises(ValueError, match="real vocab cannot exceed"):
        publish_rollout_linear_logp_context(hidden, weight, None, tp_group=None, vocab_start_index=0, global_vocab_size=real,
                                            real_vocab_size=padded)
    with pytest.raises(ValueError, match=r"\[tokens, hidden\]"):
        publish_rollout_linear_logp_context(hidden[0], weight, None, tp_group=None, vocab_start_index=0, global_vocab_size=padded,
                                            real_vocab_size=real)
    with pytest.raises(ValueError, match="bias"):
        publish_rollout_linear_logp_context(hidden, weight, torch.zeros(5), tp_group=None, vocab_start_index=0,
                                            global_vocab_size=padded, real_vocab_size=real)


def test_alignment_diagnostics_records(tmp_path, monkeypatch):
    hidden, weight, targets, real, padded = _case(8)
    monkeypatch.setenv("RL_KERNEL_ALIGNMENT_DIAGNOSTICS", "1")
    monkeypatch.setenv("RL_KERNEL_ALIGNMENT_DIAGNOSTICS_DIR", str(tmp_path))
    w = LinearLogpWrapper()
    lp = w(hidden, weight, targets, real_vocab_size=real, target="training")
    from rl_kernel_b200.reference.gemm import det_gemm_reference

    w.from_local_logits(det_gemm_reference(hidden, weight), targets, global_vocab_size=padded, real_vocab_size=real, target="rollout")
    files = sorted(p.name for p in tmp_path.iterdir())
    assert len(files) == 2 and files[0].startswith("rollout-") and files[1].startswith("training-")
    rec = torch.load(tmp_path / files[1])
    assert torch.equal(rec["result"], lp) and rec["hidden_summary"]["sha256"] == alignment_tensor_summary(hidden)["sha256"]
    roll = torch.load(tmp_path / files[0])
    assert torch.equal(roll["result"], lp) and roll["selected_local_logits"].shape == (hidden.shape[0],)
    monkeypatch.setenv("RL_KERNEL_ALIGNMENT_DIAGNOSTICS", "0")
    w(hidden, weight, targets, real_vocab_size=real)
    assert len(list(tmp_path.iterdir())) == 2


# ------------------------------------------------------------------------------------- two gloo ranks
def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, out):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))
    hidden, weight, targets, real, padded = _case(10, n=13, h=64, real=1900, padded=2048)
    per = padded // world
    shard = weight[rank * per:(rank + 1) * per].clone().requires_grad_(True)
    h = hidden.clone().requires_grad_(True)
    g = torch.randn(13, generator=torch.Generator().manual_seed(1))
    group = dist.group.WORLD
    res = {}
    w = LinearLogpWrapper()
    lp, lse = w(h, shard, targets, tp_group=group, vocab_start_index=rank * per, global_vocab_size=padded, real_vocab_size=real,
                temperature=0.7, return_lse=True)
    (lp * g).sum().backward()
    res.update(lp=lp.detach(), lse=lse.detach(), dh=h.grad.clone(), dw=shard.grad.clone(), prov=w.provenance)
    # the deterministic collective object of this package is accepted in place of a process group
    from rl_kernel_b200.distributed import TorchDistributedDeterministicCollective

    coll = TorchDistributedDeterministicCollective(group)
    res["lp_coll"] = LinearLogpWrapper()(hidden, shard.detach(), targets, tp_group=coll, vocab_start_index=rank * per,
                                         global_vocab_size=padded, real_vocab_size=real, temperature=0.7)
    # logits the rollout engine already holds, per-row temperature, id-list supports
    from rl_kernel_b200.reference.gemm import det_gemm_reference

    logits = det_gemm_reference(hidden, weight)
    local = logits[:, rank * per:(rank + 1) * per].contiguous()
    temps = torch.tensor([0.7, 1.1] * 6 + [0.7])
    res["from_logits"] = w.from_local_logits(local, targets, tp_group=group, vocab_start_index=rank * per, global_vocab_size=padded,
                                             real_vocab_size=real, temperature=temps)
    ids = (logits[:, :real].float()).topk(30, -1).indices
    tsel = ids[:, 4].contiguous()
    res["nucleus"], res["entropy"] = w.from_local_logits_sparse_nucleus(local, tsel, ids, tp_group=group, vocab_start_index=rank * per,
                                                                        global_vocab_size=padded, real_vocab_size=real,
                                                                        temperature=0.9, return_entropy=True)
    wide = (logits[:, :real].float()).topk(90, -1).indices
    res["nucleus_wide"] = w.from_local_logits_sparse_nucleus(local, tsel, wide, tp_group=group, vocab_start_index=rank * per,
                                                             global_vocab_size=padded, real_vocab_size=real, temperature=0.9)
    err = None
    try:
        w(hidden, shard.detach(), targets, tp_group=group, vocab_start_index=0 if rank else per, global_vocab_size=padded,
          real_vocab_size=real)
    except ValueError as e:
        err = str(e)
    res["err"] = err
    torch.save(res, f"{out}.{rank}")
    dist.barrier()
    dist.destroy_process_group()


def test_tensor_parallel_group_gives_the_single_rank_bits(tmp_path):
    out = str(tmp_path / "r")
    mp.spawn(_tp_worker, args=(2, _port(), out), nprocs=2, join=True)
    r0, r1 = (torch.load(f"{out}.{r}", weights_only=False) for r in range(2))
    hidden, weight, targets, real, padded = _case(10, n=13, h=64, real=1900, padded=2048)
    g = torch.randn(13, generator=torch.Generator().manual_seed(1))
    h, wt = hidden.clone().requires_grad_(True), weight.clone().requires_grad_(True)
    one = LinearLogpWrapper()
    lp, lse = one(h, wt, targets, real_vocab_size=real, temperature=0.7, return_lse=True)
    (lp * g).sum().backward()
    for r in (r0, r1):
        assert torch.equal(r["lp"], lp.detach()) and torch.equal(r["lse"], lse.detach()) and torch.equal(r["lp_coll"], lp.detach())
        assert r["prov"]["strict_entrypoint"] == "fused_lm_head_vocab_parallel_gather" and r["prov"]["tp_world_size"] == 2
        assert "does not match the rank-local shard" in r["err"]
    assert torch.equal(r0["dh"], r1["dh"])                                    # the tree sum leaves the same bits on both ranks
    assert (r0["dh"].float() - h.grad.float()).abs().max().item() < 0.03 * h.grad.float().abs().max().item() + 1e-3
    dw = torch.cat([r0["dw"], r1["dw"]])
    assert (dw.float() - wt.grad.float()).abs().max().item() < 0.03 * wt.grad.float().abs().max().item() + 1e-3
    from rl_kernel_b200.reference.gemm import det_gemm_reference

    logits = det_gemm_reference(hidden, weight)
    temps = torch.tensor([0.7, 1.1] * 6 + [0.7])
    want = one.from_local_logits(logits, targets, global_vocab_size=padded, real_vocab_size=real, temperature=temps)
    ids = (logits[:, :real].float()).topk(30, -1).indices
    tsel = ids[:, 4].contiguous()
    nuc, ent = one.from_local_logits_sparse_nucleus(logits, tsel, ids, global_vocab_size=padded, real_vocab_size=real, temperature=0.9,
                                                    return_entropy=True)
    wide = one.from_local_logits_sparse_nucleus(logits, tsel, (logits[:, :real].float()).topk(90, -1).indices, global_vocab_size=padded,
                                                real_vocab_size=real, temperature=0.9)
    for r in (r0, r1):
        assert torch.equal(r["from_logits"], want) and torch.equal(r["nucleus"], nuc) and torch.equal(r["nucleus_wide"], wide)
        assert (r["entropy"] - ent).abs().max().item() < 1e-5
