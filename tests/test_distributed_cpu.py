"""Multi-rank semantics on the CPU (gloo, 2 ranks): vocabulary-parallel log-prob under a contract, context-parallel
attention through the gather runtime and the Megatron operator, canonical (row-sliced) CP weight gradients,
sequence-parallel FFN, partial-state CP merge -- every one compared with the single-process result."""
import datetime
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=60))


def _spawn(fn, tmp_path, world=2):
    out = str(tmp_path / "r")
    mp.spawn(fn, args=(world, _port(), out), nprocs=world, join=True)
    return [torch.load(f"{out}.{r}") for r in range(world)]


# ---------------------------------------------------------------- vocabulary-parallel log-prob, contract driven
def _vp_inputs():
    g = torch.Generator().manual_seed(3)
    N, V, VP = 9, 1900, 2048
    logits = (torch.randn(N, VP, generator=g) * 3).bfloat16()
    targets = torch.randint(0, V, (N,), generator=g)
    mask = torch.tensor([True] * 7 + [False] * 2)
    return logits, targets, mask, V, VP


def _vp_worker(rank, world, port, out):
    _init(rank, world, port)
    from rl_kernel_b200.contracts.operators.logprob import LogprobContract, LogprobContractError
    from rl_kernel_b200.reference.logprob.vocab_parallel_logp import VocabParallelLogprobOp

    logits, targets, mask, V, VP = _vp_inputs()
    per = VP // world
    shard = logits[:, rank * per:(rank + 1) * per].clone().requires_grad_(True)
    c = LogprobContract.for_tokens(logits.shape[0], real_vocab_size=V, padded_vocab_size=VP, tp_rank=rank, tp_world_size=world,
                                   temperature=0.7, active_mask=mask)
    op = VocabParallelLogprobOp()
    lp, lse = op(shard, targets, contract=c, tp_group=None)
    (lp.sum() + 0.25 * lse.sum()).backward()
    _, _, ent = op.apply_with_entropy(shard.detach(), targets, contract=c)
    err = None
    try:                                             # ranks that disagree on the contract stop before any collective
        bad = LogprobContract.for_tokens(logits.shape[0], real_vocab_size=V, padded_vocab_size=VP, tp_rank=rank,
                                         tp_world_size=world, temperature=0.7 if rank == 0 else 0.8, active_mask=mask)
        op(shard.detach(), targets, contract=bad)
    except LogprobContractError as e:
        err = str(e)
    torch.save({"lp": lp.detach(), "lse": lse.detach(), "grad": shard.grad, "ent": ent, "err": err}, f"{out}.{rank}")
    dist.destroy_process_group()


def test_vocab_parallel_logprob_tp2_equals_tp1_bitwise(tmp_path):
    from rl_kernel_b200.contracts.operators.logprob import LogprobContract
    from rl_kernel_b200.reference.logprob.vocab_parallel_logp import VocabParallelLogprobOp

    res = _spawn(_vp_worker, tmp_path)
    logits, targets, mask, V, VP = _vp_inputs()
    full = logits.clone().requires_grad_(True)
    c = LogprobContract.for_tokens(logits.shape[0], real_vocab_size=V, padded_vocab_size=VP, temperature=0.7, active_mask=mask)
    lp, lse = VocabParallelLogprobOp()(full, targets, contract=c)
    (lp.sum() + 0.25 * lse.sum()).backward()
    for r in res:
        assert torch.equal(r["lp"], lp.detach()) and torch.equal(r["lse"], lse.detach())
        assert "preflight failed" in r["err"]
    assert torch.equal(torch.cat([r["grad"] for r in res], dim=1), full.grad)
    assert (lp.detach()[7:] == 0).all() and full.grad[:, V:].abs().sum() == 0
    z = logits.float()[:, :V] / 0.7
    want = torch.log_softmax(z, -1).gather(1, targets[:, None])[:, 0]
    assert (lp.detach()[:7] - want[:7]).abs().max() < 1e-5
    p = torch.softmax(z, -1)
    assert (res[0]["ent"] - (-(p * torch.log(p)).sum(-1))).abs().max() < 1e-4


# ---------------------------------------------------------------- CP attention: strict runtime + Megatron operator
HQ, HKV, D, B, S = 4, 2, 16, 2, 32


def _attn_inputs():
    g = torch.Generator().manual_seed(5)
    return (torch.randn(S, B, HQ, D, generator=g), torch.randn(S, B, HKV, D, generator=g), torch.randn(S, B, HKV, D, generator=g),
            torch.randn(S, B, HQ * D, generator=g))


def _mega_worker(rank, world, port, out):
    _init(rank, world, port)
    from rl_kernel_b200.integrations.engines.train.megatron.operators import (MegatronAttentionOperator,
                                                                               megatron_zigzag_positions)

    q, k, v, do = _attn_inputs()
    pos = megatron_zigzag_positions(S, world, rank)
    ql, kl, vl = (t[pos].clone().requires_grad_(True) for t in (q, k, v))
    op = MegatronAttentionOperator(cp_size=world, cp_rank=rank)          # no peer memory on the CPU: gather runtime
    o = op(None, ql, kl, vl)
    o.backward(do[pos])
    torch.save({"o": o.detach(), "dq": ql.grad, "dk": kl.grad, "dv": vl.grad, "pos": pos}, f"{out}.{rank}")
    dist.destroy_process_group()


def test_megatron_attention_operator_with_zigzag_cp_matches_single_rank(tmp_path):
    from rl_kernel_b200.integrations.engines.train.megatron.operators import MegatronAttentionOperator

    res = _spawn(_mega_worker, tmp_path)
    q, k, v, do = _attn_inputs()
    q1, k1, v1 = (t.clone().requires_grad_(True) for t in (q, k, v))
    o1 = MegatronAttentionOperator()(None, q1, k1, v1)
    o1.backward(do)
    for r in res:
        pos = r["pos"]
        assert (r["o"] - o1.detach()[pos]).abs().max() < 1e-5
        assert (r["dq"] - q1.grad[pos]).abs().max() < 1e-5
        assert (r["dk"] - k1.grad[pos]).abs().max() < 1e-4 and (r["dv"] - v1.grad[pos]).abs().max() < 1e-4


# ---------------------------------------------------------------- canonical CP weight gradients, SP FFN
def _canon_worker(rank, world, port, out):
    _init(rank, world, port)
    from rl_kernel_b200.distributed.algorithms import canonical_cp
    from rl_kernel_b200.distributed.algorithms.collectives import TorchDistributedDeterministicCollective
    from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn

    coll = TorchDistributedDeterministicCollective()
    g = torch.Generator().manual_seed(7)
    nseq, L, K, N = 2, 16, 24, 40
    x = torch.randn(nseq * L, K, generator=g).bfloat16()
    dy = torch.randn(nseq * L, N, generator=g).bfloat16()
    order = canonical_cp.uniform_gather_indices(nseq, L, world, "zigzag")
    # this rank's rows: sequence-major, zigzag positions ascending
    from rl_kernel_b200.distributed.cp_attention import cp_positions

    lpos = cp_positions(L, world, rank, "zigzag")
    mine = torch.cat([b * L + lpos for b in range(nseq)])
    layout = canonical_cp.CPLayout(order, mine.numel(), world, coll, cp_rank=rank)
    dw = canonical_cp.weight_gradient(x[mine], dy[mine], layout)
    lo, hi = layout.row_slice(N)
    total = coll.all_reduce(dw.clone())                 # what a framework's sum over the CP group produces
    ids = torch.randint(0, 11, (nseq * L,), generator=g)
    emb = torch.randn(11, 8, generator=g, requires_grad=True)
    e = canonical_cp.CPEmbedding.apply(ids[mine], emb, 0, layout)
    e.backward(torch.ones_like(e))
    # sequence-parallel FFN over the same two ranks, against the all-reduce form
    H, I = 64, 128
    xs = torch.randn(8, H, generator=g).bfloat16()
    wgu = (torch.randn(2 * I, H, generator=g) * 0.1).bfloat16()
    wd = (torch.randn(H, I, generator=g) * 0.1).bfloat16()
    il = I // world
    # engine layout: gate|up interleaved per canonical shard (8 shards of I/8 columns); rank r holds shards of its half
    blk = I // 8
    gate, up = wgu[:I].view(8, blk, H), wgu[I:].view(8, blk, H)
    packed = torch.stack([gate, up], 1).reshape(2 * I, H)
    w_gu_l = packed[rank * 2 * il:(rank + 1) * 2 * il].contiguous()
    wd_l = wd[:, rank * il:(rank + 1) * il].contiguous()
    y_tp = qwen3_ffn(xs, w_gu_l, wd_l, tp_size=world, collective=coll)
    rows = xs.shape[0] // world
    y_sp = qwen3_ffn(xs[rank * rows:(rank + 1) * rows], w_gu_l, wd_l, tp_size=world, collective=coll, sequence_parallel=True)
    torch.save({"dw": dw, "slice": (lo, hi), "total": total, "emb_grad": emb.grad, "y_tp": y_tp, "y_sp": y_sp,
                "packed": packed}, f"{out}.{rank}")
    dist.destroy_process_group()


def test_canonical_cp_gradients_are_row_sliced_and_sum_to_the_single_rank_gradient(tmp_path):
    from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn
    from rl_kernel_b200.ops.gemm.det_gemm import det_gemm_db
    from rl_kernel_b200.reference.embedding.embedding import embedding_grad_weight_reference

    res = _spawn(_canon_worker, tmp_path)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(32, 24, generator=g).bfloat16()
    dy = torch.randn(32, 40, generator=g).bfloat16()
    want = det_gemm_db(dy, x)                                   # single rank, logical token order
    for r, d in enumerate(res):
        lo, hi = d["slice"]
        assert torch.equal(d["dw"][lo:hi], want[lo:hi])         # its rows over ALL tokens, bit for bit
        rest = torch.ones(40, dtype=torch.bool)
        rest[lo:hi] = False
        assert d["dw"][rest].abs().sum() == 0                   # nothing else: no duplicated work, exact assembly
        assert torch.equal(d["total"], want)
    ids = torch.randint(0, 11, (32,), generator=g)
    emb = torch.randn(11, 8, generator=g)
    want_e = embedding_grad_weight_reference(ids, torch.ones(32, 8), 11)
    assert torch.equal(res[0]["emb_grad"], want_e) and res[1]["emb_grad"].abs().sum() == 0
    # SP == TP rows, and TP2 == the unsharded FFN bit for bit
    xs = torch.randn(8, 64, generator=g).bfloat16()
    wgu = (torch.randn(256, 64, generator=g) * 0.1).bfloat16()
    wd = (torch.randn(64, 128, generator=g) * 0.1).bfloat16()
    y1 = qwen3_ffn(xs, res[0]["packed"], wd)
    assert torch.equal(res[0]["y_tp"], y1) and torch.equal(res[1]["y_tp"], y1)
    assert torch.equal(torch.cat([res[0]["y_sp"], res[1]["y_sp"]]), y1)


# ---------------------------------------------------------------- partial-state CP merge (single process)
def test_cp_partial_states_merge_in_block_order_to_full_attention():
    from rl_kernel_b200.backends.cuda.attention.cp_comm import (AttentionCPBlockMetadata, AttentionCPCommunicationPlan,
                                                                AttentionCPPartialState, AttentionParallelSpec,
                                                                merge_attention_cp_partial_states,
                                                                sort_attention_cp_partial_states)

    torch.manual_seed(2)
    q, k, v = torch.randn(1, 2, 5, 8), torch.randn(1, 2, 12, 8), torch.randn(1, 2, 12, 8)
    par = AttentionParallelSpec(1, 0, 2, 0)
    blocks = (AttentionCPBlockMetadata(0, 0, 5, 0, 0), AttentionCPBlockMetadata(1, 5, 12, 1, 0))
    plan = AttentionCPCommunicationPlan(par, backend="p2p_nccl_reference", expected_blocks=blocks, expected_kv_token_range=(0, 12),
                                        query_token_ranges=((0, 3), (3, 5)))
    states = []
    for b in blocks:
        s = q @ k[:, :, b.kv_block_start:b.kv_block_end].transpose(-1, -2) / 8 ** 0.5
        lse = torch.logsumexp(s, -1)
        states.append(AttentionCPPartialState(torch.softmax(s, -1) @ v[:, :, b.kv_block_start:b.kv_block_end], lse, b))
    merged = merge_attention_cp_partial_states(states[::-1], plan=plan)          # arrival order does not matter
    s = q @ k.transpose(-1, -2) / 8 ** 0.5
    assert (merged.out - torch.softmax(s, -1) @ v).abs().max() < 1e-5 and (merged.lse - torch.logsumexp(s, -1)).abs().max() < 1e-5
    with pytest.raises(ValueError, match="manifest"):
        sort_attention_cp_partial_states(states[:1], plan=plan)
    with pytest.raises(ValueError):
        AttentionCPCommunicationPlan(par, backend="p2p_nccl_reference").validate()   # reference plans need a manifest
    prov = AttentionCPCommunicationPlan(par, backend="peer_memory").provenance()
    assert prov["cp_comm_redundant_compute_factor"] == 1 and prov["cp_comm_strict_kv_communication"] == "tma_peer_loads"


def _zero3_worker(rank, world, port, out):
    from rl_engine.integrations.engines.train.deepspeed.adapter import gather_zero3_parameter

    _init(rank, world, port)
    whole = torch.arange(10, dtype=torch.float32).view(2, 5)
    per = 6                                                  # 10 elements over 2 ranks, padded to 12
    flat = torch.cat([whole.reshape(-1), torch.zeros(2)])
    p = torch.nn.Parameter(torch.zeros(0))
    p.ds_tensor, p.ds_numel, p.ds_shape = flat[rank * per:(rank + 1) * per].clone(), 10, (2, 5)
    got = gather_zero3_parameter(p)
    if rank == 0:
        torch.save(bool(torch.equal(got, whole)), out)
    dist.barrier()
    dist.destroy_process_group()


def test_zero3_partitions_are_gathered_in_rank_order(tmp_path):
    out = str(tmp_path / "z3.pt")
    mp.spawn(_zero3_worker, args=(2, _port(), out), nprocs=2, join=True)
    assert torch.load(out)
