"""CPU plumbing of the model chain: a 2-layer Qwen3-style decoder in fp32 must give bitwise equal
selected-token log-probs for batch 1 vs batch 8, prefill vs decode, and TP 1 vs 2 (simulated and
over a Gloo process group)."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
from rl_kernel_b200.models.qwen3.reference import Qwen3DenseBIModel
from rl_kernel_b200.utils.bits import bit_equal

SPEC = Qwen3DenseSpec.scaled(layers=2, hidden=256, ffn=768, q_heads=4, kv_heads=2, head_dim=64, vocab=4096)


def _setup(seed=0):
    w = Qwen3DenseWeights.synthetic(SPEC, dtype=torch.float32, seed=seed)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, SPEC.vocab_size, (8, 24), generator=g)
    return w, ids


def test_batch_invariance_and_reference_accuracy():
    w, ids = _setup()
    model = Qwen3DenseBIModel(SPEC, w)
    full = model(ids, target_ids=ids)
    one = model(ids[3:4], target_ids=ids[3:4])
    assert bit_equal(full["selected_logp"][3:4], one["selected_logp"])
    gold = torch.log_softmax(full["logits"][:, :-1].double(), -1).gather(-1, ids[:, 1:, None])[..., 0]
    assert (full["selected_logp"].double() - gold).abs().max() < 1e-4


def test_prefill_equals_decode():
    w, ids = _setup()
    model = Qwen3DenseBIModel(SPEC, w)
    full = model(ids[:2], target_ids=ids[:2])["selected_logp"]
    cache = model.allocate_cache(2, 32)
    model(ids[:2, :10], kv_cache=cache)
    lps = []
    for t in range(10, 24):
        out = model.decode_step(ids[:2, t - 1] if False else ids[:2, t], torch.full((2,), t), cache,
                                return_logits=False)
        if t < 23:
            lps.append(model.selected_logprobs(out["hidden"].view(2, -1), ids[:2, t + 1]))
    dec = torch.stack(lps, dim=1)
    assert bit_equal(dec, full[:, 10:23])


def test_simulated_tp_invariance():
    w, ids = _setup()
    lp1 = Qwen3DenseBIModel(SPEC, w, tp_size=1)(ids[:2], target_ids=ids[:2])["selected_logp"]
    lp2 = Qwen3DenseBIModel(SPEC, w, tp_size=2)(ids[:2], target_ids=ids[:2])["selected_logp"]
    assert bit_equal(lp1, lp2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, out):
    import torch.distributed as dist

    from rl_kernel_b200.distributed import TorchDistributedDeterministicCollective

    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        w, ids = _setup()
        coll = TorchDistributedDeterministicCollective()
        model = Qwen3DenseBIModel(SPEC, w, tp_size=world, tp_rank=rank, collective=coll)
        lp = model(ids[:2], target_ids=ids[:2], return_logits=False)["selected_logp"]
        if rank == 0:
            torch.save(lp, out)
    finally:
        dist.destroy_process_group()


def test_gloo_tp2_matches_tp1(tmp_path):
    out = str(tmp_path / "lp.pt")
    mp.spawn(_tp_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    w, ids = _setup()
    torch.set_num_threads(1)
    lp1 = Qwen3DenseBIModel(SPEC, w)(ids[:2], target_ids=ids[:2], return_logits=False)["selected_logp"]
    assert bit_equal(torch.load(out), lp1)


def test_paged_kv_reference_equals_contiguous_scoring():
    from rl_kernel_b200.reference.attention import PagedKVReference, blockwise_attention_reference

    g = torch.Generator().manual_seed(4)
    hq, hkv, d, n = 4, 2, 16, 300
    k = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16)
    v = torch.randn(n, hkv, d, generator=g).to(torch.bfloat16)
    q = torch.randn(n, hq, d, generator=g).to(torch.bfloat16)
    cache = PagedKVReference(8, hkv, d)
    cache.append(7, k[:5], v[:5])          # another sequence takes pages first: tables interleave
    cache.append(3, k[:200], v[:200])
    cache.append(7, k[5:140], v[5:140])
    cache.append(3, k[200:], v[200:])
    pos = torch.arange(n)
    o_p, l_p = cache.score(3, q, pos)
    o_c, l_c = blockwise_attention_reference(q, k, v, pos, strict=False)
    assert torch.equal(o_p, o_c) and torch.equal(l_p, l_c)
    cache.release(7)
    assert len(cache.free) == 8 - 3
