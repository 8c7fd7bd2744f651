"""Multi-GPU tests at 2, 4 and 8 ranks (a size is skipped when the machine has fewer GPUs): fixed-order
collectives on symmetric memory, tensor- / context- / data-parallel bit invariance of the whole
GRPO step including the gradients, the fused compute + collective kernels, and a bounded wait that
runs out without hanging the GPU.  Each test owns its worker processes (NCCL bootstrap on
127.0.0.1); NVLS is off and the kernels use plain peer loads."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


WORLDS = (2, 4, 8)
CP_GRADS_CANONICAL = True       # every parameter gradient of a context-parallel run equals the single-GPU one bit for bit


def _need(world: int) -> None:
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, this machine has {torch.cuda.device_count()}")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port):
    import torch.distributed as dist

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    return dist


def _collective_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.distributed import balanced_tree_sum
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

    dev = torch.device("cuda", rank)
    coll = SymmetricMemoryCollective(None, dev, frame_bytes=64 << 20)
    ok = True
    for it, (n, dtype) in enumerate([(8, torch.bfloat16), (4096 * 64, torch.bfloat16), (1 << 22, torch.float32),
                                     (12288 * 1024, torch.bfloat16), (1000 * 8, torch.bfloat16)] * 4):
        g = torch.Generator(device="cuda").manual_seed(100 + it)
        parts = [torch.randn(n, device=dev, generator=g).to(dtype) for _ in range(world)]   # same on all ranks
        want = balanced_tree_sum(parts, dtype)
        got = coll.all_reduce(parts[rank])
        ok &= torch.equal(got, want)
        ag = coll.all_gather(parts[rank])
        ok &= all(torch.equal(ag[r], parts[r]) for r in range(world))
        if n % (8 * world) == 0:
            rs = coll.reduce_scatter(parts[rank])
            ok &= torch.equal(rs, want[rank * (n // world):(rank + 1) * (n // world)])
    # an all-gather whose per-rank share is larger than a frame goes in frame-sized pieces
    nbig = (64 << 20) // 2 + 8008
    bigs = [torch.randn(nbig, device=dev, generator=torch.Generator(device="cuda").manual_seed(900 + r)).to(torch.bfloat16)
            for r in range(world)]
    agb = coll.all_gather(bigs[rank])
    ok &= all(torch.equal(agb[r], bigs[r]) for r in range(world))
    del agb, bigs
    # negative cases of the protocol: each is refused on the host of EVERY rank before a kernel is launched, and the
    # group keeps working afterwards
    from rl_kernel_b200.distributed import CollectiveMismatchError

    big_a = torch.zeros(128, 64, device=dev, dtype=torch.bfloat16)
    try:                                                    # output larger than a frame (64 MiB here)
        coll.gemm_all_reduce(torch.zeros(16384, 64, device=dev, dtype=torch.bfloat16),
                             torch.zeros(4096, 64, device=dev, dtype=torch.bfloat16),
                             torch.empty(16384, 4096, device=dev, dtype=torch.bfloat16), 1)
        ok = False
    except ext.NativeLibraryError as exc:
        ok &= "frame capacity" in str(exc)
    try:                                                    # rows that do not split into whole tiles per rank
        coll.gemm_reduce_scatter(big_a, big_a, torch.empty(128 // world, 128, device=dev, dtype=torch.bfloat16), 1)
        ok = False
    except ext.NativeLibraryError as exc:
        ok &= "multiple of 128 x world" in str(exc)
    coll.verify_signatures = True
    try:                                                    # ranks disagree on the size of an all-reduce
        coll.all_reduce(torch.ones(1024 * (1 + rank), device=dev))
        ok = False
    except CollectiveMismatchError:
        pass
    ok &= bool(torch.equal(coll.all_reduce(torch.ones(1024, device=dev)), torch.full((1024,), float(world), device=dev)))
    coll.verify_signatures = False
    ok &= ext.poll_status(dev) == 0
    # staged all-reduce: the producer writes straight into the symmetric frame
    x = torch.full((256, 128), float(rank + 1), device=dev, dtype=torch.bfloat16)
    st = coll.staging_view(x.shape, x.dtype)
    st.copy_(x)
    res = coll.all_reduce_staged(st, torch.empty_like(x))
    ok &= bool((res == float(sum(range(1, world + 1)))).all())
    # fused GEMM + all-reduce == local GEMM followed by the tree all-reduce, bit for bit
    from rl_kernel_b200.backends import native as nv

    # (the last three have enough tiles for the 128 x 256 form of the fused kernel: chunked, plain, ragged edges)
    for (M, N, K, nch) in [(700, 512, 1024, 4), (1536, 1024, 512, 1), (128, 256, 512, 8), (12288, 1024, 3072, 4),
                           (10000, 512, 256, 1), (9999 // 8 * 8, 1000, 1536, 2)]:
        g = torch.Generator(device="cuda").manual_seed(7 + rank)
        a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        b = torch.randn(N, K, device=dev, generator=g).to(torch.bfloat16)
        part = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        nv.det_gemm(a, b, part, M=M, N=N, K=K, nchunks=nch, tile_n=128)
        want = coll.all_reduce(part)
        got = coll.gemm_all_reduce(a, b, torch.empty_like(part), nch)
        ok &= torch.equal(got, want)
    # CUDA graph replay keeps the sequence numbers moving
    buf = torch.ones(4096, device=dev, dtype=torch.float32)
    s = torch.cuda.Stream(dev)
    s.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(s):
        coll.all_reduce_(buf)
    torch.cuda.current_stream(dev).wait_stream(s)
    buf.fill_(1.0)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph), coll.graph_capture():
        coll.all_reduce_(buf)
    coll.graph_commit()
    for _ in range(5):
        graph.replay()
    coll.graph_replayed(5)
    torch.cuda.synchronize(dev)
    ok &= bool((buf == float(world) ** 5).all())
    ok &= bool(torch.equal(coll.all_reduce(torch.ones(8, device=dev)), torch.full((8,), float(world), device=dev)))
    ok &= ext.poll_status(dev) == 0
    coll.close()
    res = [None] * world
    dist.all_gather_object(res, bool(ok))
    if rank == 0:
        torch.save(all(res), out)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_symmetric_collectives(tmp_path, world):
    _need(world)
    out = str(tmp_path / "ok.pt")
    mp.spawn(_collective_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert torch.load(out)


def _timeout_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    from rl_kernel_b200.distributed import CollectiveTimeout
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

    dev = torch.device("cuda", rank)
    coll = SymmetricMemoryCollective(None, dev, frame_bytes=1 << 20)
    x = torch.ones(1024, device=dev)
    coll.all_reduce_(x)
    raised = False
    if rank == 0:
        coll.all_reduce_(x)          # rank 1 never joins this one: the device wait must give up
        try:
            coll.raise_on_timeout()
        except CollectiveTimeout:
            raised = True
    dist.barrier()                   # rank 1 learns on the host that the step is over
    coll.resync()
    y = torch.ones(1024, device=dev)
    coll.all_reduce_(y)              # the context is still usable on both ranks
    torch.cuda.synchronize(dev)
    fine = bool((y == float(world)).all())
    coll.close()
    if rank == 0:
        torch.save((raised, fine), out)
    dist.destroy_process_group()


def test_bounded_wait_reports_instead_of_hanging(tmp_path):
    out = str(tmp_path / "t.pt")
    mp.spawn(_timeout_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    raised, fine = torch.load(out)
    assert raised, "a missing peer must surface as CollectiveTimeout"
    assert fine, "collectives must work again after resync"


def _tp_spec():
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec

    # 8 KV heads and a feed-forward width of 8 x 256 so that 2, 4 and 8 tensor-parallel ranks all divide it
    return Qwen3DenseSpec.scaled(layers=2, hidden=1024, ffn=2048, q_heads=16, kv_heads=8, head_dim=128, vocab=4096)


def _tp_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.models.qwen3 import Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer
    from rl_kernel_b200.models.qwen3.parallel_setup import build_parallel_context

    dev = torch.device("cuda", rank)
    spec = _tp_spec()
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    ctx = build_parallel_context(world, 1, dev)
    cfg = GRPOConfig(num_prompts=2, group_size=2, prompt_len=128, response_len=48, micro_batch_seqs=2, lr=1e-4)
    tr = GRPOTrainer(spec, cfg, dev, ctx=ctx, weights=w)
    prompts = torch.randint(0, spec.vocab_size, (2, 128), generator=torch.Generator().manual_seed(5)).to(dev)
    res = tr.step(prompts, step_index=0)
    torch.cuda.synchronize(dev)
    mine = {k: res[k].cpu() for k in ("tokens", "old_logp", "train_logp", "grad_norm")}
    mine["grads"] = {k: v.cpu() for k, v in tr.policy.g.items()}
    mine["weights"] = {k: v.cpu() for k, v in tr.policy.w.items()}
    mine["status"] = ext.poll_status(dev)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        torch.save(gathered, out)
    dist.barrier()
    dist.destroy_process_group()


def _assemble(shards: list[dict], name: str) -> torch.Tensor:
    """The full tensor of parameter ``name`` from the tensor-parallel shards (PackedParams layout)."""
    parts = [s[name] for s in shards]
    if parts[0].dim() == 1:
        for p in parts[1:]:
            assert torch.equal(p, parts[0]), f"replicated {name} differs between ranks"
        return parts[0]
    if name.endswith((".wo", ".wd")):
        return torch.cat(parts, dim=1)
    return torch.cat(parts, dim=0)


@pytest.mark.parametrize("world", WORLDS)
def test_tensor_parallel_step_matches_single_gpu_bitwise(tmp_path, world):
    """One whole GRPO step (rollout, training forward / backward, clipping, AdamW) on 2, 4 or 8
    tensor-parallel ranks: sampled tokens, rollout and training log-probs, EVERY gradient, the
    gradient norm and the updated weights equal the single-GPU run bit for bit."""
    _need(world)
    from rl_kernel_b200.models.qwen3 import Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    out = str(tmp_path / "tp.pt")
    mp.spawn(_tp_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    tp = torch.load(out)
    dev = torch.device("cuda:0")
    spec = _tp_spec()
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    cfg = GRPOConfig(num_prompts=2, group_size=2, prompt_len=128, response_len=48, micro_batch_seqs=2, lr=1e-4)
    tr = GRPOTrainer(spec, cfg, dev, weights=w)
    prompts = torch.randint(0, spec.vocab_size, (2, 128), generator=torch.Generator().manual_seed(5)).to(dev)
    one = tr.step(prompts, step_index=0)
    torch.cuda.synchronize(dev)
    assert all(r["status"] == 0 for r in tp)
    for r in tp:
        assert torch.equal(r["tokens"], one["tokens"].cpu())
        assert torch.equal(r["old_logp"], one["old_logp"].cpu())
        assert torch.equal(r["train_logp"], one["train_logp"].cpu())
        assert torch.equal(r["train_logp"], r["old_logp"])
        assert torch.equal(r["grad_norm"], one["grad_norm"].cpu())
    for name in tr.policy.g:
        assert torch.equal(_assemble([r["grads"] for r in tp], name), tr.policy.g[name].cpu()), f"gradient of {name}"
        assert torch.equal(_assemble([r["weights"] for r in tp], name), tr.policy.w[name].cpu()), f"updated {name}"


def _cp_spec(world):
    """The LM head is split over the context-parallel ranks by canonical chunk, so the model needs at least
    ``world`` canonical shards (one per KV head here); four query heads per KV head as in Qwen3-8B."""
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec

    kv = max(2, world)
    return Qwen3DenseSpec.scaled(layers=2, hidden=1024, ffn=2048, q_heads=4 * kv, kv_heads=kv, head_dim=128, vocab=4096)


def _cp_cfg(world):
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig

    # zigzag shards need a sequence length that is a multiple of 2 x cp x 128
    return GRPOConfig(num_prompts=world, group_size=2, prompt_len=128, response_len=256 * world - 128,
                      micro_batch_seqs=2 * world, lr=1e-4)


def _cp_train_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOTrainer
    from rl_kernel_b200.models.qwen3.parallel_setup import build_parallel_context

    dev = torch.device("cuda", rank)
    spec = _cp_spec(world)
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    ctx = build_parallel_context(1, world, dev)
    cfg = _cp_cfg(world)
    tr = GRPOTrainer(spec, cfg, dev, ctx=ctx, weights=w)
    prompts = torch.randint(0, spec.vocab_size, (world, 128), generator=torch.Generator().manual_seed(5)).to(dev)
    res = tr.step(tr.local_prompts(prompts), step_index=0)
    torch.cuda.synchronize(dev)
    mine = {k: res[k].cpu() for k in ("tokens", "old_logp", "train_logp", "grad_norm")}
    mine["grads"] = {k: v.cpu() for k, v in tr.policy.g.items()}
    mine["status"] = ext.poll_status(dev)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        torch.save(gathered, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_context_parallel_training_matches_single_gpu(tmp_path, world):
    """Rollout on `world` independent engines + training with every sequence split over the GPUs
    gives the tokens and log-probs of one GPU bit for bit, and with canonical gradients (the
    default) every parameter gradient and the gradient norm as well."""
    _need(world)
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOTrainer

    out = str(tmp_path / "cp.pt")
    mp.spawn(_cp_train_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    cp = torch.load(out)
    dev = torch.device("cuda:0")
    spec = _cp_spec(world)
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    cfg = _cp_cfg(world)
    tr = GRPOTrainer(spec, cfg, dev, weights=w)
    prompts = torch.randint(0, spec.vocab_size, (world, 128), generator=torch.Generator().manual_seed(5)).to(dev)
    one = tr.step(prompts, step_index=0)
    torch.cuda.synchronize(dev)
    assert all(r["status"] == 0 for r in cp)
    for r in cp:
        assert torch.equal(r["tokens"], one["tokens"].cpu())
        assert torch.equal(r["old_logp"], one["old_logp"].cpu())
        assert torch.equal(r["train_logp"], one["train_logp"].cpu())
        assert torch.equal(r["train_logp"], r["old_logp"])
    if tr.engine.canonical_grads and CP_GRADS_CANONICAL:
        for r in cp:
            for name, g in tr.policy.g.items():
                assert torch.equal(r["grads"][name], g.cpu()), f"gradient of {name}"
            assert torch.equal(r["grad_norm"], one["grad_norm"].cpu())
    else:
        assert abs(float(cp[0]["grad_norm"]) - float(one["grad_norm"])) <= 2e-2 * float(one["grad_norm"])


def _cp_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    import math

    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.distributed.cp_attention import CPAttention, cp_positions
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective
    from rl_kernel_b200.models.qwen3.engine import train_tiles

    dev = torch.device("cuda", rank)
    coll = SymmetricMemoryCollective(None, dev, frame_bytes=1 << 20)
    HQ, HKV, D, B, S = 8, 2, 128, 2, 256 * world
    g = torch.Generator(device="cuda").manual_seed(3)            # same full tensors on every rank
    q = torch.randn(B, S, HQ * D, device=dev, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, HKV * D, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, HKV * D, device=dev, generator=g).to(torch.bfloat16)
    # single-GPU result
    o1 = torch.empty(B * S, HQ * D, device=dev, dtype=torch.bfloat16)
    l1 = torch.empty(B * S, HQ, device=dev)
    tiles, kvtiles = train_tiles(B, S, HQ, HKV, D, dev)
    sc = 1 / math.sqrt(D)
    q2, k2, v2 = q.view(B * S, -1), k.view(B * S, -1), v.view(B * S, -1)
    nv.attn_fwd(q2, [k2], [v2], o1, l1, tiles, sc)
    do = torch.randn(B, S, HQ * D, device=dev, generator=g).to(torch.bfloat16)
    do2 = do.view(B * S, -1)
    dl1 = torch.empty(B * S, HQ, device=dev)
    nv.attn_bwd_delta(o1, do2, dl1, B * S, HQ)
    dq1, dk1, dv1 = torch.empty_like(q2), torch.empty_like(k2), torch.empty_like(v2)
    nv.attn_bwd_dq(q2, do2, k2, v2, l1, dl1, dq1, tiles, sc)
    nv.attn_bwd_dkv(q2, do2, k2, v2, l1, dl1, dk1, dv1, kvtiles, sc)
    ok = True
    for layout in ("contiguous", "zigzag"):
        pos = cp_positions(S, world, rank, layout).to(dev)
        cp = CPAttention(coll, dev, num_q_heads=HQ, num_kv_heads=HKV, max_local_tokens=B * S // world, layout=layout)
        sel = lambda t: t[:, pos].reshape(B * pos.numel(), -1).contiguous()
        o, l = cp.forward(sel(q), sel(k), sel(v), B, S)
        ok &= torch.equal(o, sel(o1.view(B, S, -1)))
        ok &= torch.equal(l, sel(l1.view(B, S, -1)))
        dq, dk, dv = cp.backward(sel(q), sel(k), sel(v), o, l, sel(do), B, S)
        ok &= torch.equal(dq, sel(dq1.view(B, S, -1)))
        ok &= torch.equal(dk, sel(dk1.view(B, S, -1)))
        ok &= torch.equal(dv, sel(dv1.view(B, S, -1)))
    torch.cuda.synchronize(dev)
    from rl_kernel_b200.backends import extension as ext
    ok &= ext.poll_status(dev) == 0
    res = [None] * world
    dist.all_gather_object(res, bool(ok))
    if rank == 0:
        torch.save(all(res), out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_cp_attention_fwd_bwd_equals_single_gpu_bitwise(tmp_path, world):
    _need(world)
    out = str(tmp_path / "cp.pt")
    mp.spawn(_cp_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert torch.load(out)


def _push_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    import ctypes

    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.distributed.transports.symm import _DevicePtrView
    from rl_kernel_b200.integrations.common.weights import NVLinkPushBridge
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.engine import PackedParams

    dev = torch.device("cuda", rank)
    lib = ext.load()
    spec = Qwen3DenseSpec.scaled(layers=2, hidden=256, ffn=512, q_heads=16, kv_heads=8, head_dim=128, vocab=1024)
    w = Qwen3DenseWeights.synthetic(spec, seed=9)
    # destination: one tensor-parallel rollout shard per rank, living in exportable memory
    dst_layout = PackedParams(spec, rank, world, dev)
    nbytes = dst_layout.numel * 2 + 256
    h = ctypes.create_string_buffer(lib.rlk_symm_ipc_handle_bytes())
    p = ctypes.c_void_p(0)
    ext.check(lib.rlk_ipc_alloc(ctypes.c_longlong(nbytes), ctypes.byref(p), h), "ipc_alloc")
    handles = [None] * world
    dist.all_gather_object(handles, bytes(h.raw))
    mine = torch.as_tensor(_DevicePtrView(p.value, nbytes), device=dev)
    ok = True
    if rank == 0:
        # source: the TP1 trainer shard on rank 0 pushes to every rollout shard (its own and the peers')
        src = PackedParams(spec, 0, 1, dev).load(w)
        bridge = NVLinkPushBridge(src, dev)
        bases = [p.value]
        for r in range(1, world):
            peer = ctypes.c_void_p(0)
            ext.check(lib.rlk_ipc_open(handles[r], ctypes.byref(peer)), "ipc_open")
            bases.append(peer.value)
        for r in range(world):
            bridge.add_target(PackedParams(spec, r, world, torch.device("cpu")), base_ptr=bases[r],
                              version_flag_ptr=bases[r] + dst_layout.numel * 2)
        m = bridge.publish(7)
        ok &= m.metadata["rl_kernel_bridge"]["targets"] == world and m.metadata["layout"]["kind"] == "tp-canonical"
    flag = mine[dst_layout.numel * 2: dst_layout.numel * 2 + 8].view(torch.int64)
    okd = torch.zeros(1, dtype=torch.int32, device=dev)
    ext.check(lib.rlk_version_wait(ext.ptr(flag), ctypes.c_ulonglong(7), ext.ptr(okd), ext.stream_ptr(dev)), "wait")
    torch.cuda.synchronize(dev)
    ok &= int(okd.item()) == 1
    want = PackedParams(spec, rank, world, dev).load(w)
    ok &= torch.equal(mine[: dst_layout.numel * 2].view(torch.bfloat16), want.flat)
    res = [None] * world
    dist.all_gather_object(res, bool(ok))
    if rank == 0:
        torch.save(all(res), out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_weight_push_reshards_over_nvlink(tmp_path, world):
    _need(world)
    out = str(tmp_path / "push.pt")
    mp.spawn(_push_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert torch.load(out)


def _moe_case(dev, ep_rank, ep_size, coll):
    from rl_kernel_b200.models.qwen3_moe import MoEPackedParams, Qwen3MoeEngine, Qwen3MoeSpec

    spec = Qwen3MoeSpec.tiny()
    B, S, P = 8, 256, 64
    tokens = torch.randint(0, spec.vocab_size, (B, S), generator=torch.Generator().manual_seed(9)).to(dev)
    per = B // ep_size
    mine = tokens[ep_rank * per:(ep_rank + 1) * per].contiguous()
    params = MoEPackedParams(spec, ep_rank, ep_size, dev, with_grad=True).init_synthetic_(3, std=0.05)
    eng = Qwen3MoeEngine(spec, params, ep_collective=coll, max_tokens=per * S, max_positions=S + 8)
    logp = eng.train_forward_backward(mine, P, lambda x: torch.full_like(x, -1.0 / (B * (S - P))))
    eng.sync_replicated_grads()
    torch.cuda.synchronize(dev)
    return spec, params, logp


def _moe_ep_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

    dev = torch.device("cuda", rank)
    coll = SymmetricMemoryCollective(None, dev, frame_bytes=64 << 20)
    spec, params, logp = _moe_case(dev, rank, world, coll)
    res = {"logp": logp.cpu(), "w1": params.g["l0.w1"].cpu(), "w2": params.g["l1.w2"].cpu(),
           "router": params.g["l0.router"].cpu(), "wqkv": params.g["l1.wqkv"].cpu(), "status": ext.poll_status(dev)}
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        torch.save(gathered, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_moe_expert_parallel_matches_single_gpu(tmp_path, world):
    """2, 4 or 8 expert-parallel ranks (tokens and experts both split, dispatch / combine over NVLink)
    reproduce one GPU: log-probs and expert weight gradients bit for bit, replicated-parameter
    gradients to rounding (they are summed over the ranks instead of over one long token axis)."""
    _need(world)
    out = str(tmp_path / "moe.pt")
    mp.spawn(_moe_ep_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    ep = torch.load(out)
    spec, params, logp = _moe_case(torch.device("cuda:0"), 0, 1, None)
    assert all(r["status"] == 0 for r in ep)
    assert torch.equal(torch.cat([r["logp"] for r in ep]), logp.cpu())
    assert torch.equal(torch.cat([r["w1"] for r in ep]), params.g["l0.w1"].cpu())
    assert torch.equal(torch.cat([r["w2"] for r in ep]), params.g["l1.w2"].cpu())
    for name, key in (("router", "l0.router"), ("wqkv", "l1.wqkv")):
        a, b = ep[0][name].float(), params.g[key].float().cpu()
        assert all(torch.equal(ep[0][name], r[name]) for r in ep), "replicated gradients must agree across ranks"
        assert (a - b).abs().max().item() <= 0.05 * b.abs().max().item() + 1e-6, name


def _ag_gemm_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.distributed.ag_gemm import AllGatherGemm
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective

    dev = torch.device("cuda", rank)
    coll = SymmetricMemoryCollective(None, dev, frame_bytes=1 << 20)
    M, K, N = 1024, 1024, 640
    g = torch.Generator(device="cuda").manual_seed(7)             # same full matrices on every rank
    a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device=dev, generator=g).to(torch.bfloat16)
    ag = AllGatherGemm(coll, dev, M, K)
    rows = M // world
    ok = True
    for rep in range(3):                                          # buffers and counters are reusable
        a2 = (a.float() * (rep + 1)).to(torch.bfloat16)
        ag.local_shard.copy_(a2[rank * rows:(rank + 1) * rows])
        c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        ag(w, c)
        ref = torch.empty_like(c)
        nv.det_gemm(a2, w, ref, M=M, N=N, K=K)
        torch.cuda.synchronize(dev)
        ok &= torch.equal(c, ref) and torch.equal(ag.gathered, a2)
    ok &= ext.poll_status(dev) == 0
    res = [None] * world
    dist.all_gather_object(res, bool(ok))
    if rank == 0:
        torch.save(all(res), out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_all_gather_gemm_equals_gemm_of_gathered_matrix(tmp_path, world):
    _need(world)
    out = str(tmp_path / "ag.pt")
    mp.spawn(_ag_gemm_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert torch.load(out)


def _pcp_worker(rank, world, port, out):
    """Page pool spread over the GPUs (block b of every sequence lives on rank b % world); each rank
    computes a disjoint slice of the query rows and reads the other rank's pages over NVLink."""
    dist = _init(rank, world, port)
    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.distributed.cp_attention import PeerMappedBuffers
    from rl_kernel_b200.ops.attention import PagedKVCache, causal_attention, paged_attention

    dev = torch.device("cuda", rank)
    hq, hkv, d, n, pages = 8, 2, 128, 700, 8
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(n, hq, d, device=dev, generator=g).to(torch.bfloat16)
    k = torch.randn(n, hkv, d, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(n, hkv, d, device=dev, generator=g).to(torch.bfloat16)
    pm = PeerMappedBuffers(None, dev, {"k": ((pages * 128, hkv * d), torch.bfloat16),
                                       "v": ((pages * 128, hkv * d), torch.bfloat16)})
    cache = PagedKVCache(pages, hkv, d, dev, rank=rank, k_pool=pm.local("k"), v_pool=pm.local("v"))
    cache.reserve(0, n, owner_of_block=lambda b: b % world)
    mine = [b for b in range((n + 127) // 128) if b % world == rank]
    for b in mine:                                       # fill the blocks this rank owns
        lo, hi = b * 128, min(n, b * 128 + 128)
        cache.write(0, torch.arange(lo, hi), k[lo:hi].reshape(hi - lo, -1), v[lo:hi].reshape(hi - lo, -1))
    tables = [None] * world
    dist.all_gather_object(tables, cache.tables[0])
    for b in range(len(cache.tables[0])):                # learn where the other ranks put their blocks
        owner = b % world
        if owner != rank:
            cache.set_remote_page(0, b, owner, tables[owner][b] & 0xFFFFFF)
    torch.cuda.synchronize(dev)
    dist.barrier()
    per = (n + world - 1) // world
    lo, hi = rank * per, min(n, (rank + 1) * per)        # disjoint query slices
    o = paged_attention(q[lo:hi].contiguous(), cache, [0], [torch.arange(lo, hi)], peer_pools=(pm["k"], pm["v"]))
    ref = causal_attention(q, k, v, [0, n])
    torch.cuda.synchronize(dev)
    ok = torch.equal(o, ref[lo:hi]) and ext.poll_status(dev) == 0
    dist.barrier()                                       # nobody frees pages a peer still reads
    res = [None] * world
    dist.all_gather_object(res, bool(ok))
    if rank == 0:
        torch.save(all(res), out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", (2, 4))
def test_paged_context_parallel_reads_remote_pages(tmp_path, world):
    _need(world)
    out = str(tmp_path / "pcp.pt")
    mp.spawn(_pcp_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert torch.load(out)


def _pp_setup(dev, layers, has_embed, has_head):
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.engine import PackedParams, Qwen3Engine

    spec = Qwen3DenseSpec.scaled(layers=4, hidden=1024, ffn=2048, q_heads=8, kv_heads=2, head_dim=128, vocab=4096)
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    params = PackedParams(spec, 0, 1, dev, with_grad=True, layers=layers, has_embed=has_embed, has_head=has_head).load(w)
    eng = Qwen3Engine(spec, params, max_positions=512)
    micro = [torch.randint(0, spec.vocab_size, (2, 256), generator=torch.Generator().manual_seed(20 + i)).to(dev)
             for i in range(4)]
    return spec, params, eng, micro


def _pp_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    from rl_kernel_b200.parallel.pipeline import PipelineTrainer, StageLink, split_layers

    dev = torch.device("cuda", rank)
    ranges = split_layers(4, world)
    spec, params, eng, micro = _pp_setup(dev, ranges[rank], rank == 0, rank == world - 1)
    trainer = PipelineTrainer(eng, StageLink(rank, world, dev))
    logps = trainer.run(micro, 64, lambda lp, i: torch.full_like(lp, -1.0 / lp.numel()))
    torch.cuda.synchronize(dev)
    res = {"logp": [l.cpu() for l in logps], "grads": {k: v.cpu() for k, v in params.g.items()}}
    gathered = [None] * world
    dist.all_gather_object(gathered, res)
    if rank == 0:
        torch.save(gathered, out)
    dist.barrier()
    dist.destroy_process_group()


def test_pipeline_two_stages_match_single_gpu_bitwise(tmp_path):
    """1F1B over two stages (NCCL p2p between them) gives the log-probs and every gradient of the
    unsplit model bit for bit."""
    out = str(tmp_path / "pp.pt")
    mp.spawn(_pp_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    pp = torch.load(out)
    dev = torch.device("cuda:0")
    spec, params, eng, micro = _pp_setup(dev, None, True, True)
    ref = [eng.train_forward_backward(t, 64, lambda lp: torch.full_like(lp, -1.0 / lp.numel())).clone() for t in micro]
    torch.cuda.synchronize(dev)
    assert len(pp[1]["logp"]) == 4 and pp[0]["logp"] == []
    for a, b in zip(pp[1]["logp"], ref):
        assert torch.equal(a, b.cpu())
    seen = set()
    for stage in pp:
        for name, g in stage["grads"].items():
            assert torch.equal(g, params.g[name].cpu()), name
            seen.add(name)
    assert seen == set(params.g)


def _dp_worker(rank, world, port, out):
    dist = _init(rank, world, port)
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer
    from rl_kernel_b200.models.qwen3.parallel_setup import build_parallel_context

    dev = torch.device("cuda", rank)
    spec = Qwen3DenseSpec.scaled(layers=2, hidden=1024, ffn=2048, q_heads=8, kv_heads=2, head_dim=128, vocab=4096)
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    ctx = build_parallel_context(1, 1, dev, dp=world)
    cfg = GRPOConfig(num_prompts=world, group_size=2, prompt_len=128, response_len=48, micro_batch_seqs=2, lr=1e-4)
    tr = GRPOTrainer(spec, cfg, dev, ctx=ctx, weights=w)
    prompts = torch.randint(0, spec.vocab_size, (world, 128), generator=torch.Generator().manual_seed(5)).to(dev)
    res = tr.step(tr.local_prompts(prompts), step_index=0)
    torch.cuda.synchronize(dev)
    mine = {k: res[k].cpu() for k in ("tokens", "old_logp", "train_logp", "grad_norm", "rewards")}
    mine["w"] = tr.policy.w["l1.wqkv"].cpu()
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        torch.save(gathered, out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_data_parallel_replicas_match_single_gpu(tmp_path, world):
    """2, 4 or 8 whole-model replicas, each rolling out and training its own prompts: sequences and
    log-probs equal the single-GPU run bit for bit, the summed gradient agrees to rounding (the
    replicas' sums meet in a fixed tree instead of one running sum) and all replicas end the step
    with identical weights."""
    _need(world)
    from rl_kernel_b200.models.qwen3 import Qwen3DenseSpec, Qwen3DenseWeights
    from rl_kernel_b200.models.qwen3.grpo import GRPOConfig, GRPOTrainer

    out = str(tmp_path / "dp.pt")
    mp.spawn(_dp_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    dp = torch.load(out)
    dev = torch.device("cuda:0")
    spec = Qwen3DenseSpec.scaled(layers=2, hidden=1024, ffn=2048, q_heads=8, kv_heads=2, head_dim=128, vocab=4096)
    w = Qwen3DenseWeights.synthetic(spec, seed=3)
    cfg = GRPOConfig(num_prompts=world, group_size=2, prompt_len=128, response_len=48, micro_batch_seqs=2, lr=1e-4)
    tr = GRPOTrainer(spec, cfg, dev, weights=w)
    prompts = torch.randint(0, spec.vocab_size, (world, 128), generator=torch.Generator().manual_seed(5)).to(dev)
    one = tr.step(prompts, step_index=0)
    for key in ("tokens", "old_logp", "train_logp", "rewards"):
        assert torch.equal(torch.cat([r[key] for r in dp]), one[key].cpu()), key
    assert torch.equal(dp[0]["train_logp"], dp[0]["old_logp"])
    assert all(torch.equal(dp[0]["w"], r["w"]) for r in dp)
    assert all(torch.equal(dp[0]["grad_norm"], r["grad_norm"]) for r in dp)
    assert abs(float(dp[0]["grad_norm"]) - float(one["grad_norm"])) <= 2e-2 * float(one["grad_norm"])


def _fused_ops_worker(rank, world, port, out):
    """The registry's native vocabulary-parallel log-prob and context-parallel attention operators
    against single-GPU results, forward and backward."""
    dist = _init(rank, world, port)
    import math

    from rl_kernel_b200.backends import extension as ext
    from rl_kernel_b200.backends import native as nv
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective
    from rl_kernel_b200.models.qwen3.engine import train_tiles
    from rl_kernel_b200.ops.logprob import linear_logp
    from rl_kernel_b200.runtime.registry import OpBackend, kernel_registry

    dev = torch.device("cuda", rank)
    coll = SymmetricMemoryCollective(None, dev, frame_bytes=64 << 20)
    ok = True
    # ---- vocabulary-parallel fused linear log-prob
    N, H, V, VP = 300, 512, 3900, 4096
    g = torch.Generator(device="cuda").manual_seed(21)                # same tensors on every rank
    hidden = torch.randn(N, H, device=dev, generator=g).bfloat16()
    w_full = torch.zeros(VP, H, device=dev, dtype=torch.bfloat16)
    w_full[:V] = (torch.randn(V, H, device=dev, generator=g) * 0.05).bfloat16()
    targets = torch.randint(0, V, (N,), device=dev, generator=g)
    gout = torch.randn(N, device=dev, generator=g)
    op = kernel_registry.get_op("vocab_parallel_logp", real_vocab=V, padded_vocab=VP, collective=coll, temperature=0.7)
    ok &= kernel_registry.last_resolution.actual is OpBackend.B200_VOCAB_PARALLEL_LOGP
    per = VP // world
    h1 = hidden.clone().requires_grad_(True)
    ws = w_full[rank * per:(rank + 1) * per].clone().requires_grad_(True)
    lp = op(h1, ws, targets)
    lp.backward(gout)
    one = kernel_registry.get_op("vocab_parallel_logp", real_vocab=V, padded_vocab=VP, collective=None, temperature=0.7)
    h2 = hidden.clone().requires_grad_(True)
    wf = w_full.clone().requires_grad_(True)
    lp1 = one(h2, wf, targets)
    lp1.backward(gout)
    torch.cuda.synchronize(dev)
    ok &= torch.equal(lp, lp1) and torch.equal(h1.grad, h2.grad) and torch.equal(ws.grad, wf.grad[rank * per:(rank + 1) * per])
    ref = linear_logp(hidden, w_full[:V].contiguous(), targets, 0.7)       # the unsharded fused operator
    ok &= torch.equal(lp.detach(), ref)
    # ---- context-parallel attention through the registry
    HQ, HKV, D, B, S = 8, 2, 128, 2, 256 * world
    q = torch.randn(B, S, HQ * D, device=dev, generator=g).bfloat16()
    k = torch.randn(B, S, HKV * D, device=dev, generator=g).bfloat16()
    v = torch.randn(B, S, HKV * D, device=dev, generator=g).bfloat16()
    do = torch.randn(B, S, HQ * D, device=dev, generator=g).bfloat16()
    cp = kernel_registry.get_attention_op("cp", collective=coll, device=dev, num_q_heads=HQ, num_kv_heads=HKV,
                                          max_local_tokens=B * S // world, layout="zigzag")
    ok &= kernel_registry.last_resolution.actual is OpBackend.B200_CP_ATTENTION
    pos = cp.local_positions(S).to(dev)
    sel = lambda t: t[:, pos].reshape(B * pos.numel(), -1).contiguous()
    ql, kl, vl = (sel(t).requires_grad_(True) for t in (q, k, v))
    o, lse = cp(ql, kl, vl, nseq=B, seq_len=S)
    o.backward(sel(do))
    o1 = torch.empty(B * S, HQ * D, device=dev, dtype=torch.bfloat16)
    l1 = torch.empty(B * S, HQ, device=dev)
    tiles, kvtiles = train_tiles(B, S, HQ, HKV, D, dev)
    sc = 1 / math.sqrt(D)
    q2, k2, v2, do2 = (t.view(B * S, -1) for t in (q, k, v, do))
    nv.attn_fwd(q2, [k2], [v2], o1, l1, tiles, sc)
    dl = torch.empty(B * S, HQ, device=dev)
    nv.attn_bwd_delta(o1, do2, dl, B * S, HQ)
    dq1, dk1, dv1 = torch.empty_like(q2), torch.empty_like(k2), torch.empty_like(v2)
    nv.attn_bwd_dq(q2, do2, k2, v2, l1, dl, dq1, tiles, sc)
    nv.attn_bwd_dkv(q2, do2, k2, v2, l1, dl, dk1, dv1, kvtiles, sc)
    torch.cuda.synchronize(dev)
    ok &= torch.equal(o.detach(), sel(o1.view(B, S, -1))) and torch.equal(lse, sel(l1.view(B, S, -1)))
    ok &= torch.equal(ql.grad, sel(dq1.view(B, S, -1))) and torch.equal(kl.grad, sel(dk1.view(B, S, -1)))
    ok &= torch.equal(vl.grad, sel(dv1.view(B, S, -1)))
    ok &= ext.poll_status(dev) == 0
    res = [None] * world
    dist.all_gather_object(res, bool(ok))
    if rank == 0:
        torch.save(all(res), out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_registry_native_multi_gpu_operators_match_single_gpu_bitwise(tmp_path, world):
    _need(world)
    out = str(tmp_path / "ops.pt")
    mp.spawn(_fused_ops_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert torch.load(out)


def _gemm_rs_worker(rank, world, port, out):
    """Fused GEMM + reduce-scatter: rows of the fused all-reduce, of the unfused GEMM -> reduce-scatter, and the
    sequence-parallel FFN through it, all bit-equal; gradients equal the unfused path's."""
    dist = _init(rank, world, port)
    from rl_kernel_b200.distributed.transports.symm import SymmetricMemoryCollective
    from rl_kernel_b200.ops.attention.projection import sp_row_parallel_linear
    from rl_kernel_b200.ops.ffn.qwen3 import qwen3_ffn

    dev = torch.device("cuda", rank)
    coll = SymmetricMemoryCollective(None, dev, frame_bytes=64 << 20)
    ok = True
    M, N, K, nchunks = 256 * world, 1024, 512 * (8 // world), 8 // world
    g = torch.Generator(device="cuda").manual_seed(100 + rank)          # every rank holds its own K shard
    a = torch.randn(M, K, device=dev, generator=g).bfloat16()
    w = (torch.randn(N, K, device=dev, generator=g) * 0.05).bfloat16()
    full = coll.gemm_all_reduce(a, w, torch.empty(M, N, device=dev, dtype=torch.bfloat16), nchunks)
    rows = slice(rank * M // world, (rank + 1) * M // world)
    for _ in range(3):                                                   # repeated calls walk both frames
        rs = coll.gemm_reduce_scatter(a, w, torch.empty(M // world, N, device=dev, dtype=torch.bfloat16), nchunks)
        ok &= torch.equal(rs, full[rows])
    # enough tiles for the 128 x 256 form of the fused kernel: still the unfused bits, row slice included
    from rl_kernel_b200.backends import native as nv

    Mw, Kw = 12288, 1536
    aw = torch.randn(Mw, Kw, device=dev, generator=g).bfloat16()
    ww = (torch.randn(N, Kw, device=dev, generator=g) * 0.05).bfloat16()
    part = torch.empty(Mw, N, device=dev, dtype=torch.bfloat16)
    nv.det_gemm(aw, ww, part, M=Mw, N=N, K=Kw, nchunks=2)
    unfused = coll.all_reduce(part)
    fullw = coll.gemm_all_reduce(aw, ww, torch.empty(Mw, N, device=dev, dtype=torch.bfloat16), 2)
    rsw = coll.gemm_reduce_scatter(aw, ww, torch.empty(Mw // world, N, device=dev, dtype=torch.bfloat16), 2)
    ok &= torch.equal(fullw, unfused) and torch.equal(rsw, unfused[rank * Mw // world:(rank + 1) * Mw // world])
    a1, w1 = a.clone().requires_grad_(True), w.clone().requires_grad_(True)
    a2, w2 = a.clone().requires_grad_(True), w.clone().requires_grad_(True)
    y1 = sp_row_parallel_linear(a1, w1, nchunks, coll, fused=True)
    y2 = sp_row_parallel_linear(a2, w2, nchunks, coll, fused=False)
    go = torch.randn(M // world, N, device=dev, generator=g).bfloat16()
    y1.backward(go)
    y2.backward(go)
    ok &= torch.equal(y1, y2) and torch.equal(y1, full[rows]) and torch.equal(a1.grad, a2.grad) and torch.equal(w1.grad, w2.grad)
    # the sequence-parallel FFN (fused exit) against the replicated-activation FFN
    H, I = 512, 2048
    g2 = torch.Generator(device="cuda").manual_seed(7)                   # same tensors on every rank
    x = torch.randn(M, H, device=dev, generator=g2).bfloat16()
    wgu = (torch.randn(2 * I, H, device=dev, generator=g2) * 0.05).bfloat16()
    wd = (torch.randn(H, I, device=dev, generator=g2) * 0.05).bfloat16()
    per = I // world
    blk = I // 8
    # gate/up rows are interleaved per canonical shard of I / 8 columns: [gate blk, up blk] x 8
    gu = wgu.view(8, 2, blk, H)[rank * (8 // world):(rank + 1) * (8 // world)].reshape(-1, H).contiguous()
    dn = wd[:, rank * per:(rank + 1) * per].contiguous()
    y_rep = qwen3_ffn(x, gu, dn, canonical_tp=8, tp_size=world, collective=coll)
    y_sp = qwen3_ffn(x[rows].contiguous(), gu, dn, canonical_tp=8, tp_size=world, collective=coll, sequence_parallel=True)
    ok &= torch.equal(y_sp, y_rep[rows])
    torch.cuda.synchronize(dev)
    from rl_kernel_b200.backends import extension as ext

    ok &= ext.poll_status(dev) == 0
    oks = [None] * world
    dist.all_gather_object(oks, bool(ok))
    if rank == 0:
        torch.save(all(oks), out)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", WORLDS)
def test_fused_gemm_reduce_scatter_equals_all_reduce_rows_bitwise(tmp_path, world):
    _need(world)
    out = str(tmp_path / "rs.pt")
    mp.spawn(_gemm_rs_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert torch.load(out)
